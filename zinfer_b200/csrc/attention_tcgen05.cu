// Paged causal flash attention for prompt portions on the 5th-generation tensor cores
// (head size 128, bfloat16): S = Q K^T and O += P V are tcgen05.mma products with S, P and O in
// tensor memory; Q, K and V tiles come by TMA (128-byte swizzle, every CTA loads its own tiles) straight from the
// activation buffer and the cache pages.  V is read as an MN-major operand (its rows are keys,
// the contraction dimension), K and Q as K-major, P from tensor memory.  The kernel and its warp
// roles are described at the kernel.  Every mbarrier wait is bounded; a timeout records a code
// in `status`, lets copies land, frees the tensor memory and returns.
#include <cuda.h>

#include "api.h"
#include "common.cuh"
#include "gemm_internal.h"
#include "tcgen05_ptx.cuh"

namespace {
using bf16 = __nv_bfloat16;

constexpr int BQ = 128, BK = 128, D = 128, THREADS = 320;
constexpr int HALF_BYTES = 128 * 128;          // 128 rows x 64 bf16: one swizzled half tile
constexpr int TILE_BYTES = 2 * HALF_BYTES;     // a [128, 128] bf16 tile as two halves of d (or of keys)

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// MN-major operand with 128-byte swizzle: 64 MN elements (128 bytes) per row, the next 64 MN
// elements `HALF_BYTES` further (leading byte offset); groups of 8 K rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr) {
  return (uint64_t)((addr & 0x3ffffu) >> 4) | ((uint64_t)(HALF_BYTES >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: D f32, A and B bf16, M = 128, N = n; b_mn: B is MN-major.
__device__ __forceinline__ uint32_t idesc_bf16(int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void tmem_store16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_store32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
        "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
        "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D += A * B with A in tensor memory (128 lanes = rows, two bfloat16 of K per 32-bit column).
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct Barriers {
  uint64_t q_full;
  uint64_t k_full[2], v_full[2], k_empty[2], v_empty[2];
  uint64_t s_full[2], p_full[2], pv_done[2];   // per query tile of the CTA
  uint32_t tmem_slot;
};

// A CTA takes TWO neighbouring tiles of 128 query tokens (a, b) of one request and one query
// head and walks the keys in tiles of 128 once for both: while the softmax warps of one tile
// work on their scores, the tensor core runs the other tile's products.
//   warp 0      TMA producer: both Q tiles once, then K and V tiles through a two-stage ring
//   warp 1      owns tensor memory and issues the MMAs, per key tile j and query tile x:
//               O_x += P_x[j] V[j] (P read from tensor memory), then S_x[j+1] = Q_x K[j+1]^T
//   warps 2..5  softmax of tile a, warps 6..9 of tile b: thread r owns query row r = its TMEM
//               lane.  It reads its row of S (tcgen05.ld), masks, exponentiates against a
//               reference maximum and writes P as bfloat16 over the first half of S's own
//               columns (tcgen05.st).  O stays in tensor memory for the whole walk: the
//               reference maximum only moves when the row's maximum outgrows it by 2^8, and
//               only then is O read, rescaled and written back (sum and output use the same
//               reference, so the result is exact).
// The kernel is launched over the list of 128-row tiles: the CTA of an even tile of a request
// takes the next one too, the CTA of an odd tile leaves at once.
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, int out_stride,
                            const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_q,
                            const int* __restrict__ kv_lens, const int* __restrict__ tile_seq,
                            const int* __restrict__ tile_q0, int nq, int nkv, int page_size, int window,
                            float scale_log2, int* __restrict__ status) {
  pdl_launch_dependents();
  const int seq = tile_seq[blockIdx.y], q0 = tile_q0[blockIdx.y];
  if ((q0 / BQ) & 1) return;   // the CTA of the tile before this one takes both
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;                       // [2 query tiles][2 halves of d][128 rows][128 B]
  uint8_t* k_s = q_s + 2 * TILE_BYTES;       // [2 stages][2 halves of d][128 keys][128 B]
  uint8_t* v_s = k_s + 2 * TILE_BYTES;       // [2 stages][2 halves of d][128 keys][128 B]
  Barriers* bar = reinterpret_cast<Barriers*>(v_s + 2 * TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, kvh = h / (nq / nkv);
  const int tok0 = cu_q[seq], qlen = cu_q[seq + 1] - tok0, kvlen = kv_lens[seq];
  const int ctx = kvlen - qlen;
  int nqv[2], first_pos[2], kv_lo[2], kv_hi[2], n_t[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    nqv[x] = max(0, min(BQ, qlen - (q0 + x * BQ)));
    first_pos[x] = ctx + q0 + x * BQ;
    kv_lo[x] = window > 0 ? max(0, first_pos[x] - window + 1) : 0;
    kv_hi[x] = first_pos[x] + nqv[x];
  }
  const int kt0 = (kv_lo[0] / BK) * BK;      // tile a starts lowest
#pragma unroll
  for (int x = 0; x < 2; ++x) n_t[x] = nqv[x] > 0 ? (kv_hi[x] - kt0 + BK - 1) / BK : 0;
  const int n_max = max(n_t[0], n_t[1]);
  const int lo_all = kv_lo[0], hi_all = max(kv_hi[0], kv_hi[1]);
  const int* bt = block_tables + (size_t)seq * bt_stride;
  bool failed = false;

  if (threadIdx.x == 0) {
    mbar_init(&bar->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->k_full[i], 1);
      mbar_init(&bar->v_full[i], 1);
      mbar_init(&bar->k_empty[i], 1);
      mbar_init(&bar->v_empty[i], 1);
      mbar_init(&bar->s_full[i], 1);
      mbar_init(&bar->p_full[i], 4);    // one arrival per softmax warp of the tile
      mbar_init(&bar->pv_done[i], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bar->tmem_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = bar->tmem_slot;
  const uint32_t tmem_s[2] = {tmem_base, tmem_base + 128u};          // scores, then P over their first 64 columns
  const uint32_t tmem_o[2] = {tmem_base + 256u, tmem_base + 384u};
  pdl_wait();   // q and the cache pages were written by the kernels before

  if (warp == 0) {
    if (n_max > 0) {
      if (lane == 0) {
        mbar_expect_tx(&bar->q_full, (uint32_t)(nqv[1] > 0 ? 2 * TILE_BYTES : TILE_BYTES));
        for (int x = 0; x < 2; ++x) {
          if (nqv[x] <= 0) continue;
          tma_load_2d(q_s + x * TILE_BYTES, &map_q, &bar->q_full, h * D, tok0 + q0 + x * BQ);
          tma_load_2d(q_s + x * TILE_BYTES + HALF_BYTES, &map_q, &bar->q_full, h * D + 64, tok0 + q0 + x * BQ);
        }
      }
      // A key tile is 4 boxes per page (K and V, two halves of d).  Issuing a tensor copy costs its
      // thread a few hundred nanoseconds, so the boxes of a tile are issued by the warp's lanes
      // side by side, not by one thread one after the other.
      const int box_bytes = page_size * 128;
      const int pages_per_tile = BK / page_size;
      for (int j = 0; j < n_max; ++j) {
        const int s = j & 1;
        const int kt = kt0 + j * BK;
        // A tile may reach past the request's last page, or start in pages a window has given
        // back.  Such boxes are filled from a page the request does hold: their keys are masked
        // and p = 0 meets finite values (shared memory is never left uninitialised).
        int fallback = -1;
        for (int p = 0; p < pages_per_tile && fallback < 0; ++p) {
          const int key = kt + p * page_size;
          if (key < hi_all && key + page_size > lo_all) fallback = __ldg(bt + key / page_size);
        }
        if (fallback < 0) fallback = 0;
        // K's slot is free as soon as the scores of the tile two before have been computed, a whole
        // iteration before V's: K[j] is requested early enough to be there when S[j] is issued
        for (int which_kv = 0; which_kv < 2; ++which_kv) {
          int ok = 1;
          if (lane == 0) {
            uint64_t* empty = which_kv ? &bar->v_empty[s] : &bar->k_empty[s];
            ok = mbar_wait(empty, ((uint32_t)(j >> 1) & 1u) ^ 1u) ? 1 : 0;
            if (ok) mbar_expect_tx(which_kv ? &bar->v_full[s] : &bar->k_full[s], (uint32_t)TILE_BYTES);
            else atomicExch(status, 11);
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) { failed = true; break; }
          for (int b = lane; b < 2 * pages_per_tile; b += 32) {
            const int p = b >> 1, half = b & 1;
            const int key = kt + p * page_size;
            int page = (key < hi_all && key + page_size > lo_all) ? __ldg(bt + key / page_size) : -1;
            if (page < 0) page = fallback;
            const int row = (page * nkv + kvh) * page_size;
            uint8_t* dst = (which_kv ? v_s : k_s) + s * TILE_BYTES + p * box_bytes + half * HALF_BYTES;
            tma_load_2d(dst, which_kv ? &map_v : &map_k, which_kv ? &bar->v_full[s] : &bar->k_full[s], half * 64, row);
          }
          __syncwarp();
        }
        if (failed) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_max > 0) {
      const uint32_t idesc_s = idesc_bf16(BK, false), idesc_o = idesc_bf16(D, true);
      // S_x[j] = Q_x K[j]^T (K[j] must have arrived: the caller has waited for it)
      auto issue_qk = [&](int x, int j) {
        const uint32_t q_addr = smem_u32(q_s + x * TILE_BYTES), k_addr = smem_u32(k_s + (j & 1) * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (uint32_t)((kk >> 2) * HALF_BYTES + (kk & 3) * 32);
          tcgen05_mma_bf16(tmem_s[x], smem_desc_sw128(q_addr + off), smem_desc_sw128(k_addr + off), idesc_s, kk > 0 ? 1u : 0u);
        }
        tcgen05_commit(&bar->s_full[x]);
      };
      if (!mbar_wait(&bar->q_full, 0)) { failed = true; atomicExch(status, 14); }
      if (!failed && !mbar_wait(&bar->k_full[0], 0)) { failed = true; atomicExch(status, 12); }
      if (!failed) {
        tcgen05_fence_after();
        for (int x = 0; x < 2; ++x)
          if (n_t[x] > 0) issue_qk(x, 0);
        tcgen05_commit(&bar->k_empty[0]);   // K[0] is free when these products have read it
      }
      for (int j = 0; j < n_max && !failed; ++j) {
        const int s = j & 1;
        bool have_v = false, have_k = false;
        for (int x = 0; x < 2 && !failed; ++x) {
          if (j >= n_t[x]) continue;
          if (!mbar_wait(&bar->p_full[x], (uint32_t)j & 1u)) { failed = true; atomicExch(status, 15); break; }
          if (!have_v) {
            if (!mbar_wait(&bar->v_full[s], (uint32_t)(j >> 1) & 1u)) { failed = true; atomicExch(status, 16); break; }
            have_v = true;
          }
          tcgen05_fence_after();
          const uint32_t v_addr = smem_u32(v_s + s * TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // P: keys kk*16.. = 8 columns of packed pairs; V: key rows kk*16.. of the MN-major V tile
            umma_bf16_ts(tmem_o[x], tmem_s[x] + (uint32_t)kk * 8u, desc_mnmajor(v_addr + (uint32_t)kk * 16u * 128u), idesc_o,
                         (j > 0 || kk > 0) ? 1u : 0u);
          }
          tcgen05_commit(&bar->pv_done[x]);
          if (j + 1 < n_t[x]) {   // the next scores of this tile run under the other tile's softmax
            if (!have_k) {
              if (!mbar_wait(&bar->k_full[(j + 1) & 1], (uint32_t)((j + 1) >> 1) & 1u)) { failed = true; atomicExch(status, 12); break; }
              have_k = true;
              tcgen05_fence_after();
            }
            issue_qk(x, j + 1);
          }
        }
        if (!failed) {
          tcgen05_commit(&bar->v_empty[s]);                 // V[j] has been read by this iteration's products
          tcgen05_commit(&bar->k_empty[(j + 1) & 1]);       // and K[j+1] by the scores issued in it
        }
      }
    }
  } else {
    const int x = (warp - 2) >> 2;               // which query tile
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;           // this thread's query row = its TMEM lane
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    // this tile's numbers in registers (the arrays are indexed by x, which only this branch knows)
    const int nt = x ? n_t[1] : n_t[0];
    const int my_first = x ? first_pos[1] : first_pos[0];
    const int my_lo = x ? kv_lo[1] : kv_lo[0];
    const int pos = my_first + r;
    const int row_lo = window > 0 ? max(my_lo, pos - window + 1) : my_lo;   // keys row_lo .. pos are visible
    const uint32_t s_addr = (x ? tmem_s[1] : tmem_s[0]) + lane_off, o_addr = (x ? tmem_o[1] : tmem_o[0]) + lane_off;
    uint64_t* s_full = &bar->s_full[x];
    uint64_t* p_full = &bar->p_full[x];
    uint64_t* pv_done = &bar->pv_done[x];
    float m_ref = -INFINITY, l = 0.f;
    for (int j = 0; j < nt && !failed; ++j) {
      const int kt = kt0 + j * BK;
      if (!mbar_wait(s_full, (uint32_t)j & 1u)) { failed = true; atomicExch(status, 18); break; }
      tcgen05_fence_after();
      // Columns c_lo .. c_hi - 1 of this tile are visible to this row; only tiles on the diagonal,
      // at a window's edge or below the first visible key need the test at all (a warp-uniform
      // choice between two loops, so that the common tile pays nothing for the mask).
      const bool need_mask = kt + BK - 1 > my_first || window > 0 || kt < my_lo;
      const int c_hi = min(BK, pos - kt + 1), c_lo = max(0, row_lo - kt);
      // pass 1: the row's maximum over the visible keys
      float mx = -INFINITY;
      if (need_mask) {
#pragma unroll 1
        for (int c0 = 0; c0 < BK; c0 += 32) {
          float v[32];
          tmem_load32(s_addr + (uint32_t)c0, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, (c0 + i >= c_lo && c0 + i < c_hi) ? v[i] : -INFINITY);
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BK; c0 += 32) {
          float v[32];
          tmem_load32(s_addr + (uint32_t)c0, v);
          float m4[4] = {v[0], v[1], v[2], v[3]};
#pragma unroll
          for (int i = 4; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], v[i]);
          mx = fmaxf(mx, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
        }
      }
      // The reference maximum moves only when the row's maximum has outgrown it by 2^8
      // (p stays below 256); then the sum and the output in tensor memory are rescaled.
      const float cand = mx * scale_log2;
      const bool need = cand > m_ref + 8.0f;
      if (__any_sync(0xffffffffu, need)) {
        float f = 1.0f;
        if (need) {
          f = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - cand);
          m_ref = cand;
        }
        l *= f;
        if (j > 0) {
          if (!mbar_wait(pv_done, ((uint32_t)j & 1u) ^ 1u)) { failed = true; atomicExch(status, 20); break; }
          tcgen05_fence_after();
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            float v[32];
            tmem_load32(o_addr + (uint32_t)c0, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= f;
            tmem_store32(o_addr + (uint32_t)c0, v);
          }
        }
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      // pass 2: p = exp2(s * scale - reference), the row sum, P as bfloat16 pairs over S's first columns
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
      for (int c0 = 0; c0 < BK; c0 += 32) {
        float v[32];
        tmem_load32(s_addr + (uint32_t)c0, v);
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = fast_exp2(fmaf(v[i], scale_log2, -m_use));
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = (c0 + i >= c_lo && c0 + i < c_hi) ? v[i] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) sum4[i & 3] += v[i];
#pragma unroll
        for (int i = 0; i < 16; ++i) packed[i] = pack2(v[2 * i], v[2 * i + 1]);
        tmem_store16(s_addr + (uint32_t)(c0 >> 1), packed);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tmem_wait_st();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (!failed && nt > 0) {
      if (!mbar_wait(pv_done, (uint32_t)(nt - 1) & 1u)) { failed = true; atomicExch(status, 21); }
      tcgen05_fence_after();
      if (!failed) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        bf16* orow = out + (size_t)(tok0 + q0 + x * BQ + r) * out_stride + (size_t)h * D;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          float v[32];
          tmem_load32(o_addr + (uint32_t)c0, v);
          if (r < (x ? nqv[1] : nqv[0])) {
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
              uint4 w;
              w.x = pack2(v[c] * inv, v[c + 1] * inv);
              w.y = pack2(v[c + 2] * inv, v[c + 3] * inv);
              w.z = pack2(v[c + 4] * inv, v[c + 5] * inv);
              w.w = pack2(v[c + 6] * inv, v[c + 7] * inv);
              *reinterpret_cast<uint4*>(orow + c0 + c) = w;
            }
          }
        }
      }
    }
  }
  if (failed) {
    for (int i = 0; i < 64; ++i) __nanosleep(10000);   // copies in flight land before shared memory is given up
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace

// Whether the tcgen05 prefill kernel takes this shape: head size 128, pages of 8..128 tokens
// that divide 128, q rows and cache pages aligned for TMA.
extern "C" int zi_attention_prefill_tcgen05_supported(int nq, int nkv, int d, int page_size, const void* q,
                                                      int q_stride, const void* kcache, const void* vcache) {
  if (d != 128 || nkv <= 0 || nq % nkv) return 0;
  if (page_size < 8 || page_size > 128 || 128 % page_size || page_size % 8) return 0;
  if (((uintptr_t)q % 16) || (q_stride % 8) || ((uintptr_t)kcache % 16) || ((uintptr_t)vcache % 16)) return 0;
  return 1;
}

extern "C" int zi_attention_prefill_tcgen05(void* out, int out_stride, const void* q, int q_stride, int n_tokens,
                                            const void* kcache, const void* vcache, long long n_pages,
                                            const int* block_tables, int bt_stride, const int* cu_q,
                                            const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles,
                                            int nq, int nkv, int d, int page_size, int window, float scale,
                                            cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!zi_attention_prefill_tcgen05_supported(nq, nkv, d, page_size, q, q_stride, kcache, vcache))
    return zi_refuse("attention_prefill_tcgen05: needs head_dim 128, pages of 8..128 tokens dividing 128, aligned q and pages");
  CUtensorMap map_q, map_k, map_v;
  const long long cache_rows = n_pages * nkv * page_size;
  if (cache_rows > 0x7fffffffll) return zi_refuse("attention_prefill_tcgen05: the cache has too many rows for a tensor map");
  if (!zi_internal_make_map(&map_q, q, n_tokens, nq * d, q_stride, BQ) ||
      !zi_internal_make_map(&map_k, kcache, (int)cache_rows, d, d, page_size) ||
      !zi_internal_make_map(&map_v, vcache, (int)cache_rows, d, d, page_size))
    return zi_refuse("attention_prefill_tcgen05: cuTensorMapEncodeTiled failed");
  int* status = zi_internal_status_word();
  if (!status) return zi_refuse("attention_prefill_tcgen05: cannot allocate the status word");
  const size_t smem = 1024 + (size_t)6 * TILE_BYTES + sizeof(Barriers) + 64;
  auto kern = attn_prefill_tcgen05_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return zi_refuse("attention_prefill_tcgen05: cannot get %zu bytes of shared memory", smem);
  zi_launch(kern, dim3(nq, n_tiles), dim3(THREADS), smem, stream, map_q, map_k, map_v, (bf16*)out, out_stride,
            block_tables, bt_stride, cu_q, kv_lens, tile_seq, tile_q0, nq, nkv, page_size, window,
            scale * 1.4426950408889634f, status);
  return zi_check_launch("attention_prefill_tcgen05");
}

ZI_TRACE_SETTER(attention_tcgen05)
