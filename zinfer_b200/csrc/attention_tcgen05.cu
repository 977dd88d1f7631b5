// Paged causal flash attention for prompt portions on the 5th-generation tensor cores
// (head size 128, bfloat16): S = Q K^T and O_tile = P V are tcgen05.mma products with
// their accumulators in tensor memory; Q, K and V tiles come by TMA (128-byte swizzle,
// no multicast) straight from the activation buffer and the cache pages.
//
// A CTA takes 128 query tokens of one request and one query head and walks the keys in
// tiles of 128.  Warp roles (192 threads):
//   warp 0      TMA producer: Q once, then K and V tiles (one box per page and half of d)
//               through a two-stage ring;
//   warp 1      owns tensor memory and issues the MMAs: S[j+1] = Q K[j+1]^T is issued
//               before O_tile[j] = P[j] V[j], so it runs under the softmax of tile j;
//   warps 2..5  softmax: thread r owns query row r.  It reads its row of S from tensor
//               memory (tcgen05.ld), masks, keeps the running maximum and sum in 32-bit,
//               writes P as bfloat16 into shared memory in the swizzled K-major layout the
//               next MMA reads, then adds O_tile (read back from tensor memory) into its
//               32-bit output row: O = O * alpha + O_tile.
// V is read as an MN-major operand (its rows are keys, the contraction dimension), K and
// Q as K-major.  Every mbarrier wait is bounded; a timeout records a code in `status`,
// lets copies land, frees the tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "api.h"
#include "common.cuh"

namespace {
using bf16 = __nv_bfloat16;

constexpr int BQ = 128, BK = 128, D = 128, THREADS = 192;
constexpr int HALF_BYTES = 128 * 128;          // 128 rows x 64 bf16: one swizzled half tile
constexpr int TILE_BYTES = 2 * HALF_BYTES;     // a [128, 128] bf16 tile as two halves of d (or of keys)
constexpr uint32_t WAIT_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_load32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// K-major operand with 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
  return (uint64_t)((addr & 0x3ffffu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
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

struct Barriers {
  uint64_t q_full;
  uint64_t k_full[2], v_full[2], kv_empty[2];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, p_empty;
  uint64_t o_full, o_empty;
  uint32_t tmem_slot;
};

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, int out_stride,
                            const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_q,
                            const int* __restrict__ kv_lens, const int* __restrict__ tile_seq,
                            const int* __restrict__ tile_q0, int nq, int nkv, int page_size, int window,
                            float scale_log2, int* __restrict__ status) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem;                       // [2 halves of d][128 rows][128 B]
  uint8_t* k_s = q_s + TILE_BYTES;           // [2 stages][2 halves of d][128 keys][128 B]
  uint8_t* v_s = k_s + 2 * TILE_BYTES;       // [2 stages][2 halves of d][128 keys][128 B]
  uint8_t* p_s = v_s + 2 * TILE_BYTES;       // [2 halves of keys][128 rows][128 B]
  Barriers* bar = reinterpret_cast<Barriers*>(p_s + TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = tile_seq[blockIdx.y], q0 = tile_q0[blockIdx.y];
  const int h = blockIdx.x, kvh = h / (nq / nkv);
  const int tok0 = cu_q[seq], qlen = cu_q[seq + 1] - tok0, kvlen = kv_lens[seq];
  const int ctx = kvlen - qlen;
  const int nqv = min(BQ, qlen - q0);
  const int first_pos = ctx + q0, last_pos = first_pos + nqv - 1;
  const int kv_lo = window > 0 ? max(0, first_pos - window + 1) : 0;
  const int kv_hi = last_pos + 1;
  const int kt0 = (kv_lo / BK) * BK;
  const int n_tiles = nqv > 0 ? (kv_hi - kt0 + BK - 1) / BK : 0;
  const int* bt = block_tables + (size_t)seq * bt_stride;
  bool failed = false;

  if (threadIdx.x == 0) {
    mbar_init(&bar->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar->k_full[i], 1);
      mbar_init(&bar->v_full[i], 1);
      mbar_init(&bar->kv_empty[i], 1);
      mbar_init(&bar->s_full[i], 1);
      mbar_init(&bar->s_empty[i], 4);
    }
    mbar_init(&bar->p_full, 4);
    mbar_init(&bar->p_empty, 1);
    mbar_init(&bar->o_full, 1);
    mbar_init(&bar->o_empty, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bar->tmem_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = bar->tmem_slot;
  const uint32_t tmem_s[2] = {tmem_base, tmem_base + 128u};
  const uint32_t tmem_o = tmem_base + 256u;
  pdl_wait();   // q and the cache pages were written by the kernels before

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(&bar->q_full, TILE_BYTES);
      tma_load_2d(q_s, &map_q, &bar->q_full, h * D, tok0 + q0);
      tma_load_2d(q_s + HALF_BYTES, &map_q, &bar->q_full, h * D + 64, tok0 + q0);
      const int box_bytes = page_size * 128;
      const int pages_per_tile = BK / page_size;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&bar->kv_empty[s], ((uint32_t)(j >> 1) & 1u) ^ 1u)) { failed = true; atomicExch(status, 11); break; }
        const int kt = kt0 + j * BK;
        // A tile may reach past the request's last page, or start in pages a window has given
        // back.  Such boxes are filled from a page the request does hold: their keys are masked
        // and p = 0 meets finite values (shared memory is never left uninitialised).
        int fallback = -1;
        for (int p = 0; p < pages_per_tile && fallback < 0; ++p) {
          const int key = kt + p * page_size;
          if (key < kv_hi && key + page_size > kv_lo) fallback = __ldg(bt + key / page_size);
        }
        if (fallback < 0) fallback = 0;
        mbar_expect_tx(&bar->k_full[s], (uint32_t)TILE_BYTES);
        mbar_expect_tx(&bar->v_full[s], (uint32_t)TILE_BYTES);
        for (int p = 0; p < pages_per_tile; ++p) {
          const int key = kt + p * page_size;
          int page = (key < kv_hi && key + page_size > kv_lo) ? __ldg(bt + key / page_size) : -1;
          if (page < 0) page = fallback;
          const int row = (page * nkv + kvh) * page_size;
          uint8_t* kd = k_s + s * TILE_BYTES + p * box_bytes;
          uint8_t* vd = v_s + s * TILE_BYTES + p * box_bytes;
          tma_load_2d(kd, &map_k, &bar->k_full[s], 0, row);
          tma_load_2d(kd + HALF_BYTES, &map_k, &bar->k_full[s], 64, row);
          tma_load_2d(vd, &map_v, &bar->v_full[s], 0, row);
          tma_load_2d(vd + HALF_BYTES, &map_v, &bar->v_full[s], 64, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      const uint32_t idesc_s = idesc_bf16(BK, false), idesc_o = idesc_bf16(D, true);
      const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (!mbar_wait(&bar->k_full[s], ph)) { atomicExch(status, 12); return false; }
        if (!mbar_wait(&bar->s_empty[s], ph ^ 1u)) { atomicExch(status, 13); return false; }
        fence_after();
        const uint32_t k_addr = smem_u32(k_s + s * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (uint32_t)((kk >> 2) * HALF_BYTES + (kk & 3) * 32);
          umma_bf16(tmem_s[s], desc_kmajor(q_addr + off), desc_kmajor(k_addr + off), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bar->s_full[s]);
        return true;
      };
      if (!mbar_wait(&bar->q_full, 0)) { failed = true; atomicExch(status, 14); }
      if (!failed && !issue_qk(0)) failed = true;
      for (int j = 0; j < n_tiles && !failed; ++j) {
        if (j + 1 < n_tiles && !issue_qk(j + 1)) { failed = true; break; }
        const int s = j & 1;
        if (!mbar_wait(&bar->p_full, (uint32_t)j & 1u)) { failed = true; atomicExch(status, 15); break; }
        if (!mbar_wait(&bar->v_full[s], (uint32_t)(j >> 1) & 1u)) { failed = true; atomicExch(status, 16); break; }
        if (!mbar_wait(&bar->o_empty, ((uint32_t)j & 1u) ^ 1u)) { failed = true; atomicExch(status, 17); break; }
        fence_after();
        const uint32_t v_addr = smem_u32(v_s + s * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          // P: keys kk*16.. of the K-major P tile; V: key rows kk*16.. of the MN-major V tile
          const uint32_t p_off = (uint32_t)((kk >> 2) * HALF_BYTES + (kk & 3) * 32);
          umma_bf16(tmem_o, desc_kmajor(p_addr + p_off), desc_mnmajor(v_addr + (uint32_t)kk * 16u * 128u), idesc_o,
                    kk > 0 ? 1u : 0u);
        }
        umma_commit(&bar->o_full);
        umma_commit(&bar->p_empty);
        umma_commit(&bar->kv_empty[s]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;           // this thread's query row = its TMEM lane
    const int pos = first_pos + r;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    float o_acc[D];
#pragma unroll
    for (int c = 0; c < D; ++c) o_acc[c] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int j = 0; j < n_tiles && !failed; ++j) {
      const int s = j & 1;
      const int kt = kt0 + j * BK;
      if (!mbar_wait(&bar->s_full[s], (uint32_t)(j >> 1) & 1u)) { failed = true; atomicExch(status, 18); break; }
      fence_after();
      const bool need_mask = kt + BK - 1 > first_pos || window > 0 || kt < kv_lo;
      // pass 1: the row's maximum over the visible keys
      float mx = -INFINITY;
#pragma unroll
      for (int c0 = 0; c0 < BK; c0 += 32) {
        float v[32];
        tmem_load32(tmem_s[s] + lane_off + (uint32_t)c0, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = v[i];
          if (need_mask) {
            const int key = kt + c0 + i;
            if (key > pos || key < kv_lo || (window > 0 && key <= pos - window)) x = -INFINITY;
          }
          mx = fmaxf(mx, x);
        }
      }
      const float m_new = fmaxf(m, mx * scale_log2);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = fast_exp2(m - m_use);
      // P of the tile before must have been read by its MMA before it is overwritten
      if (!mbar_wait(&bar->p_empty, ((uint32_t)j & 1u) ^ 1u)) { failed = true; atomicExch(status, 19); break; }
      // pass 2: p = exp2(s * scale - max), the row sum, P to shared memory as bfloat16
      float sum = 0.f;
#pragma unroll
      for (int c0 = 0; c0 < BK; c0 += 32) {
        float v[32];
        tmem_load32(tmem_s[s] + lane_off + (uint32_t)c0, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float p = fast_exp2(fmaf(v[i], scale_log2, -m_use));
          if (need_mask) {
            const int key = kt + c0 + i;
            if (key > pos || key < kv_lo || (window > 0 && key <= pos - window)) p = 0.f;
          }
          v[i] = p;
          sum += p;
        }
        uint8_t* prow = p_s + (c0 >> 6) * HALF_BYTES + r * 128;
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          const int chunk = ((c0 & 63) + i) >> 3;
          uint4 w;
          w.x = pack2(v[i], v[i + 1]);
          w.y = pack2(v[i + 2], v[i + 3]);
          w.z = pack2(v[i + 4], v[i + 5]);
          w.w = pack2(v[i + 6], v[i + 7]);
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = w;
        }
      }
      l = l * alpha + sum;
      m = m_new;
      // S[s] has been read; P is written: make it visible to the tensor core's reads
      fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bar->s_empty[s]);
        mbar_arrive(&bar->p_full);
      }
      // O = O * alpha + P V
      if (!mbar_wait(&bar->o_full, (uint32_t)j & 1u)) { failed = true; atomicExch(status, 20); break; }
      fence_after();
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        float v[32];
        tmem_load32(tmem_o + lane_off + (uint32_t)c0, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) o_acc[c0 + i] = fmaf(o_acc[c0 + i], alpha, v[i]);
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->o_empty);
    }
    if (!failed && r < nqv) {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      bf16* orow = out + (size_t)(tok0 + q0 + r) * out_stride + (size_t)h * D;
#pragma unroll
      for (int c = 0; c < D; c += 8) {
        uint4 w;
        w.x = pack2(o_acc[c] * inv, o_acc[c + 1] * inv);
        w.y = pack2(o_acc[c + 2] * inv, o_acc[c + 3] * inv);
        w.z = pack2(o_acc[c + 4] * inv, o_acc[c + 5] * inv);
        w.w = pack2(o_acc[c + 6] * inv, o_acc[c + 7] * inv);
        *reinterpret_cast<uint4*>(orow + c) = w;
      }
    }
  }
  if (failed) {
    for (int i = 0; i < 64; ++i) __nanosleep(10000);   // copies in flight land before shared memory is given up
  }
  fence_before();
  __syncthreads();
  if (warp == 1) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// A 2-D map over row-major bf16 [rows, cols] with row pitch `ld` elements, box [box_rows, 64].
bool make_map(CUtensorMap* map, const void* ptr, long long rows, int cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int* status_word() {
  static int* word = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    if (cudaMalloc(&word, sizeof(int)) == cudaSuccess) cudaMemset(word, 0, sizeof(int));
  });
  return word;
}
}  // namespace

// Whether the tcgen05 prefill kernel takes this shape: head size 128, pages of 8..128 tokens
// that divide 128, q rows and cache pages aligned for TMA.
extern "C" int zi_attention_prefill_tcgen05_supported(int nq, int nkv, int d, int page_size, const void* q,
                                                      int q_stride, const void* kcache, const void* vcache) {
  if (d != 128 || nkv <= 0 || nq % nkv) return 0;
  if (page_size < 8 || page_size > 128 || 128 % page_size || page_size % 8) return 0;
  if (((uintptr_t)q % 16) || (q_stride % 8) || ((uintptr_t)kcache % 16) || ((uintptr_t)vcache % 16)) return 0;
  return encode_fn() != nullptr;
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
  if (!make_map(&map_q, q, n_tokens, nq * d, q_stride, BQ) || !make_map(&map_k, kcache, cache_rows, d, d, page_size) ||
      !make_map(&map_v, vcache, cache_rows, d, d, page_size))
    return zi_refuse("attention_prefill_tcgen05: cuTensorMapEncodeTiled failed");
  int* status = status_word();
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

extern "C" int zi_attention_tcgen05_status() {
  int* status = status_word();
  if (!status) return -1;
  int host = 0;
  if (cudaMemcpy(&host, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (host != 0) cudaMemset(status, 0, sizeof(int));
  return host;
}
