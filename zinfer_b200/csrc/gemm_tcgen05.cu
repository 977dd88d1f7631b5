// out[M,N] = x[M,K] * w[N,K]^T in bfloat16 on the 5th-generation tensor cores:
// TMA (cp.async.bulk.tensor, 128-byte swizzle, every CTA loads its own tiles) fills a ring of shared
// memory stages, one elected thread issues tcgen05.mma with the accumulator in
// tensor memory, and four warps read it back with tcgen05.ld for the epilogue.
//
// Both operands are K-major, which is how activations [tokens, K] and weights
// [out, K] already lie in memory.  The 128 lanes of the accumulator take rows of
// the "A side", its columns rows of the "B side":
//   * many tokens (prefill): A side = tokens, B side = weight rows;
//   * up to 128 tokens (decode, short portions): A side = weight rows, B side = tokens padded to 16..128,
//     so a CTA streams a [128, K] slab of the weight at the rate TMA can bring it
//     and no tensor-core work is wasted on padding rows.
// Split-K over gridDim.z writes 32-bit partial sums to a workspace; a second kernel
// adds them in a fixed order.
//
// Warp roles (192 threads): warp 0 = TMA producer (a few of its lanes issue side by side), warp 1 = TMEM owner and MMA
// issuer, warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w%4)..+31).
// Every wait on an mbarrier is bounded; when it runs out the kernel records a code
// in `status`, lets copies in flight land, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "api.h"
#include "common.cuh"
#include "gemm_internal.h"
#include "gemm_static_scratch.h"
#include "tcgen05_ptx.cuh"

namespace {

constexpr int TILE_A = 128;        // accumulator lanes
constexpr int BLOCK_K = 64;        // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = TILE_A * BLOCK_K * 2;
constexpr int THREADS = 192;

// -------------------------------------------------------------------- the kernel
struct GemmArgs {
  int a_rows, b_rows;        // rows of the A side (accumulator lanes) and of the B side (columns)
  int a_tiles, b_tiles, splits;
  int k_blocks, k_blocks_per_split;
  long long sa, sb;          // element (a, b) goes to out[a * sa + b * sb]
  long long pa, pb;          // or, split, as a float to partial[z * a_rows * b_rows + a * pa + b * pb]
  int BN, stages, acc_cols;  // acc_cols: TMEM columns of one accumulator (two are allocated)
  int a_is_weight;           // which side does not depend on the kernel before this one
  // SwiGLU epilogue (tokens on the lanes): the weight's rows are interleaved in blocks of 64
  // (64 gate rows, then the 64 up rows of the same features); the kernel writes
  // silu(gate) * up, half as many columns, with this row pitch.
  long long act_ld;
  // Argmax epilogue (weight rows on the lanes, one token per column): beside the 32-bit results,
  // every warp leaves the first maximum of its 32 weight rows for each token as
  // cand_val/cand_idx[token * cand_units + a / 32]; a second, small kernel picks among them.
  float* cand_val;
  int* cand_idx;
  int cand_units;
  int weights_once;          // few tokens: the weight tiles are loaded with the L2 policy "evict first"
};

constexpr int EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_ARGMAX = 2;

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// One thread's row of an accumulator (TMEM lane `lane_base`, BN columns) to memory: row `a` of the A
// side against B rows b_tile * BN ...  `a_ok` is false for rows past the end (the thread still
// takes part in the warp-wide tensor-memory loads).
template <typename TO, int EPI>
__device__ __forceinline__ void drain_accumulator(const GemmArgs& g, TO* __restrict__ out, float* __restrict__ partial,
                                                  int split, int a, bool a_ok, int b_tile, uint32_t lane_base) {
  const int BN = g.BN;
  constexpr bool SWIGLU = EPI == EPI_SWIGLU;
  if (SWIGLU) {
    // Tokens on the lanes; of every 128 columns the first 64 are gate and the next 64 up.
    for (int c0 = 0; c0 < BN; c0 += 128) {
#pragma unroll
      for (int h = 0; h < 64; h += 32) {
        float gv[32], uv[32];
        tmem_load32(lane_base + (uint32_t)(c0 + h), gv);
        tmem_load32(lane_base + (uint32_t)(c0 + 64 + h), uv);
        const int f0 = (b_tile * BN + c0) / 2 + h;                 // first output feature of this chunk
        if (!a_ok) continue;
        TO* o = out + (long long)a * g.act_ld + f0;
        if (f0 + 32 <= g.b_rows / 2 && ((uintptr_t)o & 15) == 0 && sizeof(TO) == 2) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 w;
            w.x = pack2(silu_mul(gv[j], uv[j]), silu_mul(gv[j + 1], uv[j + 1]));
            w.y = pack2(silu_mul(gv[j + 2], uv[j + 2]), silu_mul(gv[j + 3], uv[j + 3]));
            w.z = pack2(silu_mul(gv[j + 4], uv[j + 4]), silu_mul(gv[j + 5], uv[j + 5]));
            w.w = pack2(silu_mul(gv[j + 6], uv[j + 6]), silu_mul(gv[j + 7], uv[j + 7]));
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(o) + j) = w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (f0 + j < g.b_rows / 2) o[j] = from_f32<TO>(silu_mul(gv[j], uv[j]));
        }
      }
    }
  } else
  for (int c0 = 0; c0 < BN; c0 += 32) {
    float v[32];
    if (BN - c0 >= 32) {
      tmem_load32(lane_base + (uint32_t)c0, v);
    } else {  // BN == 16
      float v16[16];
      tmem_load16(lane_base + (uint32_t)c0, v16);
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = j < 16 ? v16[j] : 0.f;
    }
    const int ncol = min(32, BN - c0);
    const int b0 = b_tile * BN + c0;
    if (EPI == EPI_ARGMAX) {
      // Floats as unsigned keys in the same order (NaN counts as -inf, -0 as +0; rows past the end
      // get key 0, below every number): one warp-wide maximum and one vote per token, and the
      // first lane that holds the maximum, the lowest weight row, writes it.
      const int lane = threadIdx.x & 31;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j >= ncol || b0 + j >= g.b_rows) break;
        float x = v[j];
        if (x != x) x = -INFINITY;
        if (x == 0.f) x = 0.f;
        const uint32_t bits = __float_as_uint(x);
        const uint32_t key = a_ok ? ((bits >> 31) ? ~bits : (bits | 0x80000000u)) : 0u;
        const uint32_t top = __reduce_max_sync(0xffffffffu, key);
        const int who = __ffs(__ballot_sync(0xffffffffu, key == top)) - 1;
        if (lane == who) {
          const long long at = (long long)(b0 + j) * g.cand_units + (a >> 5);
          g.cand_val[at] = top ? x : -INFINITY;
          g.cand_idx[at] = top ? a : 0x7fffffff;
        }
      }
    }
    if (!a_ok) continue;
    if (partial) {
      float* p = partial + (size_t)split * g.a_rows * g.b_rows + (long long)a * g.pa + (long long)b0 * g.pb;
      if (g.pb == 1 && b0 + ncol <= g.b_rows && ((uintptr_t)p & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          if (j < ncol) *reinterpret_cast<float4*>(p + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncol && b0 + j < g.b_rows) p[(long long)j * g.pb] = v[j];
      }
    } else {
      TO* o = out + (long long)a * g.sa + (long long)b0 * g.sb;
      if (g.sb == 1 && b0 + ncol <= g.b_rows && ((uintptr_t)o & 15) == 0) {
        if (sizeof(TO) == 2) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (j >= ncol) break;
            uint4 w;
            w.x = pack2(v[j], v[j + 1]);
            w.y = pack2(v[j + 2], v[j + 3]);
            w.z = pack2(v[j + 4], v[j + 5]);
            w.w = pack2(v[j + 6], v[j + 7]);
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(o) + j) = w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            if (j < ncol)
              *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncol && b0 + j < g.b_rows) o[(long long)j * g.sb] = from_f32<TO>(v[j]);
      }
    }
  }
}

// A side: a_rows x K through map_a (box 64 x 128).  B side: b_rows x K through map_b
// (box 64 x BN).  Persistent: a CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...
// (A tile fastest, so neighbouring CTAs share the B tile in L2).  Two accumulators in
// tensor memory let the epilogue of one tile run under the MMAs of the next.
// EPI_SWIGLU: the epilogue writes silu(gate) * up (tokens on the lanes only).  EPI_ARGMAX: it also
// leaves each token's largest result per 32 weight rows (weight rows on the lanes only).
template <typename TO, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    TO* __restrict__ out, float* __restrict__ partial, const GemmArgs g, int* __restrict__ status) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int BN = g.BN, stages = g.stages;
  const int stage_bytes = A_TILE_BYTES + BN * BLOCK_K * 2;
  uint64_t* full = (uint64_t*)(smem + (size_t)stages * stage_bytes);
  uint64_t* empty = full + stages;
  uint64_t* accum_full = empty + stages;       // [2]
  uint64_t* accum_empty = accum_full + 2;      // [2]
  uint32_t* tmem_slot = (uint32_t*)(accum_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_per_split = g.a_tiles * g.b_tiles;
  const int total_tiles = tiles_per_split * g.splits;
  const uint32_t tmem_cols = 2u * (uint32_t)g.acc_cols;
  bool failed = false;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&accum_full[i], 1);
      mbar_init(&accum_empty[i], 4);   // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (a_tile, b_tile, first k-block, number of k-blocks)
  auto decode = [&](int tile, int& a_tile, int& b_tile, int& split, int& kb0, int& n_kb) {
    split = tile / tiles_per_split;
    const int rem = tile - split * tiles_per_split;
    b_tile = rem / g.a_tiles;
    a_tile = rem - b_tile * g.a_tiles;
    kb0 = split * g.k_blocks_per_split;
    n_kb = min(g.k_blocks, kb0 + g.k_blocks_per_split) - kb0;
  };

  if (warp == 0) {
    // Issuing a tensor copy holds its thread a few hundred nanoseconds while HBM is busy; copies
    // issued by several lanes in ONE instruction go out side by side.  So the first tile's
    // prefetch is one instruction over `pre` lanes (twice: weights before the wait for the kernel
    // before this one, activations after it), and in the loop lane 0 issues the weight's tile and
    // lane 1 the activations' in the same instruction.
    if ((int)blockIdx.x < total_tiles) {
      int a_tile, b_tile, split, kb0, n_kb;
      decode(blockIdx.x, a_tile, b_tile, split, kb0, n_kb);
      const int pre = min(stages, n_kb);
      // which: 1 = the weight's tile of k-block i into stage s, 0 = the activations'
      const uint64_t once = l2_policy_evict_first();
      auto issue = [&](int which, int s, int i) {
        uint8_t* dst = smem + (size_t)s * stage_bytes;
        const bool use_a = (which != 0) == (g.a_is_weight != 0);
        if (which != 0 && g.weights_once)
          tma_load_2d_hint(dst, &map_a, &full[s], (kb0 + i) * BLOCK_K, a_tile * TILE_A, once);
        else
          tma_load_2d(use_a ? dst : dst + A_TILE_BYTES, use_a ? &map_a : &map_b, &full[s], (kb0 + i) * BLOCK_K,
                      use_a ? a_tile * TILE_A : b_tile * BN);
      };
      if (lane < pre) {
        mbar_expect_tx(&full[lane], (uint32_t)stage_bytes);
        issue(1, lane, lane);   // weights do not depend on the kernel before this one
      }
      pdl_wait();
      if (lane < pre) issue(0, lane, lane);
      // Few tokens: lanes 0 and 1 walk the k-blocks together (both wait for the stage, lane 0 posts the
      // byte count, then ONE instruction issues both tiles).  Many tokens: the tensor pipe sets the
      // pace and one lane issuing both tiles in turn is as fast (and measured slightly faster).
      const int n_issuers = g.a_is_weight ? 2 : 1;
      if (lane < n_issuers) {
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x) {
          decode(tile, a_tile, b_tile, split, kb0, n_kb);
          for (int i = 0; i < n_kb; ++i, ++it) {
            if (tile == (int)blockIdx.x && i < pre) continue;   // requested above
            const int s = it % stages;
            const uint32_t phase = (it / stages) & 1u;
            if (!mbar_wait(&empty[s], phase ^ 1u)) { failed = true; atomicExch(status, 1); break; }
            if (lane == 0) mbar_expect_tx(&full[s], (uint32_t)stage_bytes);
            if (n_issuers == 2) {
              issue(lane == 0 ? 1 : 0, s, i);
            } else {
              issue(1, s, i);
              issue(0, s, i);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(TILE_A, BN);
      uint32_t it = 0, lt = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x, ++lt) {
        int a_tile, b_tile, split, kb0, n_kb;
        decode(tile, a_tile, b_tile, split, kb0, n_kb);
        const uint32_t acc = lt & 1u, acc_phase = (lt >> 1) & 1u;
        if (!mbar_wait(&accum_empty[acc], acc_phase ^ 1u)) { failed = true; atomicExch(status, 4); break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * (uint32_t)g.acc_cols;
        for (int i = 0; i < n_kb; ++i, ++it) {
          const int s = it % stages;
          const uint32_t phase = (it / stages) & 1u;
          if (!mbar_wait(&full[s], phase)) { failed = true; atomicExch(status, 2); break; }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * stage_bytes);
          const uint32_t b_addr = a_addr + A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            tcgen05_mma_bf16(d_tmem, smem_desc_sw128(a_addr + k * UMMA_K * 2), smem_desc_sw128(b_addr + k * UMMA_K * 2),
                             idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(&empty[s]);  // frees the stage when these MMAs have read it
        }
        if (!failed) tcgen05_commit(&accum_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;  // the TMEM lanes this warp may read
    uint32_t lt = 0;
    for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x, ++lt) {
      int a_tile, b_tile, split, kb0, n_kb;
      decode(tile, a_tile, b_tile, split, kb0, n_kb);
      const uint32_t acc = lt & 1u, acc_phase = (lt >> 1) & 1u;
      if (!mbar_wait(&accum_full[acc], acc_phase)) { failed = true; atomicExch(status, 3); break; }
      tcgen05_fence_after();
      const int a = a_tile * TILE_A + quarter * 32 + lane;
      const uint32_t lane_base = tmem_base + acc * (uint32_t)g.acc_cols + ((uint32_t)(quarter * 32) << 16);
      const bool a_ok = a < g.a_rows;
      drain_accumulator<TO, EPI>(g, out, partial, split, a, a_ok, b_tile, lane_base);
      // this accumulator may be overwritten by the MMAs of the tile after next
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&accum_empty[acc]);
    }
  }
  if (failed) {
    // let copies that may still be in flight land before shared memory is given up
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ------------------------------------------------------ the kernel for CTA pairs
// Many tokens: two CTAs of a cluster (one per SM of a pair) share tiles of 256 tokens x 256 weight
// rows.  Each CTA loads its own 128 tokens (A) and 128 of the 256 weight rows (B); the MMAs
// (tcgen05 cta_group::2, M = 256, issued by the CTA of rank 0) read both halves of B and leave each
// CTA's 128 x 256 block of the result in its own tensor memory.  A single CTA's 128 x 256 MMA reads
// 12 KB of operands from shared memory for 131 cycles of tensor work, which is what bounds it; the
// pair's reads 8 KB per SM for the same work.
// Barriers: full[s] lives in rank 0 and counts the bytes of both CTAs' copies; empty[s] and
// accum_full[i] are signalled in both CTAs by one multicast commit; accum_empty[i] lives in rank 0
// and counts the epilogue warps of both CTAs.  Every wait is bounded as in the kernel above, and
// every path ends in the cluster barrier before tensor memory is freed, so that neither CTA's
// shared memory goes away while the other may still signal into it.
constexpr int PAIR_TILE = 256;
constexpr int PAIR_STAGE_BYTES = A_TILE_BYTES + (PAIR_TILE / 2) * BLOCK_K * 2;

template <typename TO, bool SWIGLU>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         TO* __restrict__ out, const GemmArgs g, int* __restrict__ status) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = g.stages;
  uint64_t* full = (uint64_t*)(smem + (size_t)stages * PAIR_STAGE_BYTES);
  uint64_t* empty = full + stages;
  uint64_t* accum_full = empty + stages;       // [2]
  uint64_t* accum_empty = accum_full + 2;      // [2]
  uint32_t* tmem_slot = (uint32_t*)(accum_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int total_tiles = g.a_tiles * g.b_tiles;
  const uint32_t tmem_cols = 2u * (uint32_t)PAIR_TILE;
  bool failed = false;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&accum_full[i], 1);
      mbar_init(&accum_empty[i], 8);   // one arrival per epilogue warp of either CTA
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();   // the other CTA's barriers exist before anything signals them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int n_kb = g.k_blocks;

  if (warp == 0) {
    if (pair < total_tiles) {
      int b_tile = pair / g.a_tiles, a_tile = pair - b_tile * g.a_tiles;
      const int pre = min(stages, n_kb);
      // which: 1 = this CTA's half of the weight rows of k-block i into stage s, 0 = its tokens
      auto issue = [&](int which, int s, int i) {
        uint8_t* dst = smem + (size_t)s * PAIR_STAGE_BYTES;
        const uint32_t bar = cluster_addr_of(&full[s], 0);
        if (which)
          tma_load_2d_pair(dst + A_TILE_BYTES, &map_b, bar, i * BLOCK_K, b_tile * PAIR_TILE + (int)rank * (PAIR_TILE / 2));
        else
          tma_load_2d_pair(dst, &map_a, bar, i * BLOCK_K, a_tile * PAIR_TILE + (int)rank * TILE_A);
      };
      if (lane < pre) {
        if (rank == 0) mbar_expect_tx(&full[lane], 2u * (uint32_t)PAIR_STAGE_BYTES);
        issue(1, lane, lane);   // weights do not depend on the kernel before this one
      }
      pdl_wait();
      if (lane < pre) issue(0, lane, lane);
      if (lane == 0) {
        uint32_t it = 0;
        for (int tile = pair; tile < total_tiles && !failed; tile += n_pairs) {
          b_tile = tile / g.a_tiles;
          a_tile = tile - b_tile * g.a_tiles;
          for (int i = 0; i < n_kb; ++i, ++it) {
            if (tile == pair && i < pre) continue;   // requested above
            const int s = it % stages;
            const uint32_t phase = (it / stages) & 1u;
            if (!mbar_wait(&empty[s], phase ^ 1u)) { failed = true; atomicExch(status, 5); break; }
            if (rank == 0) mbar_expect_tx(&full[s], 2u * (uint32_t)PAIR_STAGE_BYTES);
            issue(1, s, i);
            issue(0, s, i);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = instr_desc_bf16(PAIR_TILE, PAIR_TILE);
      uint32_t it = 0, lt = 0;
      for (int tile = pair; tile < total_tiles && !failed; tile += n_pairs, ++lt) {
        const uint32_t acc = lt & 1u, acc_phase = (lt >> 1) & 1u;
        if (!mbar_wait(&accum_empty[acc], acc_phase ^ 1u)) { failed = true; atomicExch(status, 8); break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * (uint32_t)PAIR_TILE;
        for (int i = 0; i < n_kb; ++i, ++it) {
          const int s = it % stages;
          const uint32_t phase = (it / stages) & 1u;
          if (!mbar_wait(&full[s], phase)) { failed = true; atomicExch(status, 6); break; }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * PAIR_STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            tcgen05_mma_bf16_pair(d_tmem, smem_desc_sw128(a_addr + k * UMMA_K * 2),
                                  smem_desc_sw128(b_addr + k * UMMA_K * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          tcgen05_commit_pair(&empty[s], 3);   // frees the stage in both CTAs when these MMAs have read it
        }
        if (!failed) tcgen05_commit_pair(&accum_full[acc], 3);
      }
    }
  } else {
    const int quarter = warp & 3;  // the TMEM lanes this warp may read
    uint32_t lt = 0;
    for (int tile = pair; tile < total_tiles && !failed; tile += n_pairs, ++lt) {
      const int b_tile = tile / g.a_tiles, a_tile = tile - b_tile * g.a_tiles;
      const uint32_t acc = lt & 1u, acc_phase = (lt >> 1) & 1u;
      if (!mbar_wait(&accum_full[acc], acc_phase)) { failed = true; atomicExch(status, 7); break; }
      tcgen05_fence_after();
      const int a = a_tile * PAIR_TILE + (int)rank * TILE_A + quarter * 32 + lane;
      const uint32_t lane_base = tmem_base + acc * (uint32_t)PAIR_TILE + ((uint32_t)(quarter * 32) << 16);
      drain_accumulator<TO, SWIGLU ? EPI_SWIGLU : EPI_PLAIN>(g, out, nullptr, 0, a, a < g.a_rows, b_tile, lane_base);
      // this accumulator may be overwritten by the MMAs of the tile after next
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(cluster_addr_of(&accum_empty[acc], 0));
    }
  }
  if (failed) {
    // let copies that may still be in flight land before shared memory is given up
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// out[m * ldo + n] = sum over splits of partial[z][m][n], in order of z.
template <typename TO>
__global__ void splitk_reduce_kernel(TO* __restrict__ out, const float* __restrict__ partial, int M, int N,
                                     int splits, long long ldo) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)M * N;
  if (idx >= total) return;
  float acc = 0.f;
  for (int z = 0; z < splits; ++z) acc += partial[(size_t)z * total + idx];
  const int m = (int)(idx / N), n = (int)(idx % N);
  out[(long long)m * ldo + n] = from_f32<TO>(acc);
}

// ------------------------------------------------------------------- tensor maps
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

struct MapKey {
  const void* ptr;
  int rows, cols, ld, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.ptr;
    for (int v : {k.rows, k.cols, k.ld, k.box_rows}) h = h * 1000003u ^ (size_t)v;
    return h;
  }
};

// A 2-D map over a row-major bf16 matrix [rows, cols] with row pitch ld elements,
// box [box_rows, 64], 128-byte swizzle, zero fill out of bounds.
bool make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int ld, int box_rows) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *map = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *map);
  return true;
}

int round_up_bn(int n) {
  for (int bn : {16, 32, 64, 128, 256})
    if (n <= bn) return bn;
  return 256;
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

// For the other tcgen05 kernels of the library (declared in gemm_internal.h).
bool zi_internal_make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int ld, int box_rows) {
  return make_map(map, ptr, rows, cols, ld, box_rows);
}
int* zi_internal_status_word() { return status_word(); }

// Whether the tensor-core kernel can take these operands: bfloat16, pointers aligned
// to 16 bytes, row pitches that are multiples of 16 bytes (TMA's rules).
extern "C" int zi_gemm_tcgen05_supported(const void* x, const void* w, int K, int ldx, int ldw) {
  return ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && (ldx % 8 == 0) && (ldw % 8 == 0) && K > 0 &&
         encode_fn() != nullptr;
}

// Size in bytes of the split-K workspace this call needs (0 when it does not split).
// `plan` receives {swap, BN, splits}.
extern "C" long long zi_gemm_tcgen05_plan(int M, int N, int K, int sm_count, int* plan) {
  const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
  // Up to 128 tokens the weight's rows take the MMA's 128 lanes and the tokens its columns: every tile
  // is full, where 65..128 tokens on the lanes would fill half of a second row of tiles (measured at
  // 65, 96 and 128 tokens: every product of the layer 5 to 25 % faster; at 160 and 256 slower).
  const int swap = M <= 128 ? 1 : 0;
  const int a_rows = swap ? N : M, b_rows = swap ? M : N;
  const int BN = swap ? round_up_bn(b_rows) : (b_rows >= 256 && M >= 256 ? 256 : 128 <= b_rows ? 128 : round_up_bn(b_rows));
  const int tiles = ((a_rows + TILE_A - 1) / TILE_A) * ((b_rows + BN - 1) / BN);
  int splits = 1;
  const int slots = 2 * (sm_count > 0 ? sm_count : 148);   // CTAs resident at once, two per SM
  if (swap && 2 * tiles <= slots) {
    // few tokens, few tiles: the weight is streamed once; as many splits as still fit on the GPU
    // at once, so that every SM pulls from memory: one wave, no tail
    while (tiles * splits * 2 <= slots && splits < 16 && k_blocks / (splits * 2) >= 8) splits *= 2;
  } else if (swap && tiles < slots) {
    // between half a wave and a whole one (192 tiles on 296 slots): without a split a third of the
    // slots idle; take the split count whose units (tile x split) fill whole waves best
    double best = 0.0;
    for (int s = 1; s <= 4 && k_blocks / s >= 8; ++s) {
      const int units = tiles * s;
      const double eff = (double)units / ((double)((units + slots - 1) / slots) * slots);
      if (eff > best + 0.02) {
        best = eff;
        splits = s;
      }
    }
  }
  if (!swap && sm_count > 0 && 2 * tiles <= sm_count) {
    // A few hundred tokens: the tiles leave most SMs idle, and a CTA walks all of K at the pace
    // of its own copies (about 0.45 us a k-block).  Splitting K spreads the walk over more CTAs
    // until L2 cannot feed them (about 10 TB/s), and costs the partial sums' round trip through
    // memory and a kernel to add them (about 8 us in all, measured at 256 to 512 tokens).  Split when
    // that model promises a tenth or more (512 tokens x 4096 x 12288: 78 us whole, 61 us in two).
    const double stage_b = (double)(A_TILE_BYTES + BN * BLOCK_K * 2);
    auto walk = [&](int s) {   // us for one CTA's share of K with s splits
      const double per_kb = tiles * s * stage_b / 10e6;
      return ((double)k_blocks / s) * (per_kb > 0.45 ? per_kb : 0.45);
    };
    const double unsplit = walk(1);
    double best = unsplit * 0.9;
    for (int s = 2; s <= 16 && tiles * s <= sm_count && k_blocks / s >= 8; ++s) {
      const double t = walk(s) + 2.0 * s * (double)M * N * 4.0 / 5e6 + 8.0;
      if (t < best) {
        best = t;
        splits = s;
      }
    }
  }
  if (splits > 1) {  // the number of splits that get at least one k-block
    const int kbps = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + kbps - 1) / kbps;
  }
  plan[0] = swap;
  plan[1] = BN;
  plan[2] = splits;
  return splits > 1 ? (long long)splits * M * N * (long long)sizeof(float) : 0;
}

namespace {
// Whether the product goes to the kernel for CTA pairs: switched on (zi_gemm_tcgen05_pair_enable, or
// ZINFER_B200_GEMM_PAIR=1 in the environment), tokens on the lanes, 256-row tiles on both sides, no
// K split, and few enough padding rows (300 tokens would fill 512 rows of pair tiles but 384 of
// single tiles).  Off by default: in a prefill step both kernels run at the pace the power limit
// allows (1.2-1.3 PFLOP/s), so the pair's lighter shared-memory traffic buys nothing there.
int g_pair_enabled = -1;   // -1: ask the environment
bool use_pair_kernel(const int* plan, int M) {
  if (g_pair_enabled < 0) {
    const char* e = getenv("ZINFER_B200_GEMM_PAIR");
    g_pair_enabled = (e && e[0] == '1') ? 1 : 0;
  }
  if (!g_pair_enabled || plan[0] || plan[1] != PAIR_TILE || plan[2] != 1) return false;
  const int pair_rows = (M + PAIR_TILE - 1) / PAIR_TILE * PAIR_TILE, single_rows = (M + TILE_A - 1) / TILE_A * TILE_A;
  return pair_rows == single_rows || M >= 1024;
}
// Rows of the B side's copy box.
int b_box_rows(const int* plan, int M) { return use_pair_kernel(plan, M) ? PAIR_TILE / 2 : plan[1]; }

// Launch of the pair kernel: clusters of two CTAs, as many as are resident at once (74 on 148 SMs).
// Returns -3 when no cluster fits (the caller then has no maps for the single kernel: an error).
template <typename TO>
int launch_pair(void* out, const CUtensorMap& map_a, const CUtensorMap& map_b, GemmArgs g, int M, int N, int K,
                int* status, int swiglu, const char* what, cudaStream_t stream) {
  g.a_tiles = (M + PAIR_TILE - 1) / PAIR_TILE;
  g.b_tiles = (N + PAIR_TILE - 1) / PAIR_TILE;
  g.BN = PAIR_TILE;
  g.acc_cols = PAIR_TILE;
  g.splits = 1;
  g.k_blocks_per_split = g.k_blocks;
  g.stages = 6;
  if (g.stages > g.k_blocks) g.stages = g.k_blocks < 2 ? 2 : g.k_blocks;
  const size_t smem = 1024 + (size_t)g.stages * PAIR_STAGE_BYTES + (2 * g.stages + 4) * sizeof(uint64_t) + 16;
  auto kern = swiglu ? gemm_tcgen05_pair_kernel<TO, true> : gemm_tcgen05_pair_kernel<TO, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return zi_refuse("%s: cannot get %zu bytes of shared memory", what, smem);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // clusters resident at once: asked once per device, kernel and number of stages (no allocation here:
  // this path also serves callers that must not allocate)
  static std::mutex mu;
  static int resident[64][2][2][8];   // 0 = not asked yet, else the answer + 1
  int clusters = 0, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return zi_refuse("%s: no current device", what);
  {
    std::lock_guard<std::mutex> lock(mu);
    int& slot = resident[dev][swiglu ? 1 : 0][sizeof(TO) == 2 ? 1 : 0][g.stages];
    if (slot == 0) {
      cfg.gridDim = dim3(2 * 148);
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
      }
      slot = n + 1;
    }
    clusters = slot - 1;
  }
  if (clusters <= 0) return zi_refuse("%s: no cluster of two CTAs fits on this GPU", what);
  const int total_tiles = g.a_tiles * g.b_tiles;
  if (clusters > total_tiles) clusters = total_tiles;
  cfg.gridDim = dim3(2 * clusters);
  cfg.numAttrs = g_zi_pdl_enabled ? 2 : 1;
  e = cudaLaunchKernelEx(&cfg, kern, map_a, map_b, (TO*)out, g, status);
  if (e != cudaSuccess) return zi_refuse("%s: launch failed: %s", what, cudaGetErrorString(e));
  return zi_check_launch(what);
}

// One launch of the single-CTA kernel: as many CTAs as fit on the GPU at once, by shared memory and
// by tensor memory (512 columns per SM), or one per tile if those are fewer.
template <typename TO, int EPI>
int launch_single(void* out, const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmArgs& g, float* partial,
                  int* status, int sm_count, size_t smem, int total_tiles, const char* what, cudaStream_t stream) {
  auto kern = gemm_tcgen05_kernel<TO, EPI>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return zi_refuse("%s: cannot get %zu bytes of shared memory", what, smem);
  int per_sm = (int)((227 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : per_sm;
  const int by_tmem = 512 / (2 * g.acc_cols);
  if (per_sm > by_tmem) per_sm = by_tmem;
  if (per_sm > 2) per_sm = 2;
  int grid = per_sm * (sm_count > 0 ? sm_count : 148);
  if (grid > total_tiles) grid = total_tiles;
  if (g.a_is_weight && total_tiles > grid) {
    // Few tokens, more tiles than CTA slots (the output head: 1,187 tiles on 296 slots): as many CTAs as give
    // every one the same number of tiles (238 with five each), instead of all slots with a last round of three
    // tiles, which three CTAs would walk alone at the pace of their own copies (1 % of a step at one request).
    const int rounds = (total_tiles + grid - 1) / grid;
    grid = (total_tiles + rounds - 1) / rounds;
  }
  zi_launch(kern, dim3(grid), dim3(THREADS), smem, stream, map_a, map_b, (TO*)out, partial, g, status);
  return zi_check_launch(what);
}

// Launches the product (and, unless deferred, the split-K reduction) with the given
// tensor maps, partial-sum buffer and status word.  Both entry points end here.
int launch_gemm(void* out, int out_dtype, const CUtensorMap& map_a, const CUtensorMap& map_b, int M, int N, int K,
                int ldo, const int* plan, float* partial_buf, int* status, int sm_count, int defer_reduce,
                const char* what, cudaStream_t stream, int epi = EPI_PLAIN, float* cand_val = nullptr,
                int* cand_idx = nullptr) {
  const int swap = plan[0], BN = plan[1], splits = plan[2];
  const int swiglu = epi == EPI_SWIGLU;
  GemmArgs g;
  g.cand_val = cand_val;
  g.cand_idx = cand_idx;
  g.cand_units = swap ? (N + TILE_A - 1) / TILE_A * (TILE_A / 32) : 0;
  g.a_rows = swap ? N : M;
  g.b_rows = swap ? M : N;
  g.a_tiles = (g.a_rows + TILE_A - 1) / TILE_A;
  g.b_tiles = (g.b_rows + BN - 1) / BN;
  g.k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
  g.k_blocks_per_split = (g.k_blocks + splits - 1) / splits;
  g.splits = (g.k_blocks + g.k_blocks_per_split - 1) / g.k_blocks_per_split;
  g.sa = swap ? 1 : ldo;
  g.sb = swap ? ldo : 1;
  g.pa = swap ? 1 : N;
  g.pb = swap ? N : 1;
  g.BN = BN;
  g.acc_cols = BN < 32 ? 32 : BN;   // two accumulators: 64 .. 512 columns, a power of two
  g.a_is_weight = swap;
  // Few tokens: every weight tile is read by exactly one CTA, once a step.  Loaded with the L2 policy "evict first",
  // the 15 GB of weights that stream through L2 every step no longer push out the activations, partial sums and tables
  // that the step reads again (measured, alternating runs: 2 % of a decode step at 1 and 8 requests, 1 % at 64).
  g.weights_once = swap;
  g.act_ld = ldo;
  const int stage_bytes = A_TILE_BYTES + BN * BLOCK_K * 2;
  // few tokens: as many stages (up to 6) as still let two CTAs share an SM's shared memory
  g.stages = swap ? (111 * 1024 / stage_bytes > 6 ? 6 : 111 * 1024 / stage_bytes) : (BN >= 256 ? 4 : 6);
  if (g.stages > g.k_blocks_per_split) g.stages = g.k_blocks_per_split < 2 ? 2 : g.k_blocks_per_split;
  const size_t smem = 1024 + (size_t)g.stages * stage_bytes + (2 * g.stages + 4) * sizeof(uint64_t) + 16;
  const int total_tiles = g.a_tiles * g.b_tiles * g.splits;
  float* partial = g.splits > 1 ? partial_buf : nullptr;

  if (use_pair_kernel(plan, M)) {
    ZI_DISPATCH_DTYPE(out_dtype, TO, { return launch_pair<TO>(out, map_a, map_b, g, M, N, K, status, swiglu, what, stream); });
  }
  if (epi == EPI_ARGMAX) {
    if (out_dtype != ZI_F32 || !swap || g.splits != 1 || !cand_val || !cand_idx)
      return zi_refuse("%s: the argmax epilogue takes 32-bit results of an unsplit product of at most 128 tokens", what);
    return launch_single<float, EPI_ARGMAX>(out, map_a, map_b, g, partial, status, sm_count, smem, total_tiles, what, stream);
  }
  ZI_DISPATCH_DTYPE(out_dtype, TO, {
    int rc = swiglu ? launch_single<TO, EPI_SWIGLU>(out, map_a, map_b, g, partial, status, sm_count, smem, total_tiles, what, stream)
                    : launch_single<TO, EPI_PLAIN>(out, map_a, map_b, g, partial, status, sm_count, smem, total_tiles, what, stream);
    if (rc) return rc;
    if (partial && !defer_reduce) {
      const size_t total = (size_t)M * N;
      zi_launch(splitk_reduce_kernel<TO>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (TO*)out,
                partial, M, N, g.splits, (long long)ldo);
      rc = zi_check_launch("splitk_reduce");
      if (rc) return rc;
    }
  });
  return 0;
}
}  // namespace

// With `defer_reduce` and a split product, the partial sums are left in `workspace` as
// [splits, M, N] floats for a consumer that adds them itself, and `out` is not written.
extern "C" int zi_gemm_tcgen05(void* out, int out_dtype, const void* x, const void* w, int M, int N, int K, int ldx,
                               int ldw, int ldo, float* workspace, long long workspace_bytes, int sm_count,
                               int defer_reduce, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!zi_gemm_tcgen05_supported(x, w, K, ldx, ldw))
    return zi_refuse("gemm_tcgen05: operands must be 16-byte aligned bfloat16 with row pitches in multiples of 8");
  int plan[3];
  const long long need = zi_gemm_tcgen05_plan(M, N, K, sm_count, plan);
  if (need > workspace_bytes) return zi_refuse("gemm_tcgen05: split-K needs %lld workspace bytes, got %lld", need, workspace_bytes);
  const int swap = plan[0];
  const int a_rows = swap ? N : M, b_rows = swap ? M : N;
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, swap ? w : x, a_rows, K, swap ? ldw : ldx, TILE_A) ||
      !make_map(&map_b, swap ? x : w, b_rows, K, swap ? ldx : ldw, b_box_rows(plan, M)))
    return zi_refuse("gemm_tcgen05: cuTensorMapEncodeTiled failed");
  int* status = status_word();
  if (!status) return zi_refuse("gemm_tcgen05: cannot allocate the status word");
  return launch_gemm(out, out_dtype, map_a, map_b, M, N, K, ldo, plan, workspace, status, sm_count, defer_reduce,
                     "gemm_tcgen05", stream);
}

// gate_up product with the SwiGLU applied in the epilogue: w is [2I, K] with rows interleaved
// in blocks of 64 (64 gate rows, then the 64 up rows of the same features); out is [M, I].
// Returns -2 (without launching) when the plan would split K: the caller then uses the
// plain product and the separate SwiGLU kernel.
extern "C" int zi_gemm_tcgen05_swiglu(void* out, int out_dtype, const void* x, const void* w, int M, int N2, int K,
                                      int ldx, int ldw, int ldo, int sm_count, cudaStream_t stream) {
  if (M <= 0 || N2 <= 0) return 0;
  if (N2 % 128) return zi_refuse("gemm_swiglu: the interleaved weight needs a multiple of 128 rows, got %d", N2);
  if (!zi_gemm_tcgen05_supported(x, w, K, ldx, ldw))
    return zi_refuse("gemm_swiglu: operands must be 16-byte aligned bfloat16 with row pitches in multiples of 8");
  int plan[3];
  zi_gemm_tcgen05_plan(M, N2, K, sm_count, plan);
  if (plan[2] > 1) return -2;
  const int swap = plan[0];
  // Few tokens: the separate SwiGLU kernel is the better schedule.  While it runs, the CTAs of
  // the down product are already resident and prefetch their weights, which they cannot do
  // while this product's CTAs still hold the shared memory.  (Measured: fused is 6 us per layer slower.)
  if (swap) return -2;
  if (plan[1] < 128) return -2;
  const int a_rows = swap ? N2 : M, b_rows = swap ? M : N2;
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, swap ? w : x, a_rows, K, swap ? ldw : ldx, TILE_A) ||
      !make_map(&map_b, swap ? x : w, b_rows, K, swap ? ldx : ldw, b_box_rows(plan, M)))
    return zi_refuse("gemm_swiglu: cuTensorMapEncodeTiled failed");
  int* status = status_word();
  if (!status) return zi_refuse("gemm_swiglu: cannot allocate the status word");
  return launch_gemm(out, out_dtype, map_a, map_b, M, N2, K, ldo, plan, nullptr, status, sm_count, 0, "gemm_swiglu",
                     stream, EPI_SWIGLU);
}

// Rows of candidates per token that zi_gemm_tcgen05_argmax leaves: one per 32 weight rows,
// rounded up to whole tiles of 128.
extern "C" int zi_gemm_argmax_units(int N) { return (N + TILE_A - 1) / TILE_A * (TILE_A / 32); }

// The product into 32-bit `out` [M, N] as zi_gemm_tcgen05 makes it, and beside it, for every token, the
// first maximum of each 32 weight rows as cand_val/cand_idx [M, units] (units from
// zi_gemm_argmax_units): what an argmax over the row needs, without reading the row again.
// Returns -2 (without launching) when the product would not run with the weight rows on the lanes
// and K whole (more than 128 tokens, or so few weight rows that K is split): the caller then
// takes the plain product and the argmax kernel.
extern "C" int zi_gemm_tcgen05_argmax(float* out, const void* x, const void* w, int M, int N, int K, int ldx, int ldw,
                                      int ldo, float* cand_val, int* cand_idx, int sm_count, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!zi_gemm_tcgen05_supported(x, w, K, ldx, ldw))
    return zi_refuse("gemm_argmax: operands must be 16-byte aligned bfloat16 with row pitches in multiples of 8");
  int plan[3];
  zi_gemm_tcgen05_plan(M, N, K, sm_count, plan);
  if (!plan[0] || plan[2] > 1) return -2;
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, w, N, K, ldw, TILE_A) || !make_map(&map_b, x, M, K, ldx, plan[1]))
    return zi_refuse("gemm_argmax: cuTensorMapEncodeTiled failed");
  int* status = status_word();
  if (!status) return zi_refuse("gemm_argmax: cannot allocate the status word");
  return launch_gemm(out, ZI_F32, map_a, map_b, M, N, K, ldo, plan, nullptr, status, sm_count, 0, "gemm_argmax", stream,
                     EPI_ARGMAX, cand_val, cand_idx);
}

// Switches the kernel for CTA pairs on (1) or off (0) for products of 256 tokens and more; returns
// the setting before.
extern "C" int zi_gemm_tcgen05_pair_enable(int on) {
  const int before = g_pair_enabled > 0 ? 1 : 0;
  g_pair_enabled = on ? 1 : 0;
  return before;
}

// Reads and clears the status word of the tensor-core kernels (synchronises the
// device).  0 = every bounded wait completed.
extern "C" int zi_gemm_tcgen05_status() {
  int* status = status_word();
  if (!status) return -1;
  int host = 0;
  if (cudaMemcpy(&host, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (host != 0) cudaMemset(status, 0, sizeof(int));
  return host;
}

// ------------------------------------------------------------------------------
// Self-test of the failure path: one CTA waits, with a limit of `tries`, on an mbarrier at
// which nobody ever arrives.  The wait runs out, the kernel records `code` in the status word
// exactly as the products do, and returns normally: nothing faults and nothing hangs.  It lets
// a test see the whole chain (bounded wait -> status word -> zi_gemm_tcgen05_status -> error).
namespace {
__global__ void wait_that_runs_out_kernel(int* __restrict__ status, int code, uint32_t tries) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!mbar_wait(&bar, 0, tries)) atomicExch(status, code);
  }
}
}  // namespace

extern "C" int zi_selftest_wait_runs_out(int code, int tries, cudaStream_t stream) {
  if (code == 0 || tries <= 0 || tries > (1 << 20))
    return zi_refuse("selftest_wait_runs_out: code must be non-zero and tries in 1..2^20");
  int* status = status_word();
  if (!status) return zi_refuse("selftest_wait_runs_out: cannot allocate the status word");
  wait_that_runs_out_kernel<<<1, 32, 0, stream>>>(status, code, (uint32_t)tries);
  return zi_check_launch("selftest_wait_runs_out");
}

// ------------------------------------------------------------------------------
// The same product for callers that cannot allocate device memory (declared in
// gemm_static_scratch.h).  Split-K partial sums go to a fixed array in the
// library's own device image instead of a caller's workspace.
namespace {

// 2 Mi floats = 8 MiB: every GPU that loads this library holds them until it exits.
constexpr long long STATIC_SCRATCH_FLOATS = 2ll * 1024 * 1024;
static __device__ __align__(256) float g_static_scratch[STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_static_status;

constexpr int MAX_DEVICES = 64;
struct StaticScratch {
  float* scratch = nullptr;  // device address of g_static_scratch on that device
  int* status = nullptr;     // device address of g_static_status on that device
};

// In host code `g_static_scratch` is only a handle for the runtime, not an address
// the GPU can use: the device address is asked for once per device, with that
// device current.
bool static_scratch_for_current_device(StaticScratch* out, int* device_out) {
  static std::mutex mu;
  static StaticScratch table[MAX_DEVICES];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (!table[dev].scratch) {
    void* p = nullptr;
    void* s = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return false;
    if (cudaGetSymbolAddress(&s, g_static_status) != cudaSuccess || !s) return false;
    table[dev].scratch = (float*)p;
    table[dev].status = (int*)s;
  }
  *out = table[dev];
  *device_out = dev;
  return true;
}

// The tensor map of make_map(), encoded straight into `map` (no cache, no host allocation).
bool encode_map_direct(CUtensorMap* map, const void* ptr, int rows, int cols, int ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" long long zi_gemm_static_scratch_capacity_bytes() { return STATIC_SCRATCH_FLOATS * (long long)sizeof(float); }

// Reads and clears the library's own status word on the current device (the one a call with
// wait_status == NULL reports into).  Waits for the device; allocates nothing.
extern "C" int zi_gemm_static_scratch_status() {
  StaticScratch ss;
  int dev = -1;
  if (!static_scratch_for_current_device(&ss, &dev)) return -1;
  int host = 0;
  if (cudaMemcpy(&host, ss.status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (host != 0 && cudaMemset(ss.status, 0, sizeof(int)) != cudaSuccess) return -2;
  return host;
}

extern "C" int zi_gemm_tcgen05_static_scratch(void* out, int out_dtype, const void* x, const void* w, int M, int N,
                                              int K, int ldx, int ldw, int ldo, int sm_count, int* wait_status,
                                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!zi_gemm_tcgen05_supported(x, w, K, ldx, ldw))
    return zi_refuse("gemm_static_scratch: operands must be 16-byte aligned bfloat16 with row pitches in multiples of 8");
  int plan[3];
  const long long need = zi_gemm_tcgen05_plan(M, N, K, sm_count, plan);
  if (need > zi_gemm_static_scratch_capacity_bytes())
    return zi_refuse("gemm_static_scratch: this product splits K and needs %lld bytes of scratch; the built-in scratch "
                     "holds %lld (use zi_gemm_tcgen05 with a workspace of your own)",
                     need, zi_gemm_static_scratch_capacity_bytes());
  StaticScratch ss;
  int dev = -1;
  if (!static_scratch_for_current_device(&ss, &dev))
    return zi_refuse("gemm_static_scratch: cudaGetSymbolAddress of the built-in scratch failed on the current device");
  const int swap = plan[0];
  const int a_rows = swap ? N : M, b_rows = swap ? M : N;
  const int lda = swap ? ldw : ldx, ldb = swap ? ldx : ldw;
  CUtensorMap map_a, map_b;
  if (!encode_map_direct(&map_a, swap ? w : x, a_rows, K, lda, TILE_A) ||
      !encode_map_direct(&map_b, swap ? x : w, b_rows, K, ldb, b_box_rows(plan, M)))
    return zi_refuse("gemm_static_scratch: cuTensorMapEncodeTiled failed");
  // The status word is only ever written with a non-zero code, never cleared here: a failure of an
  // earlier call stays visible until it is read.  The partial sums need no clearing either, every
  // element that the second kernel reads is written by the first.
  int* status = wait_status ? wait_status : ss.status;
  return launch_gemm(out, out_dtype, map_a, map_b, M, N, K, ldo, plan, ss.scratch, status, sm_count, 0,
                     "gemm_static_scratch", stream);
}

ZI_TRACE_SETTER(gemm_tcgen05)
