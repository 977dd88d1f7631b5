// Whole decoder layers of a decode step (every request brings one token, at most 64
// requests) in ONE persistent kernel, one CTA per SM.
//
// A decode step reads every weight once and does almost no arithmetic: its time is the
// time the weights take to come from HBM plus whatever stands between two loads.  As a chain
// of kernels, every product of a layer pays a drain and a start in which HBM idles.  Here the
// weights of all four products of all layers of a launch are ONE stream per CTA: the TMA
// producer warp walks (layer, product, unit, k-block) and keeps its ring of shared-memory
// stages full across the boundaries of phases and layers, so the next product's weights
// are already on their way while the current one's results are written, the grid meets at a
// barrier and the small steps between products run.
//
// The ring takes nearly all of shared memory (what is in flight per SM bounds the rate at which
// HBM can be read); the attention phase borrows it for its own rings of keys and values.
//
// Warps: 0..3 = compute (accumulator read-back, residual + norm, attention over the paged cache,
// SwiGLU, and the grid barriers), 4 = tensor-memory owner and tcgen05.mma issuer, 5..7 = TMA
// producers (weights ahead of time; activations once their phase is open).
//
// A layer is h += attn(norm1(h)); h += mlp(norm2(h)) with RMSNorm, grouped-query attention
// (optional per-head q/k RMSNorm, optional rotary tables) and a SwiGLU feed-forward.  Phases
// of the compute warps, a grid barrier after each:
//   R1  h += update of the layer before (split-K partial sums); hw = bf16(h * w1); row sums of squares
//   G1  q|k|v rows = hw * Wqkv^T as split-K partial sums
//   AT  per (request, kv head, key split): rows * 1/rms, q/k norm, rotary, k and v into their
//       page, attention over the cache
//   CB  splits combined (only with more than one key split)
//   G2  output projection;  R2  h += it, hw = bf16(h * w2), sums of squares
//   G3  gate|up;  SW  act = silu(gate / rms) * (up / rms);  G4  down projection
// The 1/rms of a row is a scalar, so the norm's division moves behind the product: the
// product reads bf16(h * w) and its consumer scales by 1/sqrt(mean(h^2) + eps) in 32-bit.
//
// Products are swap-AB (weight rows on the 128 accumulator lanes, tokens padded to 16/32/64
// columns).  A product's units are (128-row tile, k split); CTA c takes units c, c + grid, ...;
// the split count is chosen so the units fill the grid evenly.  Partial sums are added by
// their consumer in split order, so results do not depend on timing.
//
// Every wait (mbarrier, grid barrier) has a time limit; a CTA whose wait runs out records a
// code in the status word, sets the abort bit of the barrier counter (which releases every
// other waiter), lets copies in flight land, frees its tensor memory and returns.
#include <cuda.h>

#include "api.h"
#include "attention_tiles.cuh"
#include "common.cuh"
#include "gemm_internal.h"
#include "tcgen05_ptx.cuh"

namespace {

#ifndef DL_CTAS_PER_SM
#define DL_CTAS_PER_SM 2
#endif
#ifndef DL_PRODUCERS
#define DL_PRODUCERS 2
#endif
constexpr int DL_COMPUTE = 128;
constexpr int DL_THREADS = DL_COMPUTE + 32 + 32 * DL_PRODUCERS;
constexpr size_t DL_SMEM_BUDGET = (size_t)227 * 1024 / DL_CTAS_PER_SM - (DL_CTAS_PER_SM > 1 ? 1024 : 0);
constexpr int TILE_A = 128, BLOCK_K = 64, UMMA_K = 16, A_TILE_BYTES = TILE_A * BLOCK_K * 2;
constexpr int CHUNK = 256;            // columns of one elementwise item, two per compute thread
constexpr int MAX_TOKENS = 64;
constexpr int MAX_STAGES = 12;
constexpr int MAX_GROUPS = 4;
constexpr unsigned ABORT_BIT = 0x80000000u;
constexpr long long WAIT_CYCLES = 4000000000ll;   // about two seconds of SM clock

struct LayerDesc {
  CUtensorMap w[4];          // Wqkv [n_qkv, hidden], Wo [hidden, nq d], Wgu [2 inter, hidden], Wdown [hidden, inter]
  const float* norm1_w;
  const float* norm2_w;
  const float* q_norm_w;     // [d] or null
  const float* k_norm_w;
  bf16* kcache;              // [pages, nkv, page_size, d]
  bf16* vcache;
  const float* cos_t;        // [n_table_pos, d / 2] or null
  const float* sin_t;
  float eps1, eps2, qk_eps, scale_log2;
  int n_table_pos, window, kv_group, pad0;
  long long pad1[4];
};
static_assert(sizeof(LayerDesc) % 128 == 0, "descriptors keep the tensor maps aligned");

struct GroupArrays {
  const int* slots;          // [tokens] page * page_size + offset of each token's k and v
  const int* block_tables;   // [requests, bt_stride]
  int bt_stride, pad;
};

struct Args {
  CUtensorMap map_hw, map_xo, map_act;   // activations [64, K], box [BN, 64]
  const LayerDesc* layers;
  int n_layers;
  int B, BN, stages, acc_cols;
  int fused_off;               // where the attention keeps its q tile and the token's own k, v (bytes from the ring's start)
  int hidden, nq, nkv, inter, n_qkv, n_gu, interleave;
  int n[4], k[4], tiles[4], kb[4], splits[4];   // the four products: rows, depth, 128-row tiles, k-blocks, k splits
  int att_splits, page_size, page_shift, chunks;  // chunks: CHUNK-column pieces of a row of h
  float* h;                    // [B, hidden] residual stream, 32-bit, updated in place
  const float* pend;           // [pend_splits][B][hidden] update not yet added, or null
  int pend_splits;
  bf16* hw;                    // [64, hidden]
  bf16* xo;                    // [64, nq d]
  bf16* act;                   // [64, inter]
  float* ssq;                  // [2][chunks][64]
  float* part[4];              // partial sums of the four products, [splits][B][n]
  float* attn_part;
  const int* positions;
  const int* cu_q;
  const int* kv_lens;
  const int* dec_seq;
  GroupArrays groups[MAX_GROUPS];
  unsigned* counter;           // grid barrier: arrivals so far (zero at launch); top bit = abort
  int* status;
};

struct Ctl {
  uint64_t full[MAX_STAGES], empty[MAX_STAGES], accum_full[2], accum_empty[2];
  uint32_t tmem;
  volatile int failed;
  volatile int opened;       // grid barriers this CTA's compute warps have passed (the producer reads it)
  volatile int att_done;     // attention phases this CTA has finished: the ring is the producer's again
  int verdict;               // what the compute warps agreed on at their last grid barrier
  float inv[MAX_TOKENS];
  float red[4];
};

// Tiles of an attention warp's ring while the attention phase has the whole ring's memory.
template <int D> struct AttCfg { static constexpr int STAGES = (D <= 64 ? 8 : 6) / DL_CTAS_PER_SM; };

struct ComputeSync {
  static __device__ __forceinline__ void sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
};

// Whether the phase has completed; never blocks.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Waits for the phase; false when the CTA has failed meanwhile or the time ran out.
__device__ __forceinline__ bool mbar_wait_timed(uint64_t* bar, uint32_t parity, volatile int* failed) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 127u) == 0 && (*failed || clock64() - t0 > WAIT_CYCLES)) return false;
  }
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ void fail(const Args& a, Ctl* ctl, int code) {
  ctl->failed = 1;
  atomicOr(a.counter, ABORT_BIT);
  atomicCAS(a.status, 0, code);
}

// The walk of one CTA through the k-blocks of all its units of all products of all layers.
struct Cursor {
  int cta, grid, layer, j, u, kb, kb_end, tile, z;
  bool done;
  __device__ void settle(const Args& a) {
    for (;;) {
      if (layer >= a.n_layers) {
        done = true;
        return;
      }
      if (u < a.tiles[j] * a.splits[j]) break;
      u = cta;
      if (++j == 4) {
        j = 0;
        ++layer;
      }
    }
    z = u / a.tiles[j];
    tile = u - z * a.tiles[j];
    kb = (int)((long long)z * a.kb[j] / a.splits[j]);
    kb_end = (int)((long long)(z + 1) * a.kb[j] / a.splits[j]);
  }
  __device__ void start(const Args& a, int cta_, int grid_) {
    cta = cta_;
    grid = grid_;
    layer = 0;
    j = 0;
    u = cta_;
    done = false;
    settle(a);
  }
  __device__ void next_unit(const Args& a) {
    u += grid;
    settle(a);
  }
  __device__ void next_kb(const Args& a) {
    if (++kb >= kb_end) next_unit(a);
  }
};

// Barriers per layer, and the number of barriers that must have been passed before the
// activations of product j of a layer may be read.
__device__ __forceinline__ int barriers_per_layer(const Args& a) { return 8 + (a.att_splits > 1 ? 1 : 0); }
__device__ __forceinline__ int opens_after(const Args& a, int layer, int j) {
  return layer * barriers_per_layer(a) + 1 + 2 * j + ((j >= 1 && a.att_splits > 1) ? 1 : 0);
}

// Grid barrier of the compute warps; `n` = barriers passed after this one.  False on abort
// (the same answer in every compute thread: they leave the layer loop only here).
__device__ __forceinline__ bool grid_barrier(const Args& a, Ctl* ctl, int ctid, int n) {
  fence_proxy_async();   // this thread's global writes come before other CTAs' TMA reads of them
  ComputeSync::sync();
  if (ctid == 0) {
    // release: what this CTA's compute threads wrote (ordered before by the barrier above) is
    // visible to whoever acquires the count
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.counter) : "memory");
    const unsigned target = (unsigned)n * gridDim.x;
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
      const unsigned v = ld_acquire(a.counter);
      if (v & ABORT_BIT) {
        ctl->failed = 1;
        break;
      }
      if (v >= target) break;
      if ((it & 63u) == 63u && clock64() - t0 > WAIT_CYCLES) {
        fail(a, ctl, 20);
        break;
      }
    }
    ctl->verdict = ctl->failed;   // one thread decides, so that all compute warps leave together
    ctl->opened = n;
  }
  ComputeSync::sync();
  return ctl->verdict == 0;
}

// h += sum of the splits of `pend` (in order); hw = bf16(h * w); sums of squares per (chunk, row).
__device__ __forceinline__ void phase_residual(const Args& a, Ctl* ctl, int ctid, const float* pend, int pend_splits,
                                               const float* __restrict__ w, float* ssq) {
  const int items = a.B * a.chunks;
  const size_t zstride = (size_t)a.B * a.hidden;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int row = item / a.chunks, chunk = item - row * a.chunks;
    const int col = chunk * CHUNK + 2 * ctid;
    float ss = 0.f;
    if (col < a.hidden) {
      float* hp = a.h + (size_t)row * a.hidden + col;
      float2 v = *reinterpret_cast<float2*>(hp);
      for (int z = 0; z < pend_splits; ++z) {
        const float2 p = *reinterpret_cast<const float2*>(pend + z * zstride + (size_t)row * a.hidden + col);
        v.x += p.x;
        v.y += p.y;
      }
      if (pend_splits > 0) *reinterpret_cast<float2*>(hp) = v;
      const float2 ww = *reinterpret_cast<const float2*>(w + col);
      *reinterpret_cast<uint32_t*>(a.hw + (size_t)row * a.hidden + col) = pack_bf16(v.x * ww.x, v.y * ww.y);
      ss = v.x * v.x + v.y * v.y;
    }
    ss = warp_sum(ss);
    ComputeSync::sync();   // red may still be read from the item before
    if ((ctid & 31) == 0) ctl->red[ctid >> 5] = ss;
    ComputeSync::sync();
    if (ctid == 0) ssq[chunk * MAX_TOKENS + row] = (ctl->red[0] + ctl->red[1]) + (ctl->red[2] + ctl->red[3]);
  }
}

// 1 / sqrt(mean(h^2) + eps) of every row into ctl->inv, from the chunk sums (in chunk order).
__device__ __forceinline__ void row_scales(const Args& a, Ctl* ctl, int ctid, const float* ssq, float eps) {
  if (ctid < a.B) {
    float s = 0.f;
    for (int c = 0; c < a.chunks; ++c) s += ssq[c * MAX_TOKENS + ctid];
    ctl->inv[ctid] = 1.0f / sqrtf(s / (float)a.hidden + eps);
  }
  ComputeSync::sync();
}

// act = silu(gate / rms) * (up / rms) from the partial sums of the gate|up product.
__device__ __forceinline__ void phase_swiglu(const Args& a, Ctl* ctl, int ctid) {
  const int chunks = (a.inter + CHUNK - 1) / CHUNK;
  const int items = a.B * chunks;
  const size_t zstride = (size_t)a.B * a.n_gu;
  for (int item = blockIdx.x; item < items; item += gridDim.x) {
    const int row = item / chunks, chunk = item - row * chunks;
    const int f = chunk * CHUNK + 2 * ctid;
    if (f >= a.inter) continue;
    int gc, uc;
    if (a.interleave > 0) {
      gc = (f / a.interleave) * 2 * a.interleave + f % a.interleave;
      uc = gc + a.interleave;
    } else {
      gc = f;
      uc = f + a.inter;
    }
    const float* p = a.part[2] + (size_t)row * a.n_gu;
    float2 g = make_float2(0.f, 0.f), u = g;
    for (int z = 0; z < a.splits[2]; ++z) {
      const float2 x = *reinterpret_cast<const float2*>(p + z * zstride + gc);
      const float2 y = *reinterpret_cast<const float2*>(p + z * zstride + uc);
      g.x += x.x;
      g.y += x.y;
      u.x += y.x;
      u.y += y.y;
    }
    const float inv = ctl->inv[row];
    g.x *= inv;
    g.y *= inv;
    u.x *= inv;
    u.y *= inv;
    *reinterpret_cast<uint32_t*>(a.act + (size_t)row * a.inter + f) =
        pack_bf16(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
  }
}

// The compute warps' side of product j: accumulators of this CTA's units out of tensor memory
// into part[j][z][token][row of the weight].
__device__ __forceinline__ void phase_epilogue(const Args& a, Ctl* ctl, int j, uint32_t tmem_base, int warp, int lane,
                                               uint32_t& lt) {
  const int quarter = warp & 3;   // the tensor-memory lanes this warp may read
  const int units = a.tiles[j] * a.splits[j];
  const int N = a.n[j];
  for (int u = blockIdx.x; u < units; u += gridDim.x, ++lt) {
    const int z = u / a.tiles[j], tile = u - z * a.tiles[j];
    const uint32_t acc = lt & 1u, acc_phase = (lt >> 1) & 1u;
    if (!mbar_wait_timed(&ctl->accum_full[acc], acc_phase, &ctl->failed)) {
      if (!ctl->failed) fail(a, ctl, 23);
      return;   // the next grid barrier ends the kernel for all warps together
    }
    tcgen05_fence_after();
    const int row = tile * TILE_A + quarter * 32 + lane;
    const uint32_t taddr = tmem_base + acc * (uint32_t)a.acc_cols + ((uint32_t)(quarter * 32) << 16);
    float* dst = a.part[j] + ((size_t)z * a.B) * N + row;
    for (int c0 = 0; c0 < a.B; c0 += 16) {
      float v[16];
      tmem_load16(taddr + (uint32_t)c0, v);
      if (row < N) {
#pragma unroll
        for (int t = 0; t < 16; ++t)
          if (c0 + t < a.B) dst[(size_t)(c0 + t) * N] = v[t];
      }
    }
    tcgen05_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&ctl->accum_empty[acc]);
  }
}

template <int D>
__global__ void __launch_bounds__(DL_THREADS, DL_CTAS_PER_SM) decode_layers_kernel(const __grid_constant__ Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = a.stages;
  const int stage_bytes = A_TILE_BYTES + a.BN * BLOCK_K * 2;
  Ctl* ctl = (Ctl*)(smem + (size_t)stages * stage_bytes);
  uint8_t* att_smem = smem;   // the attention phase borrows the (then empty) ring
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tmem_cols = 2u * (uint32_t)a.acc_cols;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->accum_full[i], 1);
      mbar_init(&ctl->accum_empty[i], 4);   // one arrival per compute warp
    }
    ctl->failed = 0;
    ctl->opened = 0;
    ctl->att_done = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = ctl->tmem;

  if (warp >= 5) {
    // ----------------------------------------------------------------- TMA producers
    // Issuing a tensor copy costs its thread a few hundred nanoseconds whatever the box's size,
    // more than HBM needs to deliver a weight tile to one SM: DL_PRODUCERS threads (lane 0 of as
    // many warps) share the items, producer p taking items p, p + DL_PRODUCERS, ...
    if (lane == 0) {
      const int p = warp - 5;
      Cursor ca, cb;
      ca.start(a, blockIdx.x, gridDim.x);
      for (int k = 0; k < p && !ca.done; ++k) ca.next_kb(a);
      cb = ca;
      uint32_t ia = p, ib = p, idle = 0;
      int fenced_att = 0, fenced_open = 0;
      long long t_idle = 0;
      while (!cb.done && !ctl->failed) {
        bool progressed = false;
        // The attention phase borrows the ring's memory: weights of the products after it wait
        // until this CTA's attention of that layer is done (the barriers that follow cover their
        // latency), and a next layer's first product until the attention before it is.
        if (!ca.done && ctl->att_done >= ca.layer + (ca.j > 0 ? 1 : 0)) {
          const int s = ia % stages;
          if (mbar_test(&ctl->empty[s], ((ia / stages) & 1u) ^ 1u)) {
            if (fenced_att < ctl->att_done) {
              fenced_att = ctl->att_done;
              __threadfence_block();
              fence_proxy_async();   // the attention's reads and writes of this memory come first
            }
            // weights do not depend on anything computed here: requested as soon as a stage is free
            mbar_expect_tx(&ctl->full[s], (uint32_t)stage_bytes);
            tma_load_2d(smem + (size_t)s * stage_bytes, &a.layers[ca.layer].w[ca.j], &ctl->full[s], ca.kb * BLOCK_K,
                        ca.tile * TILE_A);
            for (int k = 0; k < DL_PRODUCERS && !ca.done; ++k) ca.next_kb(a);
            ia += DL_PRODUCERS;
            progressed = true;
          }
        }
        if (ib < ia) {
          const int need = opens_after(a, cb.layer, cb.j);
          if (ctl->opened >= need) {
            if (fenced_open < need) {   // once per phase: what other CTAs wrote before the barrier, then TMA reads
              __threadfence_block();
              fence_proxy_async();
              fenced_open = need;
            }
            const int s = ib % stages;
            const CUtensorMap* bmap = (cb.j == 1) ? &a.map_xo : (cb.j == 3 ? &a.map_act : &a.map_hw);
            tma_load_2d(smem + (size_t)s * stage_bytes + A_TILE_BYTES, bmap, &ctl->full[s], cb.kb * BLOCK_K, 0);
            for (int k = 0; k < DL_PRODUCERS && !cb.done; ++k) cb.next_kb(a);
            ib += DL_PRODUCERS;
            progressed = true;
          }
        }
        if (progressed) {
          idle = 0;
          continue;
        }
        __nanosleep(32);
        if (++idle == 256) {
          t_idle = clock64();
        } else if (idle > 256 && (idle & 255u) == 0 && clock64() - t_idle > WAIT_CYCLES) {
          fail(a, ctl, 21);
          break;
        }
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(TILE_A, a.BN);
      Cursor c;
      c.start(a, blockIdx.x, gridDim.x);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      while (!c.done && ok) {
        const uint32_t acc = lt & 1u, acc_phase = (lt >> 1) & 1u;
        if (!mbar_wait_timed(&ctl->accum_empty[acc], acc_phase ^ 1u, &ctl->failed)) {
          if (!ctl->failed) fail(a, ctl, 24);
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * (uint32_t)a.acc_cols;
        const int n_kb = c.kb_end - c.kb;
        for (int i = 0; i < n_kb; ++i, ++it) {
          const int s = it % stages;
          if (!mbar_wait_timed(&ctl->full[s], (it / stages) & 1u, &ctl->failed)) {
            if (!ctl->failed) fail(a, ctl, 22);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * stage_bytes);
          const uint32_t b_addr = a_addr + A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
            tcgen05_mma_bf16(d_tmem, smem_desc_sw128(a_addr + k * UMMA_K * 2), smem_desc_sw128(b_addr + k * UMMA_K * 2),
                             idesc, (i > 0 || k > 0) ? 1u : 0u);
          tcgen05_commit(&ctl->empty[s]);   // frees the stage when these MMAs have read it
        }
        if (!ok) break;
        tcgen05_commit(&ctl->accum_full[acc]);
        c.next_unit(a);
        ++lt;
      }
    }
  } else {
    // ---------------------------------------------------------------- compute warps
    const int ctid = threadIdx.x;
    const int P = barriers_per_layer(a);
    const int xo_stride = a.nq * D;
    uint32_t lt = 0;
    const float* pend = a.pend;
    int pend_splits = a.pend ? a.pend_splits : 0;
    bool ok = true;
    for (int layer = 0; layer < a.n_layers && ok; ++layer) {
      const LayerDesc& L = a.layers[layer];
      int nb = layer * P;   // barriers passed so far
      phase_residual(a, ctl, ctid, pend, pend_splits, L.norm1_w, a.ssq);
      if (!(ok = grid_barrier(a, ctl, ctid, ++nb))) break;
      phase_epilogue(a, ctl, 0, tmem_base, warp, lane, lt);
      if (!(ok = grid_barrier(a, ctl, ctid, ++nb))) break;
      {   // attention
        row_scales(a, ctl, ctid, a.ssq, L.eps1);
        const GroupArrays& grp = a.groups[L.kv_group];
        FusedQK fq;
        fq.qkv = nullptr;
        fq.qkv_stride = 0;
        fq.part = a.part[0];
        fq.part_splits = a.splits[0];
        fq.part_zstride = (long long)a.B * a.n_qkv;
        fq.width = a.n_qkv;
        fq.qw = L.q_norm_w;
        fq.kw = L.k_norm_w;
        fq.eps = L.qk_eps;
        fq.cos_t = L.cos_t;
        fq.sin_t = L.sin_t;
        fq.n_table_pos = L.n_table_pos > 0 ? L.n_table_pos : 1;
        fq.positions = a.positions;
        fq.slots = grp.slots;
        fq.kcache_w = L.kcache;
        fq.vcache_w = L.vcache;
        fq.row_scale = ctl->inv;
        const int S = a.att_splits;
        const int units = a.B * a.nkv * S;
        for (int u = blockIdx.x; u < units; u += gridDim.x) {
          const int z = u % S, kvh = (u / S) % a.nkv, dec = u / (S * a.nkv);
          attn_decode_unit<D, true, ComputeSync, AttCfg<D>::STAGES>(att_smem, ctid, dec, kvh, z, a.xo, xo_stride,
                                                 S > 1 ? a.attn_part : nullptr, nullptr, 0, L.kcache, L.vcache,
                                                 grp.block_tables, grp.bt_stride, a.cu_q, a.kv_lens, a.dec_seq, a.nq,
                                                 a.nkv, a.page_size, a.page_shift, L.window, L.scale_log2, S, fq,
                                                 smem + a.fused_off);
          ComputeSync::sync();
        }
        // the ring goes back to the producer
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        ComputeSync::sync();
        if (ctid == 0) {
          __threadfence_block();
          ctl->att_done = layer + 1;
        }
      }
      if (!(ok = grid_barrier(a, ctl, ctid, ++nb))) break;
      if (a.att_splits > 1) {
        const int items = a.B * a.nq;
        for (int item = blockIdx.x; item < items; item += gridDim.x)
          attn_decode_combine_item<D>(item / a.nq, item % a.nq, ctid, DL_COMPUTE, a.xo, xo_stride, a.attn_part, a.cu_q,
                                      a.dec_seq, a.nq, a.nkv, a.att_splits);
        if (!(ok = grid_barrier(a, ctl, ctid, ++nb))) break;
      }
      phase_epilogue(a, ctl, 1, tmem_base, warp, lane, lt);
      if (!(ok = grid_barrier(a, ctl, ctid, ++nb))) break;
      phase_residual(a, ctl, ctid, a.part[1], a.splits[1], L.norm2_w, a.ssq + a.chunks * MAX_TOKENS);
      if (!(ok = grid_barrier(a, ctl, ctid, ++nb))) break;
      phase_epilogue(a, ctl, 2, tmem_base, warp, lane, lt);
      if (!(ok = grid_barrier(a, ctl, ctid, ++nb))) break;
      row_scales(a, ctl, ctid, a.ssq + a.chunks * MAX_TOKENS, L.eps2);
      phase_swiglu(a, ctl, ctid);
      if (!(ok = grid_barrier(a, ctl, ctid, ++nb))) break;
      phase_epilogue(a, ctl, 3, tmem_base, warp, lane, lt);
      if (layer + 1 < a.n_layers && !(ok = grid_barrier(a, ctl, ctid, ++nb))) break;
      pend = a.part[3];
      pend_splits = a.splits[3];
    }
    cp_async_wait<0>();
  }
  __syncwarp();
  if (ctl->failed) {
    // let copies that may still be in flight land before shared memory is given up
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 4) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ------------------------------------------------------------------------ host side
int round_bn(int b) { return b <= 16 ? 16 : (b <= 32 ? 32 : 64); }

// Split count of a product with `tiles` row tiles and `kb` k-blocks: the one (at most 16, at
// least two k-blocks per split) whose units fill `grid` CTAs most evenly; the smallest on a tie.
int choose_splits(int tiles, int kb, int grid) {
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= 16 && s * 2 <= (kb > 1 ? kb : 2); ++s) {
    const int units = tiles * s;
    const int rounds = (units + grid - 1) / grid;
    const double eff = (double)units / ((double)rounds * grid);
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = s;
    }
  }
  return best;
}

int choose_att_splits(int B, int nkv, int grid) {
  int s = grid / (B * nkv > 0 ? B * nkv : 1);
  return s < 1 ? 1 : (s > 16 ? 16 : s);
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Layout {
  int splits[4], tiles[4], kb[4], n[4], k[4];
  int chunks;
  size_t off_counter, off_hw, off_xo, off_act, off_ssq, off_part[4], off_attn, total;
};

Layout make_layout(int hidden, int nq, int nkv, int d, int inter, int grid) {
  Layout l;
  const int n[4] = {(nq + 2 * nkv) * d, hidden, 2 * inter, hidden};
  const int k[4] = {hidden, nq * d, hidden, inter};
  for (int j = 0; j < 4; ++j) {
    l.n[j] = n[j];
    l.k[j] = k[j];
    l.tiles[j] = (n[j] + TILE_A - 1) / TILE_A;
    l.kb[j] = (k[j] + BLOCK_K - 1) / BLOCK_K;
    l.splits[j] = choose_splits(l.tiles[j], l.kb[j], grid);
  }
  l.chunks = (hidden + CHUNK - 1) / CHUNK;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = align_up(off + bytes, 1024);
    return at;
  };
  l.off_counter = take(1024);
  l.off_hw = take((size_t)MAX_TOKENS * hidden * 2);
  l.off_xo = take((size_t)MAX_TOKENS * nq * d * 2);
  l.off_act = take((size_t)MAX_TOKENS * inter * 2);
  l.off_ssq = take((size_t)2 * l.chunks * MAX_TOKENS * 4);
  for (int j = 0; j < 4; ++j) l.off_part[j] = take((size_t)l.splits[j] * MAX_TOKENS * n[j] * 4);
  size_t attn = 0;
  for (int b = 1; b <= MAX_TOKENS; ++b) {
    const int s = choose_att_splits(b, nkv, grid);
    const size_t need = s > 1 ? (size_t)b * nq * s * (d + 2) * 4 : 0;
    attn = need > attn ? need : attn;
  }
  l.off_attn = take(attn > 0 ? attn : 4);
  l.total = off;
  return l;
}

size_t attention_smem(int d) {
  const int st = d <= 64 ? AttCfg<64>::STAGES : AttCfg<128>::STAGES;
  return (size_t)DC_WARPS * st * 2 * DC_KEYS * d * 2;   // the rings
}
size_t attention_fused_bytes(int d) { return (size_t)16 * d * 2 + (2 * d + 16) * sizeof(float); }

// Shared memory of a CTA: [ring][Ctl][the attention's small arrays, unless they fit behind its
// rings inside the ring's memory].  stages == 0: does not fit.
struct SmemPlan {
  int stages;
  size_t fused_off, total;
};
SmemPlan plan_smem(int d, int BN) {
  SmemPlan p = {0, 0, 0};
  const size_t stage = A_TILE_BYTES + (size_t)BN * BLOCK_K * 2;
  const size_t ctl = ((sizeof(Ctl) + 127) / 128) * 128 + 128;
  for (int st = MAX_STAGES; st >= 2; --st) {
    const size_t ring = (size_t)st * stage;
    if (ring < attention_smem(d)) break;
    const bool inside = ring >= attention_smem(d) + attention_fused_bytes(d);
    const size_t total = 1024 + ring + ctl + (inside ? 0 : attention_fused_bytes(d));
    if (total > DL_SMEM_BUDGET) continue;
    p.stages = st;
    p.fused_off = inside ? attention_smem(d) : ring + ctl;
    p.total = total;
    return p;
  }
  return p;
}

}  // namespace

extern "C" int zi_decode_layers_supported(int hidden, int nq, int nkv, int d, int inter) {
  if (!(d == 64 || d == 128)) return 0;
  if (nkv <= 0 || nq % nkv || nq / nkv > 16) return 0;
  if (hidden % 8 || inter % 8 || hidden <= 0 || inter <= 0) return 0;
  return (plan_smem(d, 16).stages >= 2 && plan_smem(d, 32).stages >= 2 && plan_smem(d, 64).stages >= 2) ? 1 : 0;
}

extern "C" long long zi_decode_layers_desc_bytes() { return (long long)sizeof(LayerDesc); }

// CTAs of a launch on a device with `sm_count` SMs (the `grid` of the calls below).
extern "C" int zi_decode_layers_grid(int sm_count) { return sm_count * DL_CTAS_PER_SM; }

// out[0..2]: workspace bytes, byte offset of the last product's partial sums, its split count;
// out[3..15]: for inspection, the byte offsets of hw, xo, act, ssq, the four products' partial sums
// and the attention's, then the four split counts.
extern "C" int zi_decode_layers_layout(int hidden, int nq, int nkv, int d, int inter, int grid, long long* out) {
  if (!zi_decode_layers_supported(hidden, nq, nkv, d, inter)) return zi_refuse("decode_layers: these sizes are not supported");
  const Layout l = make_layout(hidden, nq, nkv, d, inter, grid);
  out[0] = (long long)l.total;
  out[1] = (long long)l.off_part[3];
  out[2] = l.splits[3];
  out[3] = (long long)l.off_hw;
  out[4] = (long long)l.off_xo;
  out[5] = (long long)l.off_act;
  out[6] = (long long)l.off_ssq;
  for (int j = 0; j < 4; ++j) {
    out[7 + j] = (long long)l.off_part[j];
    out[12 + j] = l.splits[j];
  }
  out[11] = (long long)l.off_attn;
  return 0;
}

// Fills one layer's descriptor in host memory (the caller copies the table to the device).
extern "C" int zi_decode_layers_fill_desc(void* desc, const void* w_qkv, const void* w_o, const void* w_gu,
                                          const void* w_down, int hidden, int nq, int nkv, int d, int inter,
                                          const float* norm1_w, const float* norm2_w, float eps1, float eps2,
                                          const float* q_norm_w, const float* k_norm_w, float qk_eps, void* kcache,
                                          void* vcache, const float* cos_t, const float* sin_t, int n_table_pos,
                                          int window, int kv_group, float scale) {
  if (!zi_decode_layers_supported(hidden, nq, nkv, d, inter)) return zi_refuse("decode_layers: these sizes are not supported");
  if (kv_group < 0 || kv_group >= MAX_GROUPS) return zi_refuse("decode_layers: cache group %d of at most %d", kv_group, MAX_GROUPS);
  if ((cos_t == nullptr) != (sin_t == nullptr)) return zi_refuse("decode_layers: cos and sin tables go together");
  LayerDesc* L = (LayerDesc*)desc;
  memset(L, 0, sizeof(LayerDesc));
  const void* w[4] = {w_qkv, w_o, w_gu, w_down};
  const int n[4] = {(nq + 2 * nkv) * d, hidden, 2 * inter, hidden};
  const int k[4] = {hidden, nq * d, hidden, inter};
  for (int j = 0; j < 4; ++j) {
    if ((uintptr_t)w[j] % 16) return zi_refuse("decode_layers: weights must be 16-byte aligned");
    if (!zi_internal_make_map(&L->w[j], w[j], n[j], k[j], k[j], TILE_A)) return zi_refuse("decode_layers: cannot make a tensor map");
  }
  L->norm1_w = norm1_w;
  L->norm2_w = norm2_w;
  L->q_norm_w = q_norm_w;
  L->k_norm_w = k_norm_w;
  L->kcache = (bf16*)kcache;
  L->vcache = (bf16*)vcache;
  L->cos_t = cos_t;
  L->sin_t = sin_t;
  L->eps1 = eps1;
  L->eps2 = eps2;
  L->qk_eps = qk_eps;
  L->scale_log2 = scale * 1.4426950408889634f;
  L->n_table_pos = n_table_pos;
  L->window = window;
  L->kv_group = kv_group;
  return 0;
}

// Runs `n_layers` layers (descriptors `descs` on the device) on the B tokens of a decode step.
// h [B, hidden] is updated in place up to the last layer's attention; the last feed-forward's
// update is left as split-K partial sums in the workspace (see zi_decode_layers_layout) for
// the next norm to add.  `pend`: partial sums [pend_splits][B][hidden] not yet added to h.
// group_slots / group_tables / group_strides: per cache group of the step.
extern "C" int zi_decode_layers(const void* descs, int n_layers, int B, int hidden, int nq, int nkv, int d, int inter,
                                int interleave, float* h, const float* pend, int pend_splits, void* workspace,
                                long long workspace_bytes, const int* positions, const int* cu_q, const int* kv_lens,
                                const int* dec_seq, int n_groups, const int* const* group_slots,
                                const int* const* group_tables, const int* group_strides, int page_size, int grid,
                                cudaStream_t stream) {
  if (n_layers <= 0 || B <= 0) return 0;
  if (B > MAX_TOKENS) return zi_refuse("decode_layers: %d tokens (at most %d)", B, MAX_TOKENS);
  if (!zi_decode_layers_supported(hidden, nq, nkv, d, inter)) return zi_refuse("decode_layers: these sizes are not supported");
  if (interleave && (interleave % 2 || inter % interleave)) return zi_refuse("decode_layers: interleave %d does not fit %d", interleave, inter);
  if (n_groups < 1 || n_groups > MAX_GROUPS) return zi_refuse("decode_layers: %d cache groups (1..%d)", n_groups, MAX_GROUPS);
  if (grid < 1) return zi_refuse("decode_layers: empty grid");
  const Layout l = make_layout(hidden, nq, nkv, d, inter, grid);
  if ((size_t)workspace_bytes < l.total || (uintptr_t)workspace % 1024)
    return zi_refuse("decode_layers: the workspace needs %zu bytes, 1024-byte aligned", l.total);
  int* status = zi_internal_status_word();
  if (!status) return zi_refuse("decode_layers: cannot allocate the status word");
  uint8_t* ws = (uint8_t*)workspace;

  Args a;
  memset(&a, 0, sizeof(a));
  a.BN = round_bn(B);
  a.hw = (bf16*)(ws + l.off_hw);
  a.xo = (bf16*)(ws + l.off_xo);
  a.act = (bf16*)(ws + l.off_act);
  if (!zi_internal_make_map(&a.map_hw, a.hw, MAX_TOKENS, hidden, hidden, a.BN) ||
      !zi_internal_make_map(&a.map_xo, a.xo, MAX_TOKENS, nq * d, nq * d, a.BN) ||
      !zi_internal_make_map(&a.map_act, a.act, MAX_TOKENS, inter, inter, a.BN))
    return zi_refuse("decode_layers: cannot make a tensor map");
  a.layers = (const LayerDesc*)descs;
  a.n_layers = n_layers;
  a.B = B;
  const SmemPlan sp = plan_smem(d, a.BN);
  a.stages = sp.stages;
  a.fused_off = (int)sp.fused_off;
  a.acc_cols = a.BN < 32 ? 32 : a.BN;
  a.hidden = hidden;
  a.nq = nq;
  a.nkv = nkv;
  a.inter = inter;
  a.n_qkv = l.n[0];
  a.n_gu = l.n[2];
  a.interleave = interleave;
  for (int j = 0; j < 4; ++j) {
    a.n[j] = l.n[j];
    a.k[j] = l.k[j];
    a.tiles[j] = l.tiles[j];
    a.kb[j] = l.kb[j];
    a.splits[j] = l.splits[j];
    a.part[j] = (float*)(ws + l.off_part[j]);
  }
  a.att_splits = choose_att_splits(B, nkv, grid);
  a.page_size = page_size;
  a.page_shift = log2_or_minus1(page_size);
  a.chunks = l.chunks;
  a.h = h;
  a.pend = pend;
  a.pend_splits = pend ? pend_splits : 0;
  a.ssq = (float*)(ws + l.off_ssq);
  a.attn_part = (float*)(ws + l.off_attn);
  a.positions = positions;
  a.cu_q = cu_q;
  a.kv_lens = kv_lens;
  a.dec_seq = dec_seq;
  for (int gi = 0; gi < n_groups; ++gi) {
    a.groups[gi].slots = group_slots[gi];
    a.groups[gi].block_tables = group_tables[gi];
    a.groups[gi].bt_stride = group_strides[gi];
  }
  a.counter = (unsigned*)(ws + l.off_counter);
  a.status = status;

  const size_t smem = sp.total;
  auto kern = d == 64 ? decode_layers_kernel<64> : decode_layers_kernel<128>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return zi_refuse("decode_layers: cannot get %zu bytes of shared memory", smem);
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  // every CTA must be resident at once (they meet at grid barriers)
  // (The runtime's occupancy query answers 1 for this kernel whatever its size; the count is made here
  // from the same resources: registers, shared memory with its 1 KB per block, threads.)
  cudaFuncAttributes fa;
  int dev = 0, sms = 0, regs_sm = 0, smem_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, dev);
  cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
  if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess) return zi_refuse("decode_layers: cannot read the kernel's attributes");
  const int warps = (DL_THREADS + 31) / 32;
  const long long regs_block = (long long)((fa.numRegs + 7) / 8 * 8) * 32 * ((warps + 3) / 4 * 4);
  const bool fits = regs_block * DL_CTAS_PER_SM <= regs_sm &&
                    (long long)(smem + fa.sharedSizeBytes + 1024) * DL_CTAS_PER_SM <= smem_sm;
  if (!fits || grid > sms * DL_CTAS_PER_SM)
    return zi_refuse("decode_layers: %d blocks (%d registers, %zu bytes of shared memory each) cannot be resident at once on %d SMs",
                     grid, fa.numRegs, smem, sms);
  e = cudaMemsetAsync(a.counter, 0, sizeof(unsigned), stream);
  if (e != cudaSuccess) return zi_refuse("decode_layers: cannot clear the barrier counter: %s", cudaGetErrorString(e));
  // a plain launch (no programmatic early start): the kernel before it has drained, so every SM is free
  kern<<<grid, DL_THREADS, smem, stream>>>(a);
  return zi_check_launch("decode_layers");
}
