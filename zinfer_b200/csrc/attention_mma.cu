// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16,
// 32-bit accumulation, online softmax in 32-bit), for head sizes 64 and 128
// (decode also 256).  Two kernels share the tile code:
//
//  * prefill: a CTA takes 128 query tokens of one request and one query head; its
//    8 warps own 16 query rows each and walk the keys in tiles of 64, double-buffered
//    with cp.async.  Causal and window masks are applied only on tiles that need them.
//  * decode: a CTA takes one request's single query token, one kv head (all the
//    query heads of its group are the 16 rows of the MMA) and one split of the keys;
//    its 4 warps each stream their own 16 keys per tile through a private cp.async
//    ring (no block-wide barrier in the loop) and merge at the end.  With more than
//    one split, partial (max, sum, output) go to a workspace and a second kernel
//    combines them in split order.
//
// Keys and values lie in pages [page][kv head][offset][d]; shared-memory tiles are
// [key][d] with the 16-byte chunks of a row XOR-swizzled by (key & 7) so that
// ldmatrix reads are free of bank conflicts.  Keys outside the request (beyond its
// length, in pages it does not hold) are zero-filled and masked.
#include <string.h>

#include "api.h"
#include "common.cuh"
#include "gemm_internal.h"
#include "attention_tiles.cuh"

namespace {
// =============================================================================== prefill
constexpr int PF_BQ = 128, PF_BK = 64, PF_THREADS = 256;

template <int D>
__global__ void __launch_bounds__(PF_THREADS, 2)
attn_prefill_mma_kernel(bf16* __restrict__ out, int out_stride, const bf16* __restrict__ q, int q_stride,
                        const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                        const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_q,
                        const int* __restrict__ kv_lens, const int* __restrict__ tile_seq,
                        const int* __restrict__ tile_q0, int nq, int nkv, int page_size, int page_shift,
                        int window, float scale_log2) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* qs = smem;                                   // [128][D]
  uint8_t* kbuf = qs + PF_BQ * D * 2;                   // [2][64][D]
  uint8_t* vbuf = kbuf + 2 * PF_BK * D * 2;             // [2][64][D]
  constexpr int TILE_BYTES = PF_BK * D * 2;

  const int seq = tile_seq[blockIdx.y], q0 = tile_q0[blockIdx.y];
  const int h = blockIdx.x, kvh = h / (nq / nkv);   // heads vary fastest: neighbours share K and V in L2
  const int tok0 = cu_q[seq], qlen = cu_q[seq + 1] - tok0, kvlen = kv_lens[seq];
  const int ctx = kvlen - qlen;
  const int nqv = min(PF_BQ, qlen - q0);
  if (nqv <= 0) return;
  const int first_pos = ctx + q0, last_pos = first_pos + nqv - 1;
  const int kv_lo = window > 0 ? max(0, first_pos - window + 1) : 0;
  const int kv_hi = last_pos + 1;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* bt = block_tables + (size_t)seq * bt_stride;

  // Q tile -> shared memory (rows beyond the request's tokens are zero)
  for (int e = tid; e < PF_BQ * (D / 8); e += PF_THREADS) {
    const int r = e / (D / 8), c = e % (D / 8);
    const bool valid = r < nqv;
    const bf16* src = q + (size_t)(tok0 + q0 + (valid ? r : 0)) * q_stride + (size_t)h * D + c * 8;
    cp_async16(qs + swz<D>(r, c), src, valid);
  }
  const int kt0 = (kv_lo / PF_BK) * PF_BK;
  const int n_tiles = (kv_hi - kt0 + PF_BK - 1) / PF_BK;

  // Each thread copies NPER 16-byte chunks of K and of V per tile: rows r_i = tid / CH +
  // i * (256 / CH), column c = tid % CH.  The pages of its rows are looked up one tile
  // ahead, so the block-table load is not waited for when the copies are issued.
  constexpr int CH = D / 8, NPER = PF_BK * CH / PF_THREADS, RSTEP = PF_THREADS / CH;
  const int my_r = tid / CH, my_c = tid % CH;
  int pg[NPER];
  auto lookup = [&](int kt) {
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
      const int j = kt + my_r + i * RSTEP;
      pg[i] = (j >= kv_lo && j < kv_hi) ? __ldg(bt + (page_shift >= 0 ? (j >> page_shift) : (j / page_size))) : -1;
    }
  };
  auto issue = [&](int kt, int buf) {
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
      const int r = my_r + i * RSTEP, j = kt + r;
      const bool valid = pg[i] >= 0;
      const int in_page = page_shift >= 0 ? (j & (page_size - 1)) : (j % page_size);
      const size_t off = valid ? (((size_t)pg[i] * nkv + kvh) * page_size + in_page) * D + my_c * 8 : 0;
      const uint32_t so = swz<D>(r, my_c);
      cp_async16(kbuf + buf * TILE_BYTES + so, kcache + off, valid);
      cp_async16(vbuf + buf * TILE_BYTES + so, vcache + off, valid);
    }
  };
  lookup(kt0);
  issue(kt0, 0);
  cp_async_commit();
  if (n_tiles > 1) lookup(kt0 + PF_BK);

  float o[D / 8][4];
#pragma unroll
  for (int t = 0; t < D / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int row_lo = warp * 16 + (lane >> 2);           // this thread's rows: row_lo and row_lo + 8
  const int warp_first_pos = first_pos + warp * 16, warp_last_pos = min(last_pos, warp_first_pos + 15);
  const bool warp_active = warp * 16 < nqv;
  const uint32_t qs_addr = smem_addr(qs);

  for (int t = 0; t < n_tiles; ++t) {
    const int kt = kt0 + t * PF_BK;
    const int buf = t & 1;
    if (t + 1 < n_tiles) {
      issue(kt + PF_BK, buf ^ 1);
      cp_async_commit();
      if (t + 2 < n_tiles) lookup(kt + 2 * PF_BK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // a warp whose rows all lie before this tile (causal) or after it (window) has nothing to do
    const bool tile_visible = warp_active && kt <= warp_last_pos &&
                              (window <= 0 || kt + PF_BK - 1 > warp_first_pos - window);
    if (tile_visible) {
      const uint32_t ks_addr = smem_addr(kbuf + buf * TILE_BYTES), vs_addr = smem_addr(vbuf + buf * TILE_BYTES);
      float s[PF_BK / 8][4];
#pragma unroll
      for (int nt = 0; nt < PF_BK / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      // S = Q K^T; the Q fragments are re-read from shared memory for every 16 dims (keeps
      // the register count low enough for two CTAs per SM)
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t qf[4];
        const int mtx = lane >> 3;
        ldmatrix_x4(qf, qs_addr + swz<D>(warp * 16 + (mtx & 1) * 8 + (lane & 7), kk * 2 + (mtx >> 1)));
#pragma unroll
        for (int kp = 0; kp < PF_BK / 16; ++kp) {
          uint32_t bfr[4];
          ldmatrix_x4(bfr, ks_addr + swz<D>(kp * 16 + (mtx >> 1) * 8 + (lane & 7), kk * 2 + (mtx & 1)));
          mma_bf16(s[2 * kp], qf, bfr[0], bfr[1]);
          mma_bf16(s[2 * kp + 1], qf, bfr[2], bfr[3]);
        }
      }
      const bool need_mask = kt + PF_BK - 1 > warp_first_pos || window > 0 || kt < kv_lo;
#pragma unroll
      for (int nt = 0; nt < PF_BK / 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float v = s[nt][c] * scale_log2;
          if (need_mask) {
            const int j = kt + nt * 8 + 2 * (lane & 3) + (c & 1);
            const int pos = first_pos + row_lo + (c >> 1) * 8;
            const bool vis = j <= pos && j >= kv_lo && (window <= 0 || j > pos - window);
            if (!vis) v = -INFINITY;
          }
          s[nt][c] = v;
        }
      }
      softmax_step<PF_BK / 8, D / 8>(s, o, m, l);
#pragma unroll
      for (int kp = 0; kp < PF_BK / 16; ++kp) {
        uint32_t pf[4] = {pack_bf16(s[2 * kp][0], s[2 * kp][1]), pack_bf16(s[2 * kp][2], s[2 * kp][3]),
                          pack_bf16(s[2 * kp + 1][0], s[2 * kp + 1][1]), pack_bf16(s[2 * kp + 1][2], s[2 * kp + 1][3])};
        pv_16keys<D>(o, pf, vs_addr, kp * 16, lane);
      }
    }
    __syncthreads();  // the other buffer is refilled in the next iteration
  }

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float sum = l[i];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const int r = row_lo + i * 8;
    if (r < nqv) {
      const float inv = 1.0f / sum;
      bf16* orow = out + (size_t)(tok0 + q0 + r) * out_stride + (size_t)h * D + 2 * (lane & 3);
#pragma unroll
      for (int t = 0; t < D / 8; ++t)
        *reinterpret_cast<uint32_t*>(orow + t * 8) = pack_bf16(o[t][2 * i] * inv, o[t][2 * i + 1] * inv);
    }
  }
}

// ================================================================================ decode
struct BlockSync {
  static __device__ __forceinline__ void sync() { __syncthreads(); }
};

template <int D, bool FUSED, bool TR, bool TMA>
__global__ void __launch_bounds__(DC_THREADS)
attn_decode_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       int* __restrict__ status, bf16* __restrict__ out, int out_stride, float* __restrict__ partial,
                       const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kcache,
                       const bf16* __restrict__ vcache, const int* __restrict__ block_tables, int bt_stride,
                       const int* __restrict__ cu_q, const int* __restrict__ kv_lens,
                       const int* __restrict__ dec_seq, int nq, int nkv, int page_size, int page_shift, int window,
                       float scale_log2, int splits, const FusedQK fq) {
  pdl_launch_dependents();
  // (the unit waits for the kernel before this one itself, after it has asked for its first keys)
  extern __shared__ __align__(128) uint8_t smem_raw[];
  // tiles that TMA fills with the 128-byte swizzle start on 1024-byte boundaries
  uint8_t* smem = TMA ? (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023) : smem_raw;
  constexpr int RING_BYTES = DC_WARPS * DecodeCfg<D>::STAGES * 2 * DC_KEYS * D * 2;
  constexpr int FUSED_BYTES = FUSED ? 16 * D * 2 + (2 * D + 16) * (int)sizeof(float) : 0;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + RING_BYTES + ((FUSED_BYTES + 15) & ~15));
  attn_decode_unit<D, FUSED, BlockSync, DecodeCfg<D>::STAGES, TR, TMA>(
      smem, threadIdx.x, blockIdx.x, blockIdx.y, blockIdx.z, out, out_stride, partial, q, q_stride, kcache, vcache,
      block_tables, bt_stride, cu_q, kv_lens, dec_seq, nq, nkv, page_size, page_shift, window, scale_log2, splits, fq,
      nullptr, &map_k, &map_v, bars, status);
}

template <int D>
__global__ void attn_decode_combine_kernel(bf16* __restrict__ out, int out_stride, const float* __restrict__ partial,
                                           const int* __restrict__ cu_q, const int* __restrict__ dec_seq, int nq,
                                           int nkv, int splits) {
  pdl_launch_dependents();
  // which token this is comes from the step's own arrays (copied before any kernel of the step):
  // these two dependent loads need not wait for the attention kernel
  const int token = cu_q[dec_seq[blockIdx.x]];
  pdl_wait();
  attn_decode_combine_item<D>(blockIdx.x, blockIdx.y, threadIdx.x, blockDim.x, out, out_stride, partial, token, nq, nkv,
                              splits);
}


template <int D>
int launch_prefill(void* out, int out_stride, const void* q, int q_stride, const void* kc, const void* vc,
                   const int* bt, int bt_stride, const int* cu_q, const int* kv_lens, const int* tile_seq,
                   const int* tile_q0, int n_tiles, int nq, int nkv, int page_size, int window, float scale,
                   cudaStream_t stream) {
  auto kern = attn_prefill_mma_kernel<D>;
  const size_t smem = (size_t)(PF_BQ + 4 * PF_BK) * D * 2;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return zi_refuse("attention_prefill: cannot get %zu bytes of shared memory", smem);
  dim3 grid(nq, n_tiles);
  zi_launch(kern, dim3(grid), dim3(PF_THREADS), smem, stream, (bf16*)out, out_stride, (const bf16*)q, q_stride, (const bf16*)kc,
                                           (const bf16*)vc, bt, bt_stride, cu_q, kv_lens, tile_seq, tile_q0, nq, nkv,
                                           page_size, log2_or_minus1(page_size), window, scale * 1.4426950408889634f);
  return zi_check_launch("attention_prefill");
}

int g_decode_transposed = 1;   // zi_attention_decode_transposed(0) switches the transposed tile off (for comparisons)

int g_decode_tma = 1;          // see zi_attention_decode_tma

template <int D, bool FUSED, bool TR, bool TMA>
int launch_decode_as(void* out, int out_stride, float* partial, const void* q, int q_stride, const void* kc,
                     const void* vc, long long n_pages, const int* bt, int bt_stride, const int* cu_q,
                     const int* kv_lens, const int* dec_seq, int n_dec, int nq, int nkv, int page_size, int window,
                     float scale, int splits, const FusedQK& fq, cudaStream_t stream) {
  auto kern = attn_decode_mma_kernel<D, FUSED, TR, TMA>;
  CUtensorMap map_k, map_v;
  memset(&map_k, 0, sizeof(map_k));
  memset(&map_v, 0, sizeof(map_v));
  int* status = nullptr;
  if (TMA) {
    const long long rows = n_pages * nkv * page_size;
    const int box_rows = page_size >= 16 ? 16 : page_size;
    if (!zi_internal_make_map(&map_k, kc, (int)rows, D, D, box_rows) || !zi_internal_make_map(&map_v, vc, (int)rows, D, D, box_rows))
      return zi_refuse("attention_decode: cuTensorMapEncodeTiled failed");
    status = zi_internal_status_word();
    if (!status) return zi_refuse("attention_decode: cannot allocate the status word");
  }
  const size_t ring = (size_t)DC_WARPS * DecodeCfg<D>::STAGES * 2 * DC_KEYS * D * 2;
  const size_t fused = FUSED ? (size_t)16 * D * 2 + (2 * D + 16) * sizeof(float) : 0;
  const size_t smem = ring + ((fused + 15) & ~(size_t)15) + (TMA ? (size_t)DC_WARPS * DecodeCfg<D>::STAGES * 8 + 1024 : 0);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return zi_refuse("attention_decode: cannot get %zu bytes of shared memory", smem);
  dim3 grid(n_dec, nkv, splits);
  zi_launch(kern, dim3(grid), dim3(DC_THREADS), smem, stream, map_k, map_v, status, (bf16*)out, out_stride,
            splits > 1 ? partial : nullptr, (const bf16*)q, q_stride, (const bf16*)kc, (const bf16*)vc, bt, bt_stride, cu_q,
            kv_lens, dec_seq, nq, nkv, page_size, log2_or_minus1(page_size), window, scale * 1.4426950408889634f, splits, fq);
  return 0;
}

template <int D, bool FUSED>
int launch_decode(void* out, int out_stride, float* partial, const void* q, int q_stride, const void* kc,
                  const void* vc, long long n_pages, const int* bt, int bt_stride, const int* cu_q, const int* kv_lens,
                  const int* dec_seq, int n_dec, int nq, int nkv, int page_size, int window, float scale, int splits,
                  const FusedQK& fq, cudaStream_t stream) {
  // Groups of at most 8 query heads take the transposed tile (keys on the MMA's rows).  Keys and values come by
  // TMA (page boxes, pages of 8, 16, 32, ... tokens whose rows a tensor map can address) while the requests
  // are few, and by cp.async from every lane when they are many.  Measured per 36-layer step (Qwen3-8B
  // sizes, 2,048 keys): TMA 3.285 against 3.295 ms at 1 request and 3.66 against 3.68 at 8, but 4.47 against
  // 4.42 at 24 and 6.79 against 6.74 at 64: where the kernel is bound by memory, 32 lanes asking for 16 bytes
  // each keep slightly more in flight than boxes of 2 KB (g_decode_tma: 0 never, 1 by this rule, 2 always).
  const bool tr = nq / nkv <= 8 && g_decode_transposed;
  const int shift = log2_or_minus1(page_size);
  const bool tma = g_decode_tma && (g_decode_tma == 2 || n_dec <= 16) && shift >= 3 && n_pages > 0 &&
                   n_pages * nkv * page_size <= 0x7fffffffll && (uintptr_t)kc % 16 == 0 && (uintptr_t)vc % 16 == 0;
#define ZI_DECODE_AS(TR_, TMA_)                                                                                        \
  launch_decode_as<D, FUSED, TR_, TMA_>(out, out_stride, partial, q, q_stride, kc, vc, n_pages, bt, bt_stride, cu_q, kv_lens, \
                                        dec_seq, n_dec, nq, nkv, page_size, window, scale, splits, fq, stream)
  int rc0 = tr ? (tma ? ZI_DECODE_AS(true, true) : ZI_DECODE_AS(true, false))
               : (tma ? ZI_DECODE_AS(false, true) : ZI_DECODE_AS(false, false));
#undef ZI_DECODE_AS
  if (rc0) return rc0;
  int rc = zi_check_launch("attention_decode");
  if (rc) return rc;
  if (splits > 1) {
    zi_launch(attn_decode_combine_kernel<D>, dim3(n_dec, nq), dim3(D >= 128 ? 128 : 64), 0, stream, (bf16*)out,
              out_stride, partial, cu_q, dec_seq, nq, nkv, splits);
    rc = zi_check_launch("attention_decode_combine");
  }
  return rc;
}

template <bool FUSED>
int dispatch_decode(int d, void* out, int out_stride, float* partial, const void* q, int q_stride, const void* kc,
                    const void* vc, long long n_pages, const int* bt, int bt_stride, const int* cu_q, const int* kv_lens,
                    const int* dec_seq, int n_dec, int nq, int nkv, int page_size, int window, float scale, int splits,
                    const FusedQK& fq, cudaStream_t stream) {
  if (d == 64)
    return launch_decode<64, FUSED>(out, out_stride, partial, q, q_stride, kc, vc, n_pages, bt, bt_stride, cu_q, kv_lens, dec_seq,
                                    n_dec, nq, nkv, page_size, window, scale, splits, fq, stream);
  if (d == 128)
    return launch_decode<128, FUSED>(out, out_stride, partial, q, q_stride, kc, vc, n_pages, bt, bt_stride, cu_q, kv_lens,
                                     dec_seq, n_dec, nq, nkv, page_size, window, scale, splits, fq, stream);
  return launch_decode<256, FUSED>(out, out_stride, partial, q, q_stride, kc, vc, n_pages, bt, bt_stride, cu_q, kv_lens, dec_seq,
                                   n_dec, nq, nkv, page_size, window, scale, splits, fq, stream);
}
}  // namespace

extern "C" int zi_attention_prefill_tile_rows() { return PF_BQ; }

// The decode attention's tile for groups of at most 8 query heads: transposed (1, the default) or
// row-major as for larger groups (0); returns the setting before.  For tests and timing comparisons.
// Keys and values of the decode attention by TMA: 1 (the default) for up to 16 requests, 2 always, 0 never
// (cp.async from every lane); returns the setting before.  For tests and timing comparisons.
extern "C" int zi_attention_decode_tma(int mode) {
  const int before = g_decode_tma;
  g_decode_tma = mode < 0 ? 0 : (mode > 2 ? 2 : mode);
  return before;
}

extern "C" int zi_attention_decode_transposed(int on) {
  const int before = g_decode_transposed;
  g_decode_transposed = on ? 1 : 0;
  return before;
}

// Whether the tensor-core kernels take this shape (else the caller uses zi_paged_attention).
extern "C" int zi_attention_mma_supported(int nq, int nkv, int d, int decode) {
  if (nkv <= 0 || nq % nkv) return 0;
  if (decode) return (d == 64 || d == 128 || d == 256) && nq / nkv <= 16;
  return d == 64 || d == 128;
}

extern "C" int zi_attention_prefill_mma(void* out, int out_stride, const void* q, int q_stride, const void* kcache,
                                        const void* vcache, const int* block_tables, int bt_stride, const int* cu_q,
                                        const int* kv_lens, const int* tile_seq, const int* tile_q0, int n_tiles,
                                        int nq, int nkv, int d, int page_size, int window, float scale,
                                        cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!zi_attention_mma_supported(nq, nkv, d, 0)) return zi_refuse("attention_prefill: head_dim %d is not 64 or 128", d);
  if (q_stride % 8 || ((uintptr_t)q % 16)) return zi_refuse("attention_prefill: q rows must be 16-byte aligned");
  if (d == 64)
    return launch_prefill<64>(out, out_stride, q, q_stride, kcache, vcache, block_tables, bt_stride, cu_q, kv_lens,
                              tile_seq, tile_q0, n_tiles, nq, nkv, page_size, window, scale, stream);
  return launch_prefill<128>(out, out_stride, q, q_stride, kcache, vcache, block_tables, bt_stride, cu_q, kv_lens,
                             tile_seq, tile_q0, n_tiles, nq, nkv, page_size, window, scale, stream);
}

// Floats of workspace a decode launch with `splits` > 1 needs.
extern "C" long long zi_attention_decode_workspace_floats(int n_dec, int nq, int nkv, int d, int splits) {
  return splits > 1 ? (long long)n_dec * nq * splits * (d + 2) : 0;
}

// n_pages: pages of each cache (their rows are addressed through a tensor map when they come by TMA).
extern "C" int zi_attention_decode_mma(void* out, int out_stride, float* workspace, const void* q, int q_stride,
                                       const void* kcache, const void* vcache, long long n_pages, const int* block_tables,
                                       int bt_stride, const int* cu_q, const int* kv_lens, const int* dec_seq,
                                       int n_dec, int nq, int nkv, int d, int page_size, int window, float scale,
                                       int splits, cudaStream_t stream) {
  if (n_dec <= 0) return 0;
  if (!zi_attention_mma_supported(nq, nkv, d, 1))
    return zi_refuse("attention_decode: head_dim %d (64, 128, 256) or group size %d (<= 16) is not supported", d, nq / nkv);
  if (splits < 1 || (splits > 1 && !workspace)) return zi_refuse("attention_decode: %d splits need a workspace", splits);
  if (q_stride % 2) return zi_refuse("attention_decode: q rows must be 4-byte aligned");
  FusedQK none = {};
  return dispatch_decode<false>(d, out, out_stride, workspace, q, q_stride, kcache, vcache, n_pages, block_tables, bt_stride, cu_q,
                                kv_lens, dec_seq, n_dec, nq, nkv, page_size, window, scale, splits, none, stream);
}

// Decode attention that also makes q, k and v of each request's token from the fused
// projection row (per-head RMSNorm when weights are given, rotary when tables are given) and
// writes k and v into their page slots: qk_norm_rope_store and attention in one kernel.  The
// row comes either as bfloat16 `qkv` or as split-K partial sums `partials`.
extern "C" int zi_attention_decode_fused(void* out, int out_stride, float* workspace, const void* qkv, int qkv_stride,
                                         const float* partials, int part_splits, long long part_zstride,
                                         const float* qw, const float* kw, float eps, const float* cos_t,
                                         const float* sin_t, int n_table_pos, const int* positions,
                                         const int* slots, void* kcache, void* vcache, long long n_pages,
                                         const int* block_tables, int bt_stride, const int* cu_q, const int* kv_lens, const int* dec_seq,
                                         int n_dec, int nq, int nkv, int d, int page_size, int window, float scale,
                                         int splits, cudaStream_t stream) {
  if (n_dec <= 0) return 0;
  if (!zi_attention_mma_supported(nq, nkv, d, 1))
    return zi_refuse("attention_decode: head_dim %d (64, 128, 256) or group size %d (<= 16) is not supported", d, nq / nkv);
  if (splits < 1 || (splits > 1 && !workspace)) return zi_refuse("attention_decode: %d splits need a workspace", splits);
  if ((qkv == nullptr) == (partials == nullptr)) return zi_refuse("attention_decode: give the rows either whole or as partial sums");
  if ((cos_t == nullptr) != (sin_t == nullptr)) return zi_refuse("attention_decode: cos and sin tables go together");
  FusedQK fq;
  fq.qkv = (const bf16*)qkv;
  fq.qkv_stride = qkv_stride;
  fq.part = partials;
  fq.part_splits = part_splits;
  fq.part_zstride = part_zstride;
  fq.width = (nq + 2 * nkv) * d;
  fq.qw = qw;
  fq.kw = kw;
  fq.eps = eps;
  fq.cos_t = cos_t;
  fq.sin_t = sin_t;
  fq.n_table_pos = n_table_pos > 0 ? n_table_pos : 1;
  fq.positions = positions;
  fq.slots = slots;
  fq.kcache_w = (bf16*)kcache;
  fq.vcache_w = (bf16*)vcache;
  return dispatch_decode<true>(d, out, out_stride, workspace, nullptr, 0, kcache, vcache, n_pages, block_tables, bt_stride, cu_q,
                               kv_lens, dec_seq, n_dec, nq, nkv, page_size, window, scale, splits, fq, stream);
}

ZI_TRACE_SETTER(attention_mma)
