// Causal attention of query tokens against the paged cache, for any mix of prompt
// portions and single decoded tokens, any head size up to 256 in steps of 2, any
// number of heads and groups, with an optional window.  32-bit arithmetic on the
// CUDA cores (exact expf); the storage type alone differs between the float32 path
// and the plain bfloat16 path.  A query row visits its keys in ascending order in
// tiles aligned to multiples of BK, so its result does not depend on how the
// request was cut into steps or on what else is in the batch.
//
// Grid: (query tile of BQ tokens of one request, query head).  Pages are
// [page][kv head][offset][d]; the key at position j of request s lies in page
// block_tables[s][j / page_size] at offset j % page_size.
#include "api.h"
#include "common.cuh"

namespace {
constexpr int BQ = 16, BK = 32, THREADS = 128, ROWS_PER_WARP = BQ / (THREADS / 32), MAXJ = 8;

template <typename T>
__global__ void __launch_bounds__(THREADS)
paged_attention_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ q, int q_stride,
                       const T* __restrict__ kcache, const T* __restrict__ vcache,
                       const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_q,
                       const int* __restrict__ kv_lens, const int* __restrict__ tile_seq,
                       const int* __restrict__ tile_q0, int nq, int nkv, int d, int page_size, int window,
                       float scale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  float* Qs = smem;                   // [BQ][d]
  float* Ks = Qs + BQ * d;            // [BK][d+1]
  float* Vs = Ks + BK * (d + 1);      // [BK][d]
  float* Ss = Vs + BK * d;            // [BQ][BK]

  const int seq = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x];
  const int h = blockIdx.y, kvh = h / (nq / nkv);
  const int tok0 = cu_q[seq], qlen = cu_q[seq + 1] - tok0, kvlen = kv_lens[seq];
  const int ctx = kvlen - qlen;  // tokens of this request already in the cache before this step
  const int nqv = min(BQ, qlen - q0);
  if (nqv <= 0) return;
  const int first_pos = ctx + q0, last_pos = first_pos + nqv - 1;
  const int kv_begin = window > 0 ? max(0, first_pos - window + 1) : 0;
  const int kv_end = last_pos + 1;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* bt = block_tables + (size_t)seq * bt_stride;

  for (int e = tid; e < BQ * d; e += THREADS) {
    const int r = e / d, c = e % d;
    Qs[e] = r < nqv ? to_f32(q[(size_t)(tok0 + q0 + r) * q_stride + (size_t)h * d + c]) : 0.f;
  }

  float m[ROWS_PER_WARP], l[ROWS_PER_WARP], acc[ROWS_PER_WARP][MAXJ];
#pragma unroll
  for (int i = 0; i < ROWS_PER_WARP; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) acc[i][j] = 0.f;
  }

  for (int kt = (kv_begin / BK) * BK; kt < kv_end; kt += BK) {
    __syncthreads();  // previous tile fully consumed (also orders the Q load the first time)
    for (int e = tid; e < BK * d; e += THREADS) {
      const int kk = e / d, c = e % d;
      const int j = kt + kk;
      float kval = 0.f, vval = 0.f;
      if (j >= kv_begin && j < kv_end) {
        const int page = bt[j / page_size];
        if (page >= 0) {
          const size_t off = (((size_t)page * nkv + kvh) * page_size + (j % page_size)) * d + c;
          kval = to_f32(kcache[off]);
          vval = to_f32(vcache[off]);
        }
      }
      Ks[kk * (d + 1) + c] = kval;
      Vs[kk * d + c] = vval;
    }
    __syncthreads();

    float alpha[ROWS_PER_WARP];
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
      const int r = warp * ROWS_PER_WARP + i;
      alpha[i] = 1.f;
      if (r >= nqv) continue;  // uniform within the warp
      const int pos = first_pos + r, j = kt + lane;
      const float* qr = Qs + r * d;
      const float* kr = Ks + lane * (d + 1);
      float s = 0.f;
      for (int c = 0; c < d; ++c) s = fmaf(qr[c], kr[c], s);
      s *= scale;
      const bool visible = j <= pos && j >= kv_begin && (window <= 0 || j > pos - window);
      if (!visible) s = -INFINITY;
      const float m_new = fmaxf(m[i], warp_max(s));
      float p = 0.f;
      if (m_new != -INFINITY) {
        p = visible ? expf(s - m_new) : 0.f;
        alpha[i] = expf(m[i] - m_new);  // exp(-inf) = 0 on the first visible tile
      }
      l[i] = l[i] * alpha[i] + warp_sum(p);
      m[i] = m_new;
      Ss[r * BK + lane] = p;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < ROWS_PER_WARP; ++i) {
      const int r = warp * ROWS_PER_WARP + i;
      if (r >= nqv) continue;
#pragma unroll
      for (int j = 0; j < MAXJ; ++j) acc[i][j] *= alpha[i];
      for (int kk = 0; kk < BK; ++kk) {
        const float p = Ss[r * BK + kk];
#pragma unroll
        for (int j = 0; j < MAXJ; ++j) {
          const int c = lane + 32 * j;
          if (c < d) acc[i][j] = fmaf(p, Vs[kk * d + c], acc[i][j]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < ROWS_PER_WARP; ++i) {
    const int r = warp * ROWS_PER_WARP + i;
    if (r >= nqv) continue;
    const float inv = 1.0f / l[i];
    T* o = out + (size_t)(tok0 + q0 + r) * out_stride + (size_t)h * d;
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int c = lane + 32 * j;
      if (c < d) o[c] = from_f32<T>(acc[i][j] * inv);
    }
  }
}
}  // namespace

extern "C" int zi_paged_attention_tile_rows() { return BQ; }

extern "C" int zi_paged_attention(void* out, int out_stride, const void* q, int q_stride, int dtype,
                                  const void* kcache, const void* vcache, const int* block_tables, int bt_stride,
                                  const int* cu_q, const int* kv_lens, const int* tile_seq, const int* tile_q0,
                                  int n_tiles, int nq, int nkv, int d, int page_size, int window, float scale,
                                  cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (d <= 0 || d > 32 * MAXJ) return zi_refuse("paged_attention: head_dim %d is outside 1..%d", d, 32 * MAXJ);
  if (nkv <= 0 || nq % nkv) return zi_refuse("paged_attention: %d query heads do not divide into %d kv heads", nq, nkv);
  if (page_size <= 0) return zi_refuse("paged_attention: page_size %d", page_size);
  const size_t smem = (size_t)(BQ * d + BK * (d + 1) + BK * d + BQ * BK) * sizeof(float);
  dim3 grid(n_tiles, nq);
  ZI_DISPATCH_DTYPE(dtype, TT, {
    auto kern = paged_attention_kernel<TT>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return zi_refuse("paged_attention: cannot get %zu bytes of shared memory", smem);
    }
    zi_launch(kern, dim3(grid), dim3(THREADS), smem, stream, (TT*)out, out_stride, (const TT*)q, q_stride, (const TT*)kcache,
                                          (const TT*)vcache, block_tables, bt_stride, cu_q, kv_lens, tile_seq,
                                          tile_q0, nq, nkv, d, page_size, window, scale);
  });
  return zi_check_launch("paged_attention");
}

ZI_TRACE_SETTER(attention_generic)
