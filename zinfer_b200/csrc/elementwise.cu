// Memory-bound kernels around the matrix products: embedding gather, residual add
// fused with RMSNorm, per-head q/k RMSNorm fused with rotary positions and the
// write of keys and values into cache pages, SwiGLU, and the rotary table.
// All arithmetic is 32-bit; only loads and stores touch bfloat16.
#include "api.h"
#include "common.cuh"

// ---------------------------------------------------------------- embedding gather
template <typename T>
__global__ void embed_gather_kernel(float* __restrict__ h, const T* __restrict__ table,
                                    const int* __restrict__ ids, int H, int V) {
  const int t = blockIdx.x;
  const int id = ids[t];
  float* out = h + (size_t)t * H;
  if (id < 0 || id >= V) {  // the host refuses such ids; never read out of bounds
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = 0.f;
    return;
  }
  const T* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = to_f32(row[i]);
}

extern "C" int zi_embed_gather(float* h, const void* table, int table_dtype, const int* ids, int T, int H,
                               int V, cudaStream_t stream) {
  if (T <= 0) return 0;
  ZI_DISPATCH_DTYPE(table_dtype, TT,
                    embed_gather_kernel<TT><<<T, 256, 0, stream>>>(h, (const TT*)table, ids, H, V));
  return zi_check_launch("embed_gather");
}

// ------------------------------------------------------------ residual add + RMSNorm
// h[row] += delta[row] (when delta is given), out[r] = h[row] * w / sqrt(mean(h[row]^2) + eps).
// One block per row; the sum of squares is taken in a fixed order.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const float* __restrict__ w, float eps, TO* __restrict__ out,
                                   const int* __restrict__ rows, int H) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* hr = h + (size_t)row * H;
  float ss = 0.f;
  if (delta) {
    const TD* dr = delta + (size_t)row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = hr[i] + to_f32(dr[i]);
      hr[i] = v;
      ss += v * v;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = hr[i];
      ss += v * v;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  TO* o = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TO>(hr[i] * w[i] * inv);
}

extern "C" int zi_add_rmsnorm(float* h, const void* delta, int delta_dtype, const float* w, float eps, void* out,
                              int out_dtype, const int* rows, int n_rows, int H, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  ZI_DISPATCH_DTYPE(delta_dtype, TD, ZI_DISPATCH_DTYPE(out_dtype, TO, {
                      add_rmsnorm_kernel<TD, TO><<<n_rows, threads, 0, stream>>>(
                          h, (const TD*)delta, w, eps, (TO*)out, rows, H);
                    }));
  return zi_check_launch("add_rmsnorm");
}

// Plain add of the last pending update into the residual stream (rows optional).
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ h, const TD* __restrict__ delta, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) h[i] += to_f32(delta[i]);
}

extern "C" int zi_residual_add(float* h, const void* delta, int delta_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  ZI_DISPATCH_DTYPE(delta_dtype, TD,
                    residual_add_kernel<TD><<<blocks, threads, 0, stream>>>(h, (const TD*)delta, (size_t)n));
  return zi_check_launch("residual_add");
}

// --------------------------------------------------------------------------- SwiGLU
// gu is [T, 2I]: gate in the first I columns, up in the last I.  out[t,i] = silu(g) * u.
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gu, int I, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / I;
  const int i = (int)(idx - t * I);
  const float g = to_f32(gu[t * 2 * I + i]);
  const float u = to_f32(gu[t * 2 * I + I + i]);
  out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

extern "C" int zi_swiglu(void* out, const void* gu, int dtype, int T, int I, cudaStream_t stream) {
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  ZI_DISPATCH_DTYPE(dtype, TT, swiglu_kernel<TT><<<blocks, threads, 0, stream>>>((TT*)out, (const TT*)gu, I, total));
  return zi_check_launch("swiglu");
}

// --------------------------------------------------------------------- rotary table
// cos/sin [n_pos, d/2] by the 32-bit recipe: exponent = 2i/d, p = theta^exponent,
// inv_freq = 1/p, angle = pos * inv_freq, each step rounded to float.  pow, cos and
// sin are evaluated in double and rounded once, so the table holds the correctly
// rounded value of each 32-bit step.
__global__ void rope_table_kernel(float* __restrict__ cos_t, float* __restrict__ sin_t, int n_pos, int half,
                                  int d, float theta) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)n_pos * half) return;
  const int pos = (int)(idx / half), i = (int)(idx % half);
  const float exponent = (float)(2 * i) / (float)d;
  const float p = (float)pow((double)theta, (double)exponent);
  const float inv_freq = 1.0f / p;
  const float angle = (float)pos * inv_freq;
  cos_t[idx] = (float)cos((double)angle);
  sin_t[idx] = (float)sin((double)angle);
}

extern "C" int zi_rope_table(float* cos_t, float* sin_t, int n_pos, int d, float theta, cudaStream_t stream) {
  if (d <= 0 || d % 2) return zi_refuse("rope_table: head_dim %d is not even", d);
  const size_t total = (size_t)n_pos * (d / 2);
  if (total == 0) return 0;
  rope_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(cos_t, sin_t, n_pos, d / 2, d, theta);
  return zi_check_launch("rope_table");
}

// ------------------------------------------- q/k RMSNorm + rotary + write into pages
// One warp per (token, head) of the fused projection row [q heads | k heads | v heads].
// q heads: normed, rotated, written back in place.  k heads: normed, rotated, written
// to the key page slot of the token.  v heads: copied to the value page slot.
// Pages are [page][kv head][offset in page][d].
template <typename T>
__global__ void qk_norm_rope_store_kernel(T* __restrict__ qkv, int row_stride, int nq, int nkv, int d,
                                          const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                          int n_table_pos, const int* __restrict__ positions,
                                          T* __restrict__ kcache, T* __restrict__ vcache,
                                          const int* __restrict__ slots, int page_size, int write_kv) {
  const int t = blockIdx.x;
  const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int n_heads = nq + (write_kv ? 2 * nkv : 0);
  if (head >= n_heads) return;
  T* src = qkv + (size_t)t * row_stride + (size_t)head * d;
  const int half = d >> 1;

  T* dst;
  if (head < nq) {
    dst = src;
  } else {
    const int slot = slots[t];
    if (slot < 0) return;
    const int kvh = (head - nq) % nkv;
    T* base = head < nq + nkv ? kcache : vcache;
    dst = base + (((size_t)(slot / page_size) * nkv + kvh) * page_size + (slot % page_size)) * d;
  }
  if (head >= nq + nkv) {  // value head: copy
    for (int i = lane; i < d; i += 32) dst[i] = src[i];
    return;
  }
  const float* w = head < nq ? qw : kw;
  float inv = 1.f;
  if (w) {
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float v = to_f32(src[i]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)d + eps);
  }
  int pos = positions[t];
  if (pos >= n_table_pos) pos = n_table_pos - 1;  // the host refuses such positions
  for (int i = lane; i < half; i += 32) {
    float a = to_f32(src[i]), b = to_f32(src[i + half]);
    if (w) {
      a = a * w[i] * inv;
      b = b * w[i + half] * inv;
    }
    if (cos_t) {
      const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
      const float ra = a * c - b * s, rb = b * c + a * s;
      a = ra;
      b = rb;
    }
    dst[i] = from_f32<T>(a);
    dst[i + half] = from_f32<T>(b);
  }
}

extern "C" int zi_qk_norm_rope_store(void* qkv, int dtype, int T, int row_stride, int nq, int nkv, int d,
                                     const float* qw, const float* kw, float eps, const float* cos_t,
                                     const float* sin_t, int n_table_pos, const int* positions, void* kcache,
                                     void* vcache, const int* slots, int page_size, int write_kv,
                                     cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d <= 0 || d % 2) return zi_refuse("qk_norm_rope_store: head_dim %d is not even", d);
  if ((cos_t == nullptr) != (sin_t == nullptr)) return zi_refuse("qk_norm_rope_store: cos and sin tables go together");
  if (write_kv && (!kcache || !vcache || !slots || page_size <= 0))
    return zi_refuse("qk_norm_rope_store: writing keys and values needs pages and slots");
  const int n_heads = nq + (write_kv ? 2 * nkv : 0);
  const int warps = 4;
  dim3 grid(T, (n_heads + warps - 1) / warps);
  ZI_DISPATCH_DTYPE(dtype, TT, qk_norm_rope_store_kernel<TT><<<grid, warps * 32, 0, stream>>>(
                                   (TT*)qkv, row_stride, nq, nkv, d, qw, kw, eps, cos_t, sin_t, n_table_pos,
                                   positions, (TT*)kcache, (TT*)vcache, slots, page_size, write_kv));
  return zi_check_launch("qk_norm_rope_store");
}
