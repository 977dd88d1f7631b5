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
  pdl_launch_dependents();
  pdl_wait();
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
                    zi_launch(embed_gather_kernel<TT>, dim3(T), dim3(256), 0, stream, h, (const TT*)table, ids, H, V));
  return zi_check_launch("embed_gather");
}

// ------------------------------------------------------------ residual add + RMSNorm
// h[row] += delta[row] (when delta is given), out[r] = h[row] * w / sqrt(mean(h[row]^2) + eps).
// With `rows` (a gather of picked rows, possibly with repeats) h itself is not modified.
// One block per row; the sum of squares is taken in a fixed order.
// The update may also come as split-K partial sums: dpart[z][row][i], z < splits, added in order.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const float* __restrict__ dpart, int splits, size_t zstride,
                                   const float* __restrict__ w, float eps, TO* __restrict__ out,
                                   const int* __restrict__ rows, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* hr = h + (size_t)row * H;
  float ss = 0.f;
  if (dpart) {
    const float* dr = dpart + (size_t)row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float d = 0.f;
      for (int z = 0; z < splits; ++z) d += dr[z * zstride + i];
      const float v = hr[i] + d;
      if (!rows) hr[i] = v;
      ss += v * v;
    }
  } else if (delta) {
    const TD* dr = delta + (size_t)row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = hr[i] + to_f32(dr[i]);
      if (!rows) hr[i] = v;
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
  if (!rows) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TO>(hr[i] * w[i] * inv);
  } else {
    // picked rows: h is left as it is (a row may be picked twice), the sum is formed again
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float v = hr[i];
      if (dpart) {
        float d = 0.f;
        for (int z = 0; z < splits; ++z) d += dpart[z * zstride + (size_t)row * H + i];
        v += d;
      } else if (delta) {
        v += to_f32(delta[(size_t)row * H + i]);
      }
      o[i] = from_f32<TO>(v * w[i] * inv);
    }
  }
}

// The same with the row held in registers: one read of h and delta, one write of h and
// of the result.  Needs H % 4 == 0 and H <= 4 * VPT * blockDim.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

// PART: the update comes as split-K partial sums (`dpart`), else whole (`delta`) or not at all.
template <typename TD, typename TO, int VPT, bool PART>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                       const float* __restrict__ dpart, int splits, size_t zstride,
                                       const float* __restrict__ w, float eps, TO* __restrict__ out,
                                       const int* __restrict__ rows, int H, int n_rows) {
  pdl_launch_dependents();
  __shared__ float scratch[33];
  const int nvec = H >> 2;
  float4 ww[VPT];   // the norm's weights do not depend on the kernel before this one
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    ww[i] = idx < nvec ? Vec4<float>::load(w + 4 * idx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  // Many rows (a prompt): as many blocks as are resident at once walk the rows, so that there is no
  // last, partly filled round of blocks and the blocks of an SM drift apart (one loads while another stores).
  for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
  const int row = rows ? rows[r] : r;
  float* hr = h + (size_t)row * H;
  float4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      float4 a = Vec4<float>::load(hr + 4 * idx);
      if (PART) {
        // the splits are read eight (then four) at a time so that their loads are in flight
        // together; they are still added in order of z
        float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* base = dpart + (size_t)row * H + 4 * idx;
        int z = 0;
        for (; z + 8 <= splits; z += 8) {
          float4 p[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) p[j] = Vec4<float>::load(base + (size_t)(z + j) * zstride);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            d.x += p[j].x; d.y += p[j].y; d.z += p[j].z; d.w += p[j].w;
          }
        }
        for (; z + 4 <= splits; z += 4) {
          const float4 p0 = Vec4<float>::load(base + (size_t)z * zstride);
          const float4 p1 = Vec4<float>::load(base + (size_t)(z + 1) * zstride);
          const float4 p2 = Vec4<float>::load(base + (size_t)(z + 2) * zstride);
          const float4 p3 = Vec4<float>::load(base + (size_t)(z + 3) * zstride);
          d.x = (((d.x + p0.x) + p1.x) + p2.x) + p3.x;
          d.y = (((d.y + p0.y) + p1.y) + p2.y) + p3.y;
          d.z = (((d.z + p0.z) + p1.z) + p2.z) + p3.z;
          d.w = (((d.w + p0.w) + p1.w) + p2.w) + p3.w;
        }
        for (; z < splits; ++z) {
          const float4 p = Vec4<float>::load(base + (size_t)z * zstride);
          d.x += p.x; d.y += p.y; d.z += p.z; d.w += p.w;
        }
        a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
        if (!rows) Vec4<float>::store(hr + 4 * idx, a);   // picked rows leave h as it is (a row may be picked twice)
      } else if (delta) {
        const float4 d = Vec4<TD>::load(delta + (size_t)row * H + 4 * idx);
        a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
        if (!rows) Vec4<float>::store(hr + 4 * idx, a);
      }
      v[i] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  TO* o = out + (size_t)r * H;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec)
      Vec4<TO>::store(o + 4 * idx, make_float4(v[i].x * ww[i].x * inv, v[i].y * ww[i].y * inv, v[i].z * ww[i].z * inv,
                                               v[i].w * ww[i].w * inv));
  }
  }
}

// SMs of the current device (asked once).
static int sm_count_of_current_device() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      sms = n;
    else
      return 148;
  }
  return sms;
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* h, const void* delta, const float* dpart, int splits, size_t zstride,
                              const float* w, float eps, void* out, const int* rows, int n_rows, int H,
                              cudaStream_t stream) {
  const bool aligned = H % 4 == 0 && ((uintptr_t)h % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                       ((uintptr_t)out % 16 == 0) && ((uintptr_t)delta % 16 == 0) && ((uintptr_t)dpart % 16 == 0) &&
                       zstride % 4 == 0;
  const int nvec = H / 4;
  // few rows (decode): one vector per thread, so that a row's loads are all in flight at once
  // many rows (a prompt): blocks of 512 with two vectors a thread keep the most bytes in flight per SM (measured:
  // 8,192 rows of 4,096 in 70 us against 76 with 256 threads and 97 with 128)
  const int threads = n_rows <= 256 ? (nvec > 512 ? 1024 : nvec > 256 ? 512 : 256) : (nvec >= 1024 ? 512 : 256);
  if (aligned && nvec <= threads * 8) {
    const int vpt = (nvec + threads - 1) / threads;
    // as many blocks as are resident at once (asked once per kernel and block size), or one per row if those are fewer
#define ZI_LAUNCH_VPT(V, P)                                                                                        \
  do {                                                                                                             \
    auto kern = add_rmsnorm_vec_kernel<TD, TO, V, P>;                                                              \
    static int per_sm[3] = {0, 0, 0};                                                                              \
    int& slot = per_sm[threads == 256 ? 0 : threads == 512 ? 1 : 2];                                               \
    if (slot == 0 && (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&slot, kern, threads, 0) != cudaSuccess || slot < 1)) \
      slot = 1;                                                                                                    \
    const int resident = sm_count_of_current_device() * slot;                                                      \
    zi_launch(kern, dim3(n_rows < resident ? n_rows : resident), dim3(threads), 0, stream, h, (const TD*)delta, dpart, \
              splits, zstride, w, eps, (TO*)out, rows, H, n_rows);                                                 \
  } while (0)
#define ZI_LAUNCH_PART(V)            \
  do {                               \
    if (dpart) ZI_LAUNCH_VPT(V, true); \
    else ZI_LAUNCH_VPT(V, false);    \
  } while (0)
    if (vpt <= 1) ZI_LAUNCH_PART(1);
    else if (vpt <= 2) ZI_LAUNCH_PART(2);
    else if (vpt <= 4) ZI_LAUNCH_PART(4);
    else ZI_LAUNCH_PART(8);
#undef ZI_LAUNCH_PART
#undef ZI_LAUNCH_VPT
  } else {
    const int t2 = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    zi_launch(add_rmsnorm_kernel<TD, TO>, dim3(n_rows), dim3(t2), 0, stream, h, (const TD*)delta, dpart, splits, zstride, w, eps, (TO*)out,
                                                          rows, H);
  }
  return zi_check_launch("add_rmsnorm");
}

extern "C" int zi_add_rmsnorm(float* h, const void* delta, int delta_dtype, const float* delta_partials, int splits,
                              long long split_stride, const float* w, float eps, void* out, int out_dtype,
                              const int* rows, int n_rows, int H, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (delta && delta_partials) return zi_refuse("add_rmsnorm: give the update either whole or as partial sums");
  ZI_DISPATCH_DTYPE(delta_dtype, TD, ZI_DISPATCH_DTYPE(out_dtype, TO, {
                      return launch_add_rmsnorm<TD, TO>(h, delta, delta_partials, splits, (size_t)split_stride, w, eps,
                                                        out, rows, n_rows, H, stream);
                    }));
  return 0;
}

// Plain add of the last pending update into the residual stream (rows optional).
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ h, const TD* __restrict__ delta, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) h[i] += to_f32(delta[i]);
}

extern "C" int zi_residual_add(float* h, const void* delta, int delta_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  ZI_DISPATCH_DTYPE(delta_dtype, TD,
                    zi_launch(residual_add_kernel<TD>, dim3(blocks), dim3(threads), 0, stream, h, (const TD*)delta, (size_t)n));
  return zi_check_launch("residual_add");
}

// --------------------------------------------------------------------------- SwiGLU
// gu is [T, 2I].  interleave == 0: gate in the first I columns, up in the last I.
// interleave == 64: blocks of 128 columns hold 64 gate then the 64 up values of the same
// features.  out[t,i] = silu(g) * u.
__device__ __forceinline__ void gate_up_columns(int i, int I, int interleave, int& gcol, int& ucol) {
  if (interleave) {
    gcol = (i / interleave) * 2 * interleave + (i % interleave);
    ucol = gcol + interleave;
  } else {
    gcol = i;
    ucol = i + I;
  }
}

template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gu, int I, size_t total, int interleave) {
  pdl_launch_dependents();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / I;
  const int i = (int)(idx - t * I);
  int gc, uc;
  gate_up_columns(i, I, interleave, gc, uc);
  const float g = to_f32(gu[t * 2 * I + gc]);
  const float u = to_f32(gu[t * 2 * I + uc]);
  out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// gate and up given as split-K partial sums part[z][t][2I]; four elements per thread.
template <typename T>
__global__ void swiglu_partials_kernel(T* __restrict__ out, const float* __restrict__ part, int splits, size_t zstride,
                                       int I, size_t total_vec, int interleave) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_vec) return;
  const int per_row = I >> 2;
  const size_t t = idx / per_row;
  const int i = (int)(idx - t * per_row) * 4;
  float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
  int gc, uc;
  gate_up_columns(i, I, interleave, gc, uc);
  for (int z0 = 0; z0 < splits; z0 += 4) {   // four splits' loads in flight together, added in order of z
    float4 a[4], b[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float* p = part + (size_t)(z0 + j) * zstride + t * 2 * I;
      const bool on = z0 + j < splits;
      a[j] = on ? *reinterpret_cast<const float4*>(p + gc) : make_float4(0.f, 0.f, 0.f, 0.f);
      b[j] = on ? *reinterpret_cast<const float4*>(p + uc) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (z0 + j < splits) {
        g.x += a[j].x; g.y += a[j].y; g.z += a[j].z; g.w += a[j].w;
        u.x += b[j].x; u.y += b[j].y; u.z += b[j].z; u.w += b[j].w;
      }
    }
  }
  Vec4<T>::store(out + t * I + i, make_float4(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y,
                                              g.z / (1.0f + expf(-g.z)) * u.z, g.w / (1.0f + expf(-g.w)) * u.w));
}

// Eight elements per thread (16-byte loads of bfloat16, two of float); needs I % 8 == 0.
template <typename T>
__global__ void swiglu_vec_kernel(T* __restrict__ out, const T* __restrict__ gu, int I, size_t total_vec,
                                  int interleave) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_vec) return;
  const int per_row = I >> 3;
  const size_t t = idx / per_row;
  const int i = (int)(idx - t * per_row) * 8;
  int gc, uc;
  gate_up_columns(i, I, interleave, gc, uc);
  const T* g = gu + t * 2 * I + gc;
  const T* u = gu + t * 2 * I + uc;
  T* o = out + t * I + i;
#pragma unroll
  for (int k = 0; k < 8; k += 4) {
    const float4 gv = Vec4<T>::load(g + k), uv = Vec4<T>::load(u + k);
    Vec4<T>::store(o + k, make_float4(gv.x / (1.0f + expf(-gv.x)) * uv.x, gv.y / (1.0f + expf(-gv.y)) * uv.y,
                                      gv.z / (1.0f + expf(-gv.z)) * uv.z, gv.w / (1.0f + expf(-gv.w)) * uv.w));
  }
}

extern "C" int zi_swiglu_partials(void* out, int dtype, const float* partials, int splits, long long split_stride,
                                  int T, int I, int interleave, cudaStream_t stream) {
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  if (I % 4 || (uintptr_t)partials % 16 || (uintptr_t)out % 8 || split_stride % 4)
    return zi_refuse("swiglu_partials: needs I %% 4 == 0 and aligned buffers");
  const size_t total_vec = total / 4;
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(swiglu_partials_kernel<TT>, dim3((unsigned)((total_vec + 255) / 256)), dim3(256), 0, stream, 
                                   (TT*)out, partials, splits, (size_t)split_stride, I, total_vec, interleave));
  return zi_check_launch("swiglu_partials");
}

extern "C" int zi_swiglu(void* out, const void* gu, int dtype, int T, int I, int interleave, cudaStream_t stream) {
  if (interleave && (interleave % 8 || I % interleave)) return zi_refuse("swiglu: interleave %d does not fit I = %d", interleave, I);
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  const int threads = 256;
  if (I % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gu % 16 == 0) {
    const size_t total_vec = total / 8;
    const unsigned blocks = (unsigned)((total_vec + threads - 1) / threads);
    ZI_DISPATCH_DTYPE(dtype, TT,
                      zi_launch(swiglu_vec_kernel<TT>, dim3(blocks), dim3(threads), 0, stream, (TT*)out, (const TT*)gu, I, total_vec, interleave));
    return zi_check_launch("swiglu");
  }
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(swiglu_kernel<TT>, dim3(blocks), dim3(threads), 0, stream, (TT*)out, (const TT*)gu, I, total, interleave));
  return zi_check_launch("swiglu");
}

// --------------------------------------------------------------------- rotary table
// cos/sin [n_pos, d/2] by the 32-bit recipe: exponent = 2i/d, p = theta^exponent,
// inv_freq = 1/p, angle = pos * inv_freq, each step rounded to float.  pow, cos and
// sin are evaluated in double and rounded once, so the table holds the correctly
// rounded value of each 32-bit step.
__global__ void rope_table_kernel(float* __restrict__ cos_t, float* __restrict__ sin_t, int n_pos, int half,
                                  int d, float theta) {
  pdl_launch_dependents();
  pdl_wait();
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
  zi_launch(rope_table_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, cos_t, sin_t, n_pos, d / 2, d, theta);
  return zi_check_launch("rope_table");
}

// ------------------------------------------- q/k RMSNorm + rotary + write into pages
// One warp per (token, head) of the fused projection row [q heads | k heads | v heads].
// q heads: normed, rotated, written to q_out (which may be the source itself).  k heads:
// normed, rotated, written to the key page slot of the token.  v heads: copied to the
// value page slot.  The source row is either `src` (activation dtype) or split-K partial
// sums part[z][t][width] that are added in order.  Pages are [page][kv head][offset][d].
template <typename T>
__global__ void qk_norm_rope_store_kernel(const T* src, int src_stride, const float* __restrict__ part,
                                          int splits, size_t zstride, int part_width, T* q_out,
                                          int q_stride, int nq, int nkv, int d, const float* __restrict__ qw,
                                          const float* __restrict__ kw, float eps, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, int n_table_pos,
                                          const int* __restrict__ positions, T* __restrict__ kcache,
                                          T* __restrict__ vcache, const int* __restrict__ slots, int page_size,
                                          int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int n_heads = nq + (write_kv ? 2 * nkv : 0);
  const int half = d >> 1;
  // one block per token; its warps take the heads in turn
  for (int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5); head < n_heads;
       head += gridDim.y * (blockDim.x >> 5)) {
  auto load = [&](int i) -> float {
    if (part) {
      const float* p = part + (size_t)t * part_width + (size_t)head * d + i;
      float v = 0.f;
      int z = 0;
      for (; z + 4 <= splits; z += 4) {   // four loads in flight, added in order
        const float p0 = p[(size_t)z * zstride], p1 = p[(size_t)(z + 1) * zstride];
        const float p2 = p[(size_t)(z + 2) * zstride], p3 = p[(size_t)(z + 3) * zstride];
        v = (((v + p0) + p1) + p2) + p3;
      }
      for (; z < splits; ++z) v += p[(size_t)z * zstride];
      return v;
    }
    return to_f32(src[(size_t)t * src_stride + (size_t)head * d + i]);
  };

  T* dst;
  if (head < nq) {
    dst = q_out + (size_t)t * q_stride + (size_t)head * d;
  } else {
    const int slot = slots[t];
    if (slot < 0) continue;
    const int kvh = (head - nq) % nkv;
    T* base = head < nq + nkv ? kcache : vcache;
    dst = base + (((size_t)(slot / page_size) * nkv + kvh) * page_size + (slot % page_size)) * d;
  }
  if (head >= nq + nkv) {  // value head: copy
    for (int i = lane; i < d; i += 32) dst[i] = from_f32<T>(load(i));
    continue;
  }
  // the head's pairs (i, i + d/2) this lane owns, read once into registers (d <= 256)
  constexpr int MAXP = 4;
  float a[MAXP], b[MAXP];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXP; ++j) {
    const int i = lane + 32 * j;
    a[j] = b[j] = 0.f;
    if (i < half) {
      a[j] = load(i);
      b[j] = load(i + half);
      ss = sum_squares_step(ss, a[j], b[j]);
    }
  }
  const float* w = head < nq ? qw : kw;
  float inv = 1.f;
  if (w) {
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)d + eps);
  }
  int pos = positions[t];
  if (pos >= n_table_pos) pos = n_table_pos - 1;  // the host refuses such positions
#pragma unroll
  for (int j = 0; j < MAXP; ++j) {
    const int i = lane + 32 * j;
    if (i >= half) continue;
    float x = a[j], y = b[j];
    if (w) {
      x = norm_scale(x, w[i], inv);
      y = norm_scale(y, w[i + half], inv);
    }
    if (cos_t) rotate_pair(x, y, cos_t[(size_t)pos * half + i], sin_t[(size_t)pos * half + i]);
    dst[i] = from_f32<T>(x);
    dst[i + half] = from_f32<T>(y);
  }
  }  // heads
}

// The same for many tokens of bfloat16 rows (prompt portions), 16 bytes per access: HALF / 8
// lanes share a (token, head), each with 8 consecutive elements of the head's first half and
// the 8 that pair with them in the second; a warp works on 32 / (HALF / 8) heads at once.
// d in {16, 32, 64, 128, 256}.
template <int D>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_vec_kernel(const __nv_bfloat16* src, int src_stride, __nv_bfloat16* q_out,   // may be the same rows
                              int q_stride, int nq, int nkv, const float* __restrict__ qw,
                              const float* __restrict__ kw, float eps, const float* __restrict__ cos_t,
                              const float* __restrict__ sin_t, int n_table_pos, const int* __restrict__ positions,
                              __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                              const int* __restrict__ slots, int page_size, int n_heads, long long n_items) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int HALF = D / 2, LPI = HALF / 8;            // lanes per (token, head)
  const long long item_raw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) / LPI;
  const bool in_range = item_raw < n_items;
  const long long item = in_range ? item_raw : n_items - 1;   // lanes past the end load a valid row and store nothing
  const int sub = threadIdx.x % LPI;
  const int t = (int)(item / n_heads), head = (int)(item % n_heads);
  const int i0 = sub * 8;
  const __nv_bfloat16* sp = src + (size_t)t * src_stride + (size_t)head * D + i0;
  const uint4 ra = *reinterpret_cast<const uint4*>(sp), rb = *reinterpret_cast<const uint4*>(sp + HALF);
  float a[8], b[8];
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&ra);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&rb);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 fa = __bfloat1622float2(pa[j]), fb = __bfloat1622float2(pb[j]);
    a[2 * j] = fa.x;
    a[2 * j + 1] = fa.y;
    b[2 * j] = fb.x;
    b[2 * j + 1] = fb.y;
  }
  // the sum of squares of the head, by every lane of the warp (no lane leaves before the shuffles)
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss = sum_squares_step(ss, a[j], b[j]);
#pragma unroll
  for (int o = LPI / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o, LPI);
  if (!in_range) return;
  __nv_bfloat16* dst;
  if (head < nq) {
    dst = q_out + (size_t)t * q_stride + (size_t)head * D + i0;
  } else {
    const int slot = slots[t];
    if (slot < 0) return;
    const int kvh = (head - nq) % nkv;
    __nv_bfloat16* base = head < nq + nkv ? kcache : vcache;
    dst = base + (((size_t)(slot / page_size) * nkv + kvh) * page_size + (slot % page_size)) * D + i0;
  }
  if (head >= nq + nkv) {        // value head: copy
    *reinterpret_cast<uint4*>(dst) = ra;
    *reinterpret_cast<uint4*>(dst + HALF) = rb;
    return;
  }
  const float* w = head < nq ? qw : kw;
  const float inv = w ? 1.0f / sqrtf(ss / (float)D + eps) : 1.f;
  int pos = positions[t];
  if (pos >= n_table_pos) pos = n_table_pos - 1;  // the host refuses such positions
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (w) {
      a[j] = norm_scale(a[j], w[i0 + j], inv);
      b[j] = norm_scale(b[j], w[i0 + j + HALF], inv);
    }
    if (cos_t) rotate_pair(a[j], b[j], cos_t[(size_t)pos * HALF + i0 + j], sin_t[(size_t)pos * HALF + i0 + j]);
  }
  uint4 oa, ob;
  __nv_bfloat162* qa = reinterpret_cast<__nv_bfloat162*>(&oa);
  __nv_bfloat162* qb = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    qa[j] = __floats2bfloat162_rn(a[2 * j], a[2 * j + 1]);
    qb[j] = __floats2bfloat162_rn(b[2 * j], b[2 * j + 1]);
  }
  *reinterpret_cast<uint4*>(dst) = oa;
  *reinterpret_cast<uint4*>(dst + HALF) = ob;
}

template <int D>
static void launch_qk_vec(const void* src, int T, int src_stride, void* q_out, int q_stride, int nq, int nkv,
                          const float* qw, const float* kw, float eps, const float* cos_t, const float* sin_t,
                          int n_table_pos, const int* positions, void* kcache, void* vcache, const int* slots,
                          int page_size, int n_heads, cudaStream_t stream) {
  const long long n_items = (long long)T * n_heads;
  const long long threads = n_items * (D / 16);
  zi_launch(qk_norm_rope_store_vec_kernel<D>, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, stream,
            (const __nv_bfloat16*)src, src_stride, (__nv_bfloat16*)q_out, q_stride, nq, nkv, qw, kw, eps, cos_t, sin_t,
            n_table_pos, positions, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, slots, page_size, n_heads, n_items);
}

extern "C" int zi_qk_norm_rope_store(const void* src, int dtype, int T, int src_stride, const float* partials,
                                     int splits, long long split_stride, void* q_out, int q_stride, int nq, int nkv,
                                     int d, const float* qw, const float* kw, float eps, const float* cos_t,
                                     const float* sin_t, int n_table_pos, const int* positions, void* kcache,
                                     void* vcache, const int* slots, int page_size, int write_kv,
                                     cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d <= 0 || d % 2 || d > 256) return zi_refuse("qk_norm_rope_store: head_dim %d is not an even number up to 256", d);
  if ((cos_t == nullptr) != (sin_t == nullptr)) return zi_refuse("qk_norm_rope_store: cos and sin tables go together");
  if ((src == nullptr) == (partials == nullptr)) return zi_refuse("qk_norm_rope_store: give the rows either whole or as partial sums");
  if (write_kv && (!kcache || !vcache || !slots || page_size <= 0))
    return zi_refuse("qk_norm_rope_store: writing keys and values needs pages and slots");
  const int n_heads = nq + (write_kv ? 2 * nkv : 0);
  // more than a few tokens of bfloat16 rows: the kernel with 16-byte accesses
  const bool vec = T > 16 && dtype == ZI_BF16 && src && (d == 16 || d == 32 || d == 64 || d == 128 || d == 256) &&
                   src_stride % 8 == 0 && q_stride % 8 == 0 && (uintptr_t)src % 16 == 0 && (uintptr_t)q_out % 16 == 0 &&
                   (!write_kv || ((uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0)) &&
                   (!qw || (uintptr_t)qw % 16 == 0) && (!kw || (uintptr_t)kw % 16 == 0);
  if (vec) {
#define ZI_QK_VEC(DD)                                                                                            \
  launch_qk_vec<DD>(src, T, src_stride, q_out, q_stride, nq, nkv, qw, kw, eps, cos_t, sin_t, n_table_pos, positions, \
                    kcache, vcache, slots, page_size, n_heads, stream)
    if (d == 16) ZI_QK_VEC(16);
    else if (d == 32) ZI_QK_VEC(32);
    else if (d == 64) ZI_QK_VEC(64);
    else if (d == 128) ZI_QK_VEC(128);
    else ZI_QK_VEC(256);
#undef ZI_QK_VEC
    return zi_check_launch("qk_norm_rope_store");
  }
  // few tokens (decode): a warp per head, so that all heads run at once; many tokens: 8 warps share a token's heads
  const int warps = T <= 256 ? 4 : 8;
  dim3 grid(T, T <= 256 ? (n_heads + warps - 1) / warps : 1);
  ZI_DISPATCH_DTYPE(dtype, TT, zi_launch(qk_norm_rope_store_kernel<TT>, dim3(grid), dim3(warps * 32), 0, stream, 
                                   (const TT*)src, src_stride, partials, splits, (size_t)split_stride, n_heads * d,
                                   (TT*)q_out, q_stride, nq, nkv, d, qw, kw, eps, cos_t, sin_t, n_table_pos, positions,
                                   (TT*)kcache, (TT*)vcache, slots, page_size, write_kv));
  return zi_check_launch("qk_norm_rope_store");
}

// h[i] += sum over splits of part[z][i], in order of z (for consumers that take no partial sums).
__global__ void residual_add_partials_kernel(float* __restrict__ h, const float* __restrict__ part, int splits,
                                             size_t zstride, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float d = 0.f;
  for (int z = 0; z < splits; ++z) d += part[z * zstride + i];
  h[i] += d;
}

extern "C" int zi_residual_add_partials(float* h, const float* partials, int splits, long long split_stride,
                                        long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  zi_launch(residual_add_partials_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, h, partials, splits,
                                                                             (size_t)split_stride, (size_t)n);
  return zi_check_launch("residual_add_partials");
}

// ids[dst[i]] = prev[src[i]] for i < n with dst[i] >= 0: the tokens a step feeds that were
// sampled by the step before it are taken on the device, so the host need not wait for them.
__global__ void patch_tokens_kernel(int* __restrict__ ids, const int* __restrict__ prev, const int* __restrict__ dst,
                                    const int* __restrict__ src, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && dst[i] >= 0) ids[dst[i]] = prev[src[i]];
}

extern "C" int zi_patch_tokens(int* ids, const int* prev, const int* dst, const int* src, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  zi_launch(patch_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, ids, prev, dst, src, n);
  return zi_check_launch("patch_tokens");
}

ZI_TRACE_SETTER(elementwise)
