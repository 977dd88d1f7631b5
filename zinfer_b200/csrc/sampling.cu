// Sampling from 32-bit logits on the device: greedy (first maximum wins) and the
// reference's chain of penalties, top-k, temperature, min-p, top-p and one draw
// (src/sampling/sampler.zig:18-91), one block per row.
//
// The reference sorts candidates by descending logit and cuts prefixes of that
// order.  Here every cut is a threshold on a 64-bit composite key (order-preserving
// bits of the adjusted logit, then the inverted token id, so ties go to the lower
// id and keys are unique), found by radix selection over histograms.  Weights
// exp(z - max) are accumulated as 2^-40 fixed-point integers, so sums do not
// depend on the order of the additions and a draw is reproducible bit for bit.
#include "api.h"
#include "common.cuh"

namespace {
constexpr int THREADS = 1024;
constexpr double FIXED_ONE = 1099511627776.0;  // 2^40

__device__ __forceinline__ float adjusted_logit(float logit, int count, float rep, float pres, float freq) {
  // src/sampling/sampler.zig:186-201
  if (count == 0) return logit;
  float a = logit;
  if (rep > 0.f && rep != 1.f) a = a < 0.f ? a * rep : a / rep;
  a -= pres;
  a -= (float)count * freq;
  return a;
}

__device__ __forceinline__ unsigned long long composite_key(float a, int v) {
  unsigned int b = __float_as_uint(a);
  if (a != a) b = 0xff800000u;  // NaN sorts as -inf
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return ((unsigned long long)b << 32) | (unsigned long long)(0xffffffffu - (unsigned int)v);
}

struct RowView {
  const float* logits;
  const int* counts;  // may be null
  int V;
  float rep, pres, freq;
  __device__ __forceinline__ float adjusted(int v) const {
    return adjusted_logit(logits[v], counts ? counts[v] : 0, rep, pres, freq);
  }
};

// ---------------------------------------------------------------------------- argmax
__device__ void block_argmax(const RowView& row, float* best_val_out, int* best_idx_out, float* sval, int* sidx) {
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int v = threadIdx.x; v < row.V; v += blockDim.x) {
    float a = row.adjusted(v);
    if (a != a) a = -INFINITY;
    if (a > bv || (a == bv && v < bi)) { bv = a; bi = v; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { sval[warp] = bv; sidx[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = lane < nwarp ? sval[lane] : -INFINITY;
    bi = lane < nwarp ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sval[0] = bv; sidx[0] = bi == 0x7fffffff ? 0 : bi; }
  }
  __syncthreads();
  *best_val_out = sval[0];
  *best_idx_out = sidx[0];
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(int* __restrict__ out, const float* __restrict__ logits,
                                                         int ld, int V) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sval[32];
  __shared__ int sidx[32];
  RowView row{logits + (size_t)blockIdx.x * ld, nullptr, V, 1.f, 0.f, 0.f};
  float bv;
  int bi;
  block_argmax(row, &bv, &bi, sval, sidx);
  if (threadIdx.x == 0) out[blockIdx.x] = bi;
}

// Two-stage argmax for few rows over a large vocabulary: `chunks` blocks per row each
// find the first maximum of their slice, a second kernel picks among them.
__global__ void __launch_bounds__(256) argmax_partial_kernel(float* __restrict__ pval, int* __restrict__ pidx,
                                                             const float* __restrict__ logits, int ld, int V,
                                                             int chunks) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sval[32];
  __shared__ int sidx[32];
  const int r = blockIdx.x, c = blockIdx.y;
  const int per = (V + chunks - 1) / chunks;
  const int lo = c * per, hi = min(V, lo + per);
  const float* row = logits + (size_t)r * ld;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int v = lo + threadIdx.x; v < hi; v += blockDim.x) {
    float a = row[v];
    if (a != a) a = -INFINITY;
    if (a > bv || (a == bv && v < bi)) { bv = a; bi = v; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sval[warp] = bv; sidx[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = lane < (blockDim.x >> 5) ? sval[lane] : -INFINITY;
    bi = lane < (blockDim.x >> 5) ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { pval[r * chunks + c] = bv; pidx[r * chunks + c] = bi; }
  }
}

__global__ void argmax_final_kernel(int* __restrict__ out, const float* __restrict__ pval,
                                    const int* __restrict__ pidx, int chunks) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < chunks; c += 32) {
    const float v = pval[r * chunks + c];
    const int i = pidx[r * chunks + c];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
}

// ------------------------------------------------------------------- radix selection
// Finds the composite key c* such that the measure of members with key > c* is
// below `target` and the measure of members with key >= c* reaches it.
template <typename Member>
__device__ unsigned long long radix_select(const Member& member, int V, unsigned long long target,
                                           unsigned long long* hist, unsigned long long* bcast) {
  unsigned long long prefix = 0, mask = 0;
  for (int pass = 0; pass < 8; ++pass) {
    const int shift = 56 - 8 * pass;
    __syncthreads();
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int v = threadIdx.x; v < V; v += blockDim.x) {
      unsigned long long key, meas;
      if (member(v, key, meas) && (key & mask) == prefix && meas)
        atomicAdd(&hist[(key >> shift) & 255], meas);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long cum = 0;
      int digit = 0;
      for (int b = 255; b >= 0; --b) {
        if (cum + hist[b] >= target) { digit = b; break; }
        cum += hist[b];
      }
      bcast[0] = (unsigned long long)digit;
      bcast[1] = target - cum;
    }
    __syncthreads();
    prefix |= bcast[0] << shift;
    mask |= 0xffull << shift;
    target = bcast[1];
  }
  return prefix;
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

struct SampleParams {
  const float* temperature;
  const int* top_k;
  const float* top_p;
  const float* min_p;
  const float* rep;
  const float* pres;
  const float* freq;
  const int* count_rows;          // row of the count table per logits row, or -1
  int* counts;                    // [*, V] occurrences of each token in the request so far; may be null
  const unsigned long long* seeds;
  const int* draw_index;          // how many tokens the request has drawn before
};

__global__ void __launch_bounds__(THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, int ld, int V, SampleParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sval[32];
  __shared__ int sidx[32];
  __shared__ unsigned long long hist[256];
  __shared__ unsigned long long bcast[2];
  __shared__ unsigned long long ssum;
  const int r = blockIdx.x;
  int* my_counts = (p.counts && p.count_rows && p.count_rows[r] >= 0) ? p.counts + (size_t)p.count_rows[r] * V : nullptr;
  RowView row{logits + (size_t)r * ld, my_counts, V, p.rep ? p.rep[r] : 1.f, p.pres ? p.pres[r] : 0.f,
              p.freq ? p.freq[r] : 0.f};
  const float temperature = p.temperature[r];
  const int top_k = p.top_k ? p.top_k[r] : 0;
  float amax;
  int token;
  block_argmax(row, &amax, &token, sval, sidx);

  if (temperature > 0.f && top_k != 1) {
    // top-k: threshold on the composite key with exactly k members at or above it
    unsigned long long t_topk = 0;
    if (top_k > 0 && top_k < V) {
      auto member = [&](int v, unsigned long long& key, unsigned long long& meas) {
        key = composite_key(row.adjusted(v), v);
        meas = 1;
        return true;
      };
      t_topk = radix_select(member, V, (unsigned long long)top_k, hist, bcast);
    }
    const float zmax = amax / temperature;
    const float min_p = fminf(fmaxf(p.min_p ? p.min_p[r] : 0.f, 0.f), 1.f);
    const float top_p = fminf(fmaxf(p.top_p ? p.top_p[r] : 1.f, 0.f), 1.f);
    // members after top-k and min-p, with fixed-point weight exp(z - zmax)
    auto member1 = [&](int v, unsigned long long& key, unsigned long long& meas) {
      const float a = row.adjusted(v);
      key = composite_key(a, v);
      if (key < t_topk) return false;
      const float e = expf(a / temperature - zmax);
      if (min_p > 0.f && !(e >= min_p) && v != token) return false;
      meas = (unsigned long long)((double)e * FIXED_ONE);
      return true;
    };
    auto total_of = [&](auto& mem) {
      __syncthreads();
      if (threadIdx.x == 0) ssum = 0;
      __syncthreads();
      unsigned long long local = 0;
      for (int v = threadIdx.x; v < V; v += blockDim.x) {
        unsigned long long key, meas;
        if (mem(v, key, meas)) local += meas;
      }
      if (local) atomicAdd(&ssum, local);
      __syncthreads();
      return ssum;
    };
    unsigned long long t_topp = 0;
    if (top_p < 1.f) {
      const unsigned long long sum1 = total_of(member1);
      unsigned long long target = (unsigned long long)ceil((double)top_p * (double)sum1);
      if (target < 1) target = 1;
      if (target > sum1) target = sum1;
      t_topp = radix_select(member1, V, target, hist, bcast);
    }
    auto member2 = [&](int v, unsigned long long& key, unsigned long long& meas) {
      return member1(v, key, meas) && key >= t_topp;
    };
    const unsigned long long kept = total_of(member2);
    if (kept > 0) {
      const unsigned long long bits = splitmix64(splitmix64(p.seeds[r]) ^ (unsigned long long)(unsigned int)p.draw_index[r]);
      const double u = (double)(bits >> 11) * (1.0 / 9007199254740992.0);
      unsigned long long rdraw = (unsigned long long)(u * (double)kept);
      if (rdraw >= kept) rdraw = kept - 1;
      const unsigned long long chosen = radix_select(member2, V, rdraw + 1, hist, bcast);
      const unsigned int inv = (unsigned int)(chosen & 0xffffffffull);
      const int cand = (int)(0xffffffffu - inv);
      if (cand >= 0 && cand < V) token = cand;
    }
  }
  if (threadIdx.x == 0) {
    out[r] = token;
    if (my_counts) my_counts[token] += 1;
  }
}

__global__ void count_tokens_kernel(int* __restrict__ counts, const int* __restrict__ tokens, int n, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const int t = tokens[i];
    if (t >= 0 && t < V) atomicAdd(&counts[t], 1);
  }
}
}  // namespace

// `workspace` (may be null) holds 2 * R * chunks 32-bit words for the two-stage form.
extern "C" int zi_argmax_chunks(int R, int V) { return (V >= 16384 && R <= 256) ? 32 : 0; }

extern "C" int zi_argmax(int* out, const float* logits, int R, int V, int ld, void* workspace, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) return zi_refuse("argmax: empty logits");
  const int chunks = zi_argmax_chunks(R, V);
  if (chunks > 0 && workspace) {
    float* pval = (float*)workspace;
    int* pidx = (int*)workspace + (size_t)R * chunks;
    zi_launch(argmax_partial_kernel, dim3(R, chunks), dim3(256), 0, stream, pval, pidx, logits, ld, V, chunks);
    int rc = zi_check_launch("argmax (partial)");
    if (rc) return rc;
    zi_launch(argmax_final_kernel, dim3(R), dim3(32), 0, stream, out, pval, pidx, chunks);
    return zi_check_launch("argmax (final)");
  }
  zi_launch(argmax_kernel, dim3(R), dim3(THREADS), 0, stream, out, logits, ld, V);
  return zi_check_launch("argmax");
}

extern "C" int zi_sample(int* out, const float* logits, int R, int V, int ld, const float* temperature,
                         const int* top_k, const float* top_p, const float* min_p, const float* rep,
                         const float* pres, const float* freq, const int* count_rows, int* counts,
                         const unsigned long long* seeds, const int* draw_index, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) return zi_refuse("sample: empty logits");
  if (!temperature || !seeds || !draw_index) return zi_refuse("sample: temperature, seeds and draw_index are required");
  SampleParams p{temperature, top_k, top_p, min_p, rep, pres, freq, count_rows, counts, seeds, draw_index};
  zi_launch(sample_kernel, dim3(R), dim3(THREADS), 0, stream, out, logits, ld, V, p);
  return zi_check_launch("sample");
}

// counts[t] += 1 for each token (a request's prompt, when it enters with penalties on).
extern "C" int zi_count_tokens(int* counts, const int* tokens, int n, int V, cudaStream_t stream) {
  if (n <= 0) return 0;
  zi_launch(count_tokens_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, counts, tokens, n, V);
  return zi_check_launch("count_tokens");
}
