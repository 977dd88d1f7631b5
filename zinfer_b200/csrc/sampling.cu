// Sampling from 32-bit logits on the device: greedy (first maximum wins) and the
// reference's chain of penalties, top-k, temperature, min-p, top-p and one draw
// (src/sampling/sampler.zig:18-91), one thread-block cluster per row.
//
// The reference sorts candidates by descending logit and cuts prefixes of that order.
// Here every cut is a threshold in the order (adjusted logit descending, token id
// ascending), found by radix selection four bits at a time with the bins in registers
// (no atomics in any sum of weights, so sums do not depend on timing and a draw is reproducible
// bit for bit).  Only the bound for a short top-k list counts keys with integer atomics in
// shared memory, 12 bits at a time: a count is the same in whatever order it is made.
#include <cooperative_groups.h>

#include <type_traits>

#include "api.h"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace {
constexpr int THREADS = 1024;
constexpr int SMALL_K = 1024;   // top-k up to this many candidates are listed, sorted and walked as the reference does

__device__ __forceinline__ float adjusted_logit(float logit, int count, float rep, float pres, float freq) {
  // src/sampling/sampler.zig:186-201
  if (count == 0) return logit;
  float a = logit;
  if (rep > 0.f && rep != 1.f) a = a < 0.f ? a * rep : a / rep;
  a -= pres;
  a -= (float)count * freq;
  return a;
}

struct RowView {
  const float* logits;
  const int* counts;  // may be null
  int V;
  float rep, pres, freq;
};

// Calls f(v, adjusted logit of v) for the tokens first, first + stride, ... in rising order.  The
// loads of four tokens go out together.
constexpr int VISIT_UNROLL = 4;
template <typename F>
__device__ __forceinline__ void for_each_token(const RowView& row, int first, int stride, F&& f) {
  for (int v0 = first; v0 < row.V; v0 += VISIT_UNROLL * stride) {
    float lg[VISIT_UNROLL];
    int cn[VISIT_UNROLL];
#pragma unroll
    for (int j = 0; j < VISIT_UNROLL; ++j) {
      const int v = v0 + j * stride;
      lg[j] = v < row.V ? row.logits[v] : 0.f;
      cn[j] = (row.counts && v < row.V) ? row.counts[v] : 0;
    }
#pragma unroll
    for (int j = 0; j < VISIT_UNROLL; ++j) {
      const int v = v0 + j * stride;
      if (v < row.V) f(v, adjusted_logit(lg[j], cn[j], row.rep, row.pres, row.freq));
    }
  }
}

// ---------------------------------------------------------------------------- argmax
// First maximum among the tokens first, first + stride, ... of every thread of the block.
__device__ void block_argmax(const RowView& row, int first, int stride, float* best_val_out, int* best_idx_out,
                             float* sval, int* sidx) {
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for_each_token(row, first, stride, [&](int v, float a) {
    if (a != a) a = -INFINITY;
    if (a > bv || (a == bv && v < bi)) { bv = a; bi = v; }
  });
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
  block_argmax(row, threadIdx.x, blockDim.x, &bv, &bi, sval, sidx);
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

// Picks among `chunks` candidates per row (value, token id): the largest value, and of equal values
// the lowest id.  Any block of whole warps.
__global__ void __launch_bounds__(256) argmax_final_kernel(int* __restrict__ out, const float* __restrict__ pval,
                                                           const int* __restrict__ pidx, int chunks) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sval[8];
  __shared__ int sidx[8];
  const size_t r = blockIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
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
  if (blockDim.x > 32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) { sval[warp] = bv; sidx[warp] = bi; }
    __syncthreads();
    if (warp != 0) return;
    bv = lane < nwarp ? sval[lane] : -INFINITY;
    bi = lane < nwarp ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
  }
  if (threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
}

// ------------------------------------------------------------------- radix selection
// Candidates are ordered by (key descending, token id ascending), key being the
// order-preserving bits of the adjusted logit.  A cut of that order is a pair (key threshold,
// id limit): a token is inside if its key is above the threshold, or equal to it with an id
// up to the limit.  Thresholds are found four bits at a time: every thread counts (or sums
// weights of) its tokens into 16 bins held in registers, the bins are added up in a fixed
// order, and all threads walk the 16 totals from the top.  No atomics in any sum: the sums do
// not depend on timing, so a draw is reproducible bit for bit.
//
// A row is always cut into SLICES slices of blockDim.x threads each: thread t of slice s owns the
// tokens (s * blockDim.x + t) + j * SLICES * blockDim.x.  One pass of one block over 150,000 tokens
// is bound by instruction issue on its SM (40 us), so the row's slices are spread over the CTAs of
// a thread-block cluster (8, 4, 2 or 1 CTAs, by the number of rows), which exchange their
// slices' totals through distributed shared memory.  Every sum is made per slice and the slices
// are added in order, so the result does not depend on how many CTAs shared the row.
__device__ __forceinline__ unsigned int order_key(float a) {
  unsigned int b = __float_as_uint(a);
  if (a != a) b = 0xff800000u;  // NaN sorts as -inf
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Cut {
  unsigned int key;   // threshold on the key
  int id_limit;       // among tokens with exactly that key, ids up to this are inside
};
__device__ __forceinline__ bool inside(const Cut& c, unsigned int key, int v) {
  return key > c.key || (key == c.key && v <= c.id_limit);
}

constexpr int SLICES = 8;

// The CTAs that share a row, and the shared memory they exchange totals through (the same
// variables in every CTA, so that one address serves for all ranks).
struct Team {
  cg::cluster_group cl;
  int rank, per;              // this CTA's rank; slices per CTA (SLICES / CTAs of the cluster)
  unsigned int pass;          // its parity picks the exchange buffer
  unsigned int* warp_buf;     // [SLICES][32][16] words: per-warp bins of each of this CTA's slices
  unsigned int* slice_buf;    // [2][SLICES][16] words: per-slice totals, written by the slice's owner
  unsigned int* tot_buf;      // [16] words: the row's totals, for all threads of this CTA
  __device__ __forceinline__ int first(int slice) const { return slice * (int)blockDim.x + (int)threadIdx.x; }
  __device__ __forceinline__ int stride() const { return SLICES * (int)blockDim.x; }
};

// One pass over the row: acc(v, adjusted logit, bins) adds token v into the calling thread's 16
// bins; every thread of every CTA of the team receives the row's 16 totals in `tot`.  Within a
// slice the bins are added over each warp by shuffles and over the warps in order.
template <typename T, typename F>
__device__ __forceinline__ void team_sum16(const RowView& row, Team& tm, T (&tot)[16], F&& acc) {
  static_assert(sizeof(T) == 4, "bins are 32-bit");
  T* slices = reinterpret_cast<T*>(tm.slice_buf) + (tm.pass & 1u) * SLICES * 16;
  T* warps = reinterpret_cast<T*>(tm.warp_buf);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int i = 0; i < tm.per; ++i) {
    const int slice = tm.rank * tm.per + i;
    T bins[16];
#pragma unroll
    for (int b = 0; b < 16; ++b) bins[b] = 0;
    for_each_token(row, tm.first(slice), tm.stride(), [&](int v, float a) { acc(v, a, bins); });
#pragma unroll
    for (int b = 0; b < 16; ++b) {
      T v = bins[b];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      bins[b] = v;
    }
    if (lane == 0)
#pragma unroll
      for (int b = 0; b < 16; ++b) warps[(i * 32 + warp) * 16 + b] = bins[b];
  }
  __syncthreads();
  if ((int)threadIdx.x < tm.per * 16) {
    const int i = threadIdx.x >> 4, b = threadIdx.x & 15;
    T t = 0;
    for (int w = 0; w < nwarp; ++w) t += warps[(i * 32 + w) * 16 + b];   // fixed order
    slices[(tm.rank * tm.per + i) * 16 + b] = t;
  }
  tm.cl.sync();   // every slice's totals are written (and, one pass on, the other buffer is free again)
  if (threadIdx.x < 16) {
    T t = 0;
    for (int s = 0; s < SLICES; ++s) {   // fixed order, whoever made the slice
      const T* theirs = tm.cl.map_shared_rank(slices, s / tm.per);
      t += theirs[s * 16 + threadIdx.x];
    }
    reinterpret_cast<T*>(tm.tot_buf)[threadIdx.x] = t;
  }
  __syncthreads();
#pragma unroll
  for (int b = 0; b < 16; ++b) tot[b] = reinterpret_cast<T*>(tm.tot_buf)[b];
  tm.pass += 1;
}

// First maximum of the row's adjusted logits, for every thread of the team.
__device__ void team_argmax(const RowView& row, Team& tm, float* best_val, int* best_idx, float* sval, int* sidx) {
  unsigned int* slices = tm.slice_buf + (tm.pass & 1u) * SLICES * 16;
  for (int i = 0; i < tm.per; ++i) {
    const int slice = tm.rank * tm.per + i;
    float bv;
    int bi;
    block_argmax(row, tm.first(slice), tm.stride(), &bv, &bi, sval, sidx);
    if (threadIdx.x == 0) {
      slices[slice * 16] = __float_as_uint(bv);
      slices[slice * 16 + 1] = (unsigned int)bi;
    }
    __syncthreads();   // sval/sidx are reused by the next slice
  }
  tm.cl.sync();
  if (threadIdx.x == 0) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int s = 0; s < SLICES; ++s) {
      const unsigned int* theirs = tm.cl.map_shared_rank(slices, s / tm.per);
      const float v = __uint_as_float(theirs[s * 16]);
      const int idx = (int)theirs[s * 16 + 1];
      if (v > bv || (v == bv && idx < bi)) { bv = v; bi = idx; }
    }
    tm.tot_buf[0] = __float_as_uint(bv);
    tm.tot_buf[1] = (unsigned int)bi;
  }
  __syncthreads();
  *best_val = __uint_as_float(tm.tot_buf[0]);
  *best_idx = (int)tm.tot_buf[1];
  tm.pass += 1;
}

// The cut with `target` measure inside it (measure(above the cut) < target <= measure(with
// the cut's own key)).  F(v, adjusted logit, key&, weight&) -> bool says whether token v is a
// candidate and gives its key and weight; WEIGHTED false counts candidates instead.
template <bool WEIGHTED, typename F>
__device__ Cut select_cut(const RowView& row, Team& tm, const F& cand, double target) {
  using T = typename std::conditional<WEIGHTED, float, int>::type;
  unsigned int prefix = 0, mask = 0;
  double remaining = target;
  double eq_total = 0.0;
  for (int pass = 0; pass < 8; ++pass) {
    const int shift = 28 - 4 * pass;
    T tot[16];
    team_sum16<T>(row, tm, tot, [&](int v, float a, T (&bins)[16]) {
      unsigned int key;
      float w;
      if (!cand(v, a, key, w) || (key & mask) != prefix) return;
      const unsigned int d = (key >> shift) & 15u;
      const T inc = WEIGHTED ? (T)w : (T)1;
#pragma unroll
      for (int b = 0; b < 16; ++b) bins[b] += (d == (unsigned)b) ? inc : (T)0;
    });
    double cum = 0.0;
    int digit = 0;
#pragma unroll
    for (int b = 15; b >= 0; --b) {
      if (cum + (double)tot[b] >= remaining || b == 0) {
        digit = b;
        eq_total = (double)tot[b];
        break;
      }
      cum += (double)tot[b];
    }
    remaining -= cum;
    prefix |= (unsigned)digit << shift;
    mask |= 15u << shift;
  }
  // `remaining` of the measure must come from the tokens whose key equals the threshold
  Cut cut{prefix, 0x7fffffff};
  // how many of those tokens (all of equal weight): all of them unless fewer suffice
  int n_eq = 0, need = 0;
  {
    int tot[16];
    team_sum16<int>(row, tm, tot, [&](int v, float a, int (&bins)[16]) {
      unsigned int key;
      float w;
      if (cand(v, a, key, w) && key == prefix) bins[0] += 1;
    });
    n_eq = tot[0];
  }
  if (n_eq <= 1) return cut;
  if (WEIGHTED) {
    const double w_each = eq_total / (double)n_eq;
    need = w_each > 0.0 ? (int)ceil(remaining / w_each - 1e-9) : n_eq;
  } else {
    need = (int)remaining;
  }
  if (need >= n_eq) return cut;
  if (need < 1) need = 1;
  // the need-th smallest id among the tokens with the threshold key (ids below 2^20)
  unsigned int iprefix = 0, imask = 0;
  int left = need;
  for (int pass = 0; pass < 5; ++pass) {
    const int shift = 16 - 4 * pass;
    int tot[16];
    team_sum16<int>(row, tm, tot, [&](int v, float a, int (&bins)[16]) {
      unsigned int key;
      float w;
      if (!cand(v, a, key, w) || key != prefix || ((unsigned)v & imask) != iprefix) return;
      const unsigned int d = ((unsigned)v >> shift) & 15u;
#pragma unroll
      for (int b = 0; b < 16; ++b) bins[b] += (d == (unsigned)b) ? 1 : 0;
    });
    int cum = 0, digit = 15;
#pragma unroll
    for (int b = 0; b < 16; ++b) {
      if (cum + tot[b] >= left) {
        digit = b;
        break;
      }
      cum += tot[b];
    }
    left -= cum;
    iprefix |= (unsigned)digit << shift;
    imask |= 15u << shift;
  }
  cut.id_limit = (int)iprefix;
  return cut;
}

// A key lower bound `lb` with at least k and (if the data allow) at most `limit` tokens at or
// above it, and the row's first maximum, in as few passes over the row as the data allow: usually
// one.  Every CTA counts its tokens by the top 12 bits of their keys into 4,096 bins in shared
// memory (integer atomics: a count does not depend on the order of its increments), keeping the
// running maximum on the way; after a cluster barrier every thread adds four bins over the CTAs,
// and a block-wide sum from the top finds the bin in which the k-th key lies.  Only if that bin
// holds more tokens than may be listed is the row read again, for the next 12 bits (and once more
// for the last 8).  Returns the number of tokens with key >= lb.  `hist` is this CTA's 4,096 words.
constexpr int HIST_BINS = 4096;   // four per thread of a block of THREADS
static_assert(HIST_BINS == 4 * THREADS, "every thread adds four neighbouring bins");
__device__ int hist_lower_bound(const RowView& row, Team& tm, int k, int limit, unsigned int& lb, unsigned int* hist,
                                float* best_val, int* best_idx, float* sval, int* sidx) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int n_ctas = SLICES / tm.per;
  unsigned int prefix = 0, mask = 0;
  int remaining = k, above = 0, n_ge = row.V;
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = pass == 0 ? 20 : pass == 1 ? 8 : 0;
    const unsigned int width = pass == 2 ? 0xffu : 0xfffu;
    for (int b = threadIdx.x; b < HIST_BINS; b += blockDim.x) hist[b] = 0u;
    __syncthreads();
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = 0; i < tm.per; ++i) {
      const int slice = tm.rank * tm.per + i;
      for_each_token(row, tm.first(slice), tm.stride(), [&](int v, float a) {
        const unsigned int key = order_key(a);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & width], 1u);
        if (pass == 0) {
          if (a != a) a = -INFINITY;
          if (a > bv || (a == bv && v < bi)) { bv = a; bi = v; }
        }
      });
    }
    if (pass == 0) {
      // this CTA's first maximum: over each warp by shuffles, over the warps by warp 0
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
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
        if (lane == 0) {
          unsigned int* mine = tm.slice_buf + (tm.pass & 1u) * SLICES * 16;
          mine[0] = __float_as_uint(bv);
          mine[1] = (unsigned int)bi;
        }
      }
    }
    tm.cl.sync();   // every CTA's bins (and maximum) are complete
    // four neighbouring bins per thread, added over the CTAs; the highest bins in the highest threads
    int t[4] = {0, 0, 0, 0};
    if ((int)threadIdx.x * 4 < HIST_BINS) {
      for (int c = 0; c < n_ctas; ++c) {
        const uint4 theirs = *reinterpret_cast<const uint4*>(tm.cl.map_shared_rank(hist, c) + threadIdx.x * 4);
        t[0] += (int)theirs.x;
        t[1] += (int)theirs.y;
        t[2] += (int)theirs.z;
        t[3] += (int)theirs.w;
      }
    }
    if (pass == 0 && threadIdx.x == 0) {
      float gv = -INFINITY;
      int gi = 0x7fffffff;
      for (int c = 0; c < n_ctas; ++c) {
        const unsigned int* theirs = tm.cl.map_shared_rank(tm.slice_buf + (tm.pass & 1u) * SLICES * 16, c);
        const float v = __uint_as_float(theirs[0]);
        const int idx = (int)theirs[1];
        if (v > gv || (v == gv && idx < gi)) { gv = v; gi = idx; }
      }
      tm.tot_buf[0] = __float_as_uint(gv);
      tm.tot_buf[1] = (unsigned int)(gi == 0x7fffffff ? 0 : gi);
    }
    tm.cl.sync();   // nobody reads another CTA's bins after this: they may be cleared or reused
    if (pass == 0) tm.pass += 1;
    // tokens in bins above this thread's four: within the warp (higher lanes), then the warps above
    const int mine = t[0] + t[1] + t[2] + t[3];
    int incl = mine;   // this lane and the lanes above it
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_down_sync(0xffffffffu, incl, o);
      if (lane + o < 32) incl += up;
    }
    if (lane == 0) sidx[warp] = incl;   // the warp's total
    if (threadIdx.x == 0) tm.tot_buf[2] = 0xffffffffu;
    __syncthreads();
    int higher = incl - mine;
    for (int w = warp + 1; w < nwarp; ++w) higher += sidx[w];
    // exactly one thread's bins hold the place where the count from the top reaches `remaining`
    if (higher < remaining && higher + mine >= remaining) {
      int cum = higher;
#pragma unroll
      for (int b = 3; b >= 0; --b) {
        if (cum + t[b] >= remaining) {
          tm.tot_buf[2] = (unsigned int)(threadIdx.x * 4 + b);
          tm.tot_buf[3] = (unsigned int)cum;
          tm.tot_buf[4] = (unsigned int)t[b];
          break;
        }
        cum += t[b];
      }
    }
    __syncthreads();
    unsigned int digit = tm.tot_buf[2];
    int cum = (int)tm.tot_buf[3], in_bin = (int)tm.tot_buf[4];
    if (digit == 0xffffffffu) {   // fewer tokens than asked for: everything is inside
      digit = 0u;
      cum = 0;
      in_bin = 0;
    }
    __syncthreads();   // tot_buf and sidx are free again
    remaining -= cum;
    above += cum;
    prefix |= digit << shift;
    mask |= width << shift;
    n_ge = above + in_bin;
    if (n_ge <= limit) break;
  }
  *best_val = __uint_as_float(tm.tot_buf[0]);
  *best_idx = (int)tm.tot_buf[1];
  lb = prefix;
  return n_ge;
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

// One row per cluster of gridDim.x / rows CTAs (a power of two up to SLICES).
__global__ void __launch_bounds__(THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, int ld, int V, SampleParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sval[32];
  __shared__ int sidx[32];
  __shared__ __align__(16) unsigned int warp_buf[SLICES * 32 * 16];   // (also the 4,096 bins of hist_lower_bound)
  __shared__ unsigned int slice_buf[2 * SLICES * 16];
  __shared__ unsigned int tot_buf[16];
  __shared__ float cand_a[SMALL_K];      // the short list of candidates (used in the CTA of rank 0)
  __shared__ int cand_v[SMALL_K];
  __shared__ float sort_a[SMALL_K];
  __shared__ int sort_v[SMALL_K];
  __shared__ int n_cand, chosen;
  __shared__ double scan_buf[SLICES * 32];   // warp totals of this CTA's slices, at [slice][warp]
  __shared__ double all_tot[SLICES * 32];    // the same of every slice, and their running sums
  __shared__ double prefix_s[SLICES * 32];

  Team tm{cg::this_cluster(), 0, 0, 0u, warp_buf, slice_buf, tot_buf};
  const int n_ctas = (int)tm.cl.num_blocks();
  tm.rank = (int)tm.cl.block_rank();
  tm.per = SLICES / n_ctas;
  const int r = blockIdx.x / n_ctas;
  if (threadIdx.x == 0) {
    n_cand = 0;
    chosen = -1;
  }
  int* my_counts = (p.counts && p.count_rows && p.count_rows[r] >= 0) ? p.counts + (size_t)p.count_rows[r] * V : nullptr;
  RowView row{logits + (size_t)r * ld, my_counts, V, p.rep ? p.rep[r] : 1.f, p.pres ? p.pres[r] : 0.f,
              p.freq ? p.freq[r] : 0.f};
  const float temperature = p.temperature[r];
  const int top_k = p.top_k ? p.top_k[r] : 0;
  float amax;
  int token;
  // top-k with few candidates: a coarse key bound that leaves a short list (at least k long), found
  // in the pass that finds the maximum
  const bool few = temperature > 0.f && top_k > 1 && top_k <= SMALL_K && top_k < V;
  unsigned int lb = 0;
  int n_listed = V;
  // (the cluster barrier inside either also publishes n_cand and chosen)
  if (few) n_listed = hist_lower_bound(row, tm, top_k, SMALL_K, lb, warp_buf, &amax, &token, sval, sidx);
  else team_argmax(row, tm, &amax, &token, sval, sidx);

  if (temperature > 0.f && top_k != 1) {
    const float zmax = amax / temperature;
    const float min_p = fminf(fmaxf(p.min_p ? p.min_p[r] : 0.f, 0.f), 1.f);
    const float top_p = fminf(fmaxf(p.top_p ? p.top_p[r] : 1.f, 0.f), 1.f);
    const unsigned long long bits = splitmix64(splitmix64(p.seeds[r]) ^ (unsigned long long)(unsigned int)p.draw_index[r]);
    const double u = (double)(bits >> 11) * (1.0 / 9007199254740992.0);
    if (top_k > 0 && top_k < V && n_listed <= SMALL_K) {
      // Few candidates: every CTA sends its own to the CTA of rank 0, which orders them as the
      // reference does (logit descending, id ascending) and lets one thread run the reference's
      // loop over that short list.
      int* n0 = tm.cl.map_shared_rank(&n_cand, 0);
      float* a0 = tm.cl.map_shared_rank(cand_a, 0);
      int* v0 = tm.cl.map_shared_rank(cand_v, 0);
      for (int i = 0; i < tm.per; ++i) {
        const int slice = tm.rank * tm.per + i;
        for_each_token(row, tm.first(slice), tm.stride(), [&](int v, float a) {
          if (order_key(a) >= lb) {
            const int slot = atomicAdd(n0, 1);   // the order of arrival does not matter: the list is sorted next
            if (slot < SMALL_K) {
              a0[slot] = a;
              v0[slot] = v;
            }
          }
        });
      }
      tm.cl.sync();
      if (tm.rank == 0) {
        const int n_all = min(n_cand, SMALL_K);
        const int n = min(n_all, top_k);                       // the list is sorted: its first k are the top k
        for (int i = threadIdx.x; i < n_all; i += blockDim.x) {   // rank sort: the place of i is the number of candidates before it
          const unsigned int ki = order_key(cand_a[i]);
          const int vi = cand_v[i];
          int rank = 0;
          for (int j = 0; j < n_all; ++j) {
            const unsigned int kj = order_key(cand_a[j]);
            rank += (kj > ki || (kj == ki && cand_v[j] < vi)) ? 1 : 0;
          }
          sort_a[rank] = cand_a[i];
          sort_v[rank] = vi;
        }
        __syncthreads();
        if (threadIdx.x == 0 && n > 0) {
          // src/sampling/sampler.zig:38-90 on the sorted candidates
          double sum = 0.0;
          for (int i = 0; i < n; ++i) {
            const float e = expf(sort_a[i] / temperature - zmax);
            cand_a[i] = e;
            sum += (double)e;
          }
          int keep = n;
          if (min_p > 0.f) {
            const float thr = cand_a[0] * min_p;
            keep = 0;
            while (keep < n && cand_a[keep] >= thr) ++keep;
            keep = max(keep, 1);
            sum = 0.0;
            for (int i = 0; i < keep; ++i) sum += (double)cand_a[i];
          }
          if (top_p < 1.f) {
            double cum = 0.0;
            int np = 0;
            while (np < keep) {
              cum += (double)cand_a[np] / sum;
              ++np;
              if (cum >= (double)top_p) break;
            }
            keep = min(max(np, 1), keep);
          }
          double kept = 0.0;
          for (int i = 0; i < keep; ++i) kept += (double)cand_a[i];
          int pick = sort_v[0];
          if (kept > 0.0) {
            double thr = u * kept;
            pick = sort_v[keep - 1];
            for (int i = 0; i < keep; ++i) {
              thr -= (double)cand_a[i];
              if (thr <= 0.0) {
                pick = sort_v[i];
                break;
              }
            }
          }
          cand_v[0] = pick;
        }
        __syncthreads();
        if (n > 0) token = cand_v[0];
      }
    } else {
      // many candidates: the cut with exactly k of them inside, then thresholds over the whole row
      Cut cut_k{0u, 0x7fffffff};
      if (top_k > 0 && top_k < V) {
        auto all = [&](int, float a, unsigned int& key, float& w) {
          key = order_key(a);
          w = 1.f;
          return true;
        };
        cut_k = select_cut<false>(row, tm, all, (double)top_k);
      }
      // candidates after top-k and min-p, with weight exp(z - zmax)
      auto cand1 = [&](int v, float a, unsigned int& key, float& w) {
        key = order_key(a);
        if (!inside(cut_k, key, v)) return false;
        w = expf(a / temperature - zmax);
        return !(min_p > 0.f) || w >= min_p || v == token;
      };
      Cut cut_p{0u, 0x7fffffff};
      if (top_p < 1.f) {
        // the sum of the candidates' weights, in a fixed order
        float tot[16];
        team_sum16<float>(row, tm, tot, [&](int v, float a, float (&bins)[16]) {
          unsigned int key;
          float w;
          if (cand1(v, a, key, w)) bins[0] += w;
        });
        cut_p = select_cut<true>(row, tm, cand1, fmax((double)top_p * (double)tot[0], 1e-30));
      }
      auto cand2 = [&](int v, float a, unsigned int& key, float& w) { return cand1(v, a, key, w) && inside(cut_p, key, v); };
      // The draw: tokens in the order (slice, thread, the thread's strided tokens); find where the
      // running sum of weights passes u * total.  A thread's share of a slice, scanned over its warp:
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
      auto scan_slice = [&](int slice, float& mine, float& incl, float& excl) {
        mine = 0.f;
        for_each_token(row, tm.first(slice), tm.stride(), [&](int v, float a) {
          unsigned int key;
          float w;
          if (cand2(v, a, key, w)) mine += w;
        });
        incl = mine;                               // inclusive scan within the warp
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        excl = __shfl_up_sync(0xffffffffu, incl, 1);   // the lane below's end is this lane's start, exactly
      };
      for (int i = 0; i < tm.per; ++i) {
        const int slice = tm.rank * tm.per + i;
        float mine, incl, excl;
        scan_slice(slice, mine, incl, excl);
        if (lane == 31) scan_buf[slice * 32 + warp] = (double)incl;
      }
      tm.cl.sync();
      const int n_parts = SLICES * 32;            // (slice, warp) totals; warps a block does not have count zero
      if ((int)threadIdx.x < n_parts) {
        const int s = threadIdx.x >> 5, w = threadIdx.x & 31;
        const double* theirs = tm.cl.map_shared_rank(scan_buf, s / tm.per);
        all_tot[threadIdx.x] = w < (int)(blockDim.x >> 5) ? theirs[threadIdx.x] : 0.0;
      }
      __syncthreads();
      if ((int)threadIdx.x < n_parts) {
        double before = 0.0;
        for (int j = 0; j < (int)threadIdx.x; ++j) before += all_tot[j];   // fixed order
        prefix_s[threadIdx.x] = before;
      }
      __syncthreads();
      const double kept = prefix_s[n_parts - 1] + all_tot[n_parts - 1];
      if (kept > 0.0) {
        const double target = u * kept;
        int* chosen0 = tm.cl.map_shared_rank(&chosen, 0);
        for (int i = 0; i < tm.per; ++i) {
          const int slice = tm.rank * tm.per + i;
          // Only a warp whose share [before, before + its total) holds the target (or ends the
          // row) can hold the thread that does: the others need not look again.
          const double before = prefix_s[slice * 32 + warp], mine_w = all_tot[slice * 32 + warp];
          if (!(mine_w > 0.0 && target >= before && (target < before + mine_w || before + mine_w >= kept))) continue;
          float mine, incl, excl;
          scan_slice(slice, mine, incl, excl);     // the same sums again, bit for bit (whole warp, no barrier inside)
          const double lo = before + (lane > 0 ? (double)excl : 0.0), hi = before + (double)incl;
          // exactly one thread's interval [lo, hi) holds the target (the last non-empty one takes hi == kept)
          if (mine > 0.f && target >= lo && (target < hi || hi >= kept)) {
            double run = lo;
            int pick = -1;
            bool passed = false;
            for_each_token(row, tm.first(slice), tm.stride(), [&](int v, float a) {
              unsigned int key;
              float w;
              if (passed || !cand2(v, a, key, w)) return;
              pick = v;
              run += (double)w;
              passed = run > target;
            });
            if (pick >= 0) atomicMax(chosen0, pick);
          }
        }
      }
      tm.cl.sync();
      if (tm.rank == 0 && chosen >= 0) token = chosen;
    }  // many candidates
  }
  if (tm.rank == 0 && threadIdx.x == 0) {
    out[r] = token;
    if (my_counts) my_counts[token] += 1;
  }
  tm.cl.sync();   // no CTA leaves while another may still read its shared memory
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

// The argmax of R rows from `units` candidates per row, as the output head's product leaves them
// (zi_gemm_tcgen05_argmax): cand_val/cand_idx [R, units].
extern "C" int zi_argmax_candidates(int* out, const float* cand_val, const int* cand_idx, int R, int units,
                                    cudaStream_t stream) {
  if (R <= 0) return 0;
  if (units <= 0) return zi_refuse("argmax: no candidates");
  zi_launch(argmax_final_kernel, dim3(R), dim3(units > 256 ? 256 : 32), 0, stream, out, cand_val, cand_idx, units);
  return zi_check_launch("argmax (candidates)");
}

// CTAs that share a row of the sampling kernel: as many (8, 4, 2, 1) as still give every CTA an SM
// of its own.
extern "C" int zi_sample_ctas_per_row(int R, int sm_count) {
  int n_ctas = SLICES;
  while (n_ctas > 1 && (long long)R * n_ctas > sm_count) n_ctas /= 2;
  return n_ctas;
}

extern "C" int zi_sample(int* out, const float* logits, int R, int V, int ld, const float* temperature,
                         const int* top_k, const float* top_p, const float* min_p, const float* rep,
                         const float* pres, const float* freq, const int* count_rows, int* counts,
                         const unsigned long long* seeds, const int* draw_index, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) return zi_refuse("sample: empty logits");
  if (!temperature || !seeds || !draw_index) return zi_refuse("sample: temperature, seeds and draw_index are required");
  SampleParams p{temperature, top_k, top_p, min_p, rep, pres, freq, count_rows, counts, seeds, draw_index};
  int sms = 0, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  const int n_ctas = zi_sample_ctas_per_row(R, sms);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(R * n_ctas));
  cfg.blockDim = dim3(THREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)n_ctas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_zi_pdl_enabled ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, sample_kernel, out, logits, ld, V, p);
  if (e != cudaSuccess) return zi_refuse("sample: launch failed: %s", cudaGetErrorString(e));
  return zi_check_launch("sample");
}

// counts[t] += 1 for each token (a request's prompt, when it enters with penalties on).
extern "C" int zi_count_tokens(int* counts, const int* tokens, int n, int V, cudaStream_t stream) {
  if (n <= 0) return 0;
  zi_launch(count_tokens_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, counts, tokens, n, V);
  return zi_check_launch("count_tokens");
}

ZI_TRACE_SETTER(sampling)
