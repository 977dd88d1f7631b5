// Tile code of the tensor-core attention kernels (mma.sync m16n8k16 on bfloat16, 32-bit
// accumulation and softmax): fragment loads from XOR-swizzled shared-memory tiles, the online
// softmax step, cp.async copies of paged keys and values, and the decode unit (one request's
// token, one kv head, one split of the keys) that both the decode kernel and the kernel that
// runs whole layers of a decode step are made of.
#pragma once
#include "common.cuh"
#include "tcgen05_ptx.cuh"

namespace {
using bf16 = __nv_bfloat16;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Byte offset of 16-byte chunk `c` of row `r` in a swizzled [rows][D] bf16 tile.
template <int D> __device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)(r * D * 2 + ((c ^ (r & 7)) << 4));
}

// The same for a tile that TMA filled (TL): one box of [16 rows][64 values = 128 bytes] per 64 columns
// with the hardware's 128-byte swizzle (chunk ^ (row & 7) within a row of 128 bytes), the boxes of
// a tile one after the other.  A tile's base is 1024-byte aligned.
template <int D, bool TL> __device__ __forceinline__ uint32_t tile_off(int r, int c) {
  if (TL) return (uint32_t)((c >> 3) * 2048 + r * 128 + (((c & 7) ^ (r & 7)) << 4));
  return swz<D>(r, c);
}

// S (16 x 16 keys) += Q (16 x D) * K^T for the 16 keys at rows key0.. of tile `ks`.
// qf: the warp's Q fragments, [D/16][4].  s: two n-tiles of 8 keys.
template <int D, bool TL = false>
__device__ __forceinline__ void qk_16keys(float (&s)[2][4], const uint32_t (&qf)[D / 16][4], uint32_t ks_addr,
                                          int key0, int lane) {
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t b[4];
    const int m = lane >> 3;
    ldmatrix_x4(b, ks_addr + tile_off<D, TL>(key0 + (m >> 1) * 8 + (lane & 7), kk * 2 + (m & 1)));
    mma_bf16(s[0], qf[kk], b[0], b[1]);
    mma_bf16(s[1], qf[kk], b[2], b[3]);
  }
}
// O (16 x D) += P (16 x 16 keys) * V for the 16 keys at rows key0.. of tile `vs`.
template <int D, bool TL = false>
__device__ __forceinline__ void pv_16keys(float (&o)[D / 8][4], const uint32_t (&pf)[4], uint32_t vs_addr, int key0,
                                          int lane) {
#pragma unroll
  for (int np = 0; np < D / 16; ++np) {
    uint32_t b[4];
    const int m = lane >> 3;
    ldmatrix_x4_trans(b, vs_addr + tile_off<D, TL>(key0 + (m & 1) * 8 + (lane & 7), np * 2 + (m >> 1)));
    mma_bf16(o[2 * np], pf, b[0], b[1]);
    mma_bf16(o[2 * np + 1], pf, b[2], b[3]);
  }
}

// One step of the online softmax for the two rows a thread holds (lane/4 and lane/4+8)
// over `NT` n-tiles of 8 keys; s holds scores already scaled to the exp2 domain, with
// masked entries at -inf.  Rescales o, updates m and l (l is per thread; rows are
// summed across the 4 lanes of a quad at the end), and leaves P in s.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int NT, int ON>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&o)[ON][4], float (&m)[2], float (&l)[2]) {
  float alpha[2];
  bool grew = false;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float mx = -INFINITY;
#pragma unroll
    for (int t = 0; t < NT; ++t) mx = fmaxf(mx, fmaxf(s[t][2 * i], s[t][2 * i + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m[i], mx);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    alpha[i] = fast_exp2(m[i] - m_use);
    grew |= m_new != m[i];
    float sum = 0.f;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      s[t][2 * i] = fast_exp2(s[t][2 * i] - m_use);
      s[t][2 * i + 1] = fast_exp2(s[t][2 * i + 1] - m_use);
      sum += s[t][2 * i] + s[t][2 * i + 1];
    }
    l[i] = l[i] * alpha[i] + sum;
    m[i] = m_new;
  }
  // the running maximum rarely moves after the first tiles: skip the rescale of the
  // output accumulators when no row of the warp needs it
  if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
    for (int t = 0; t < ON; ++t) {
      o[t][0] *= alpha[0];
      o[t][1] *= alpha[0];
      o[t][2] *= alpha[1];
      o[t][3] *= alpha[1];
    }
  }
}

// Copies `n_keys` keys starting at position `key_pos0` of one kv head into a swizzled
// tile at rows row0.., for both K and V, 16 bytes per cp.async.  `tid`/`nthreads`
// enumerate the copying threads.  Keys outside [kv_lo, kv_hi) or in no page are zero.
// `page_shift` >= 0 says page_size == 1 << page_shift (shifts instead of divisions).
template <int D>
__device__ __forceinline__ void load_kv_rows(uint8_t* ks, uint8_t* vs, int row0, int n_keys, int key_pos0, int kv_lo,
                                             int kv_hi, const bf16* __restrict__ kcache,
                                             const bf16* __restrict__ vcache, const int* __restrict__ bt, int nkv,
                                             int kvh, int page_size, int page_shift, int tid, int nthreads) {
  constexpr int CH = D / 8;  // 16-byte chunks per key
  for (int e = tid; e < n_keys * CH; e += nthreads) {
    const int r = e / CH, c = e % CH;
    const int j = key_pos0 + r;
    bool valid = j >= kv_lo && j < kv_hi;
    size_t off = 0;
    if (valid) {
      const int blk = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
      const int in_page = page_shift >= 0 ? (j & (page_size - 1)) : (j % page_size);
      const int page = __ldg(bt + blk);
      valid = page >= 0;
      if (valid) off = (((size_t)page * nkv + kvh) * page_size + in_page) * D + c * 8;
    }
    const uint32_t so = swz<D>(row0 + r, c);
    cp_async16(ks + so, kcache + off, valid);
    cp_async16(vs + so, vcache + off, valid);
  }
}

// The same for one warp's 16 keys when the page of key r is already in lane r's
// register `pg` (-1: no page or outside the request): no dependent load stands between
// the loop and its copies.
template <int D>
__device__ __forceinline__ void load_kv_rows_pg(uint8_t* ks, uint8_t* vs, int key_pos0, int pg,
                                                const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                                                int nkv, int kvh, int page_size, int page_shift, int lane) {
  constexpr int CH = D / 8;
  if (page_shift >= 4) {
    // Pages of 16, 32, 64, ... tokens: the warp's 16 keys (which start at a multiple of 16) lie in
    // ONE page, so the tile has one base address and every copy a fixed offset from it; only
    // whether a key is valid still differs from row to row.
    const int page = __reduce_max_sync(0xffffffffu, lane < 16 ? pg : -1);
    const size_t base = page >= 0 ? (((size_t)page * nkv + kvh) * page_size + (key_pos0 & (page_size - 1))) * D : 0;
    const bf16* kb = kcache + base;
    const bf16* vb = vcache + base;
#pragma unroll
    for (int e0 = 0; e0 < 16 * CH; e0 += 32) {
      const int e = e0 + lane;
      const int r = e / CH, c = e % CH;                    // compile-time shifts: CH is a power of two
      const bool valid = __shfl_sync(0xffffffffu, pg, r) >= 0;
      const int off = valid ? r * D + c * 8 : 0;
      const uint32_t so = swz<D>(r, c);
      cp_async16(ks + so, kb + off, valid);
      cp_async16(vs + so, vb + off, valid);
    }
    return;
  }
#pragma unroll
  for (int e0 = 0; e0 < 16 * CH; e0 += 32) {
    const int e = e0 + lane;
    const int r = e / CH, c = e % CH;
    const int page = __shfl_sync(0xffffffffu, pg, r);
    const int j = key_pos0 + r;
    const int in_page = page_shift >= 0 ? (j & (page_size - 1)) : (j % page_size);
    const bool valid = page >= 0;
    const size_t off = valid ? (((size_t)page * nkv + kvh) * page_size + in_page) * D + c * 8 : 0;
    const uint32_t so = swz<D>(r, c);
    cp_async16(ks + so, kcache + off, valid);
    cp_async16(vs + so, vcache + off, valid);
  }
}

// ---- the decode tile with the KEYS on the MMA's rows (groups of at most 8 query heads) ----------
// With one token per request the queries of a kv head are only its group's heads (4 in Qwen3-8B);
// as MMA rows they would fill 4 of 16.  Transposed, S^T = K Q^T has the 16 keys as rows and the
// heads as the 8 columns of ONE n-tile, and O^T = V^T P^T has the head size as rows: half the
// MMAs and a quarter of the exponentials of the row-major form, and half the accumulators.

// Transposes an 8 x 8 matrix of 16-bit values held one row per 4 lanes (lane l: row l / 4,
// columns 2 (l % 4) and + 1, packed): the C fragment of P^T becomes the B fragment PV needs.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

// S^T (16 keys x 8 heads) = K (16 x D, the tile at ks_addr) * Q^T.  qb: the warp's Q^T fragments
// [D/16][2] (B operand: head lane/4, columns 2 (lane%4) .. of each 8-wide half of the 16 values).
// Two accumulators take alternate steps so that their MMAs do not wait for each other.
template <int D, bool TL = false>
__device__ __forceinline__ void qk_16keys_t(float (&s)[4], const uint32_t (&qb)[D / 16][2], uint32_t ks_addr, int lane) {
  float s2[4] = {0.f, 0.f, 0.f, 0.f};
  const int mi = lane >> 3;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, ks_addr + tile_off<D, TL>((mi & 1) * 8 + (lane & 7), kk * 2 + (mi >> 1)));
    if (kk & 1) mma_bf16(s2, a, qb[kk][0], qb[kk][1]);
    else mma_bf16(s, a, qb[kk][0], qb[kk][1]);
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) s[c] += s2[c];
}
// O^T (D x 8 heads) += V^T (D x 16 keys, from the tile at vs_addr) * P^T (16 keys x 8 heads: pb0, pb1).
template <int D, bool TL = false>
__device__ __forceinline__ void pv_16keys_t(float (&ot)[D / 16][4], uint32_t pb0, uint32_t pb1, uint32_t vs_addr, int lane) {
  const int mi = lane >> 3;
#pragma unroll
  for (int np = 0; np < D / 16; ++np) {
    uint32_t a[4];
    ldmatrix_x4_trans(a, vs_addr + tile_off<D, TL>((mi >> 1) * 8 + (lane & 7), np * 2 + (mi & 1)));
    mma_bf16(ot[np], a, pb0, pb1);
  }
}

// One warp's 16 keys (K and V) by TMA: boxes of [min(page_size, 16) keys][64 values] straight from the
// pages into a tile laid out for tile_off<D, true>, completion counted in bytes on `bar`.  Pages of 8
// tokens take two boxes per 64 columns, pages of 16, 32, ... one.  Lane r < 16 holds the page of key r
// (-1: outside the request or its window, or a page given back): a box is fetched when any of its keys
// has a page, else its rows are zeroed (what shared memory held before must never meet the MMA, where
// 0 x NaN would not be 0).  Called by the whole warp; lane 0 issues.
template <int D>
__device__ __forceinline__ void tma_kv_tile(uint8_t* ks, uint8_t* vs, uint64_t* bar, int key_pos0, int pg,
                                            const CUtensorMap* map_k, const CUtensorMap* map_v, int nkv, int kvh,
                                            int page_size, int lane) {
  constexpr int COLS = D / 64;                       // boxes side by side
  const int box_rows = page_size >= 16 ? 16 : page_size;
  const int n_boxes = 16 / box_rows;
  int box_page[2];
#pragma unroll
  for (int b = 0; b < 2; ++b) {
    // the page of a box: that of any of its keys (they share it); -1 if none has one
    const int lo = b * box_rows, hi = lo + box_rows;
    const int mine = (b < n_boxes && lane >= lo && lane < hi && lane < 16) ? pg : -1;
    box_page[b] = __reduce_max_sync(0xffffffffu, mine);
  }
  int fetched = 0;
#pragma unroll
  for (int b = 0; b < 2; ++b)
    if (b < n_boxes && box_page[b] >= 0) ++fetched;
  if (lane == 0) mbar_expect_tx(bar, (uint32_t)(fetched * 2 * COLS * box_rows * 128));
  __syncwarp();   // the byte count is posted before any copy can complete
  // The copies go out side by side, one per lane in ONE instruction (a thread that issues a tensor copy is
  // held a few hundred nanoseconds while memory is busy): lane = (box, 64-column part, K or V).
  const int per_box = COLS * 2;
  if (lane < n_boxes * per_box) {
    const int bx = lane / per_box, rem = lane % per_box, c = rem >> 1, is_v = rem & 1;
    const int page = bx == 0 ? box_page[0] : box_page[1];
    if (page >= 0) {
      const int row = (page * nkv + kvh) * page_size + ((key_pos0 + bx * box_rows) & (page_size - 1));
      tma_load_2d((is_v ? vs : ks) + c * 2048 + bx * box_rows * 128, is_v ? map_v : map_k, bar, c * 64, row);
    }
  }
#pragma unroll
  for (int bx = 0; bx < 2; ++bx) {
    if (bx >= n_boxes || box_page[bx] >= 0) continue;
    for (int e = lane; e < COLS * box_rows * 8; e += 32) {   // 16-byte chunks of the box's rows
      const int c = e / (box_rows * 8), rem = e % (box_rows * 8);
      const uint32_t off = (uint32_t)(c * 2048 + bx * box_rows * 128 + rem * 16);
      *reinterpret_cast<uint4*>(ks + off) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(vs + off) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // before a later copy lands on these rows
  }
}

// ================================================================================ decode
constexpr int DC_THREADS = 128, DC_WARPS = 4, DC_KEYS = 16, DC_TILE = DC_WARPS * DC_KEYS;
// stages of a warp's private ring: 3 x 8 KB x 4 warps = 96 KB per CTA at d = 128, two CTAs per SM
template <int D> struct DecodeCfg { static constexpr int STAGES = D <= 64 ? 4 : (D <= 128 ? 3 : 2); };

// What the fused form needs to make q, k and v of the step's token itself from the fused
// projection row [q heads | k heads | v heads] (bfloat16, or split-K partial sums).
struct FusedQK {
  const bf16* qkv;          // [T, >= width] or null
  int qkv_stride;
  const float* part;        // [part_splits][T][width] or null
  int part_splits;
  long long part_zstride;
  int width;                // (nq + 2 nkv) * d
  const float* qw;          // per-head RMSNorm weights of q and k, or null
  const float* kw;
  float eps;
  const float* cos_t;       // rotary tables [n_table_pos][d/2], or null
  const float* sin_t;
  int n_table_pos;
  const int* positions;     // [T]
  const int* slots;         // [T] where the token's k and v go (page * page_size + offset)
  bf16* kcache_w;           // the same pages as kcache / vcache, written here
  bf16* vcache_w;
};

// partial[((dec * nkv + kvh) * splits + z) * g + row] holds D output values, then max, then sum.
// FUSED: the kernel also does what qk_norm_rope_store does for its token: every block makes
// the q heads of its group (RMSNorm, rotary) in shared memory; the block of the last split
// makes the token's key and value, writes them to their page, and folds them into its result
// as one more key (the streamed keys then end before the token's own position).
// One unit of decode attention: request `dec`'s token, kv head `kvh`, split `z` of `splits`
// of its keys, by DC_THREADS threads (`tid`) with DC_WARPS private rings in `smem`.
// Sync::sync() is a barrier of exactly these threads.  A caller that runs several units one
// after the other puts a barrier between them (the merge at the end reads all rings).
// STAGES: tiles of a warp's ring (STAGES - 1 in flight); shared memory needed:
// DC_WARPS * STAGES * 2 * DC_KEYS * D * 2 bytes, and for FUSED 16 * D * 2 + (2 D + 16) * 4 more
// (behind the rings, or at `fused_area`, 128-byte aligned).
// TR: the transposed tile (keys on the MMA's rows) for groups of at most 8 query heads; the
// caller chooses it, the results agree with the other form up to rounding.
// TMA: the keys and values come by cp.async.bulk.tensor (tma_kv_tile; pages of 8, 16, 32, ... tokens),
// one lane issuing, completion on a barrier per warp and stage (`bars`, DC_WARPS * STAGES of them, which
// the caller places in shared memory; `smem` is then 1024-byte aligned) with a bounded wait that records
// a code in `status`; else by cp.async from every lane.
template <int D, bool FUSED, class Sync, int STAGES = DecodeCfg<D>::STAGES, bool TR = false, bool TMA = false>
__device__ __forceinline__ void attn_decode_unit(
    uint8_t* smem, int tid, int dec, int kvh, int z, bf16* __restrict__ out, int out_stride,
    float* __restrict__ partial, const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kcache,
    const bf16* __restrict__ vcache, const int* __restrict__ block_tables, int bt_stride,
    const int* __restrict__ cu_q, const int* __restrict__ kv_lens, const int* __restrict__ dec_seq, int nq, int nkv,
    int page_size, int page_shift, int window, float scale_log2, int splits, const FusedQK& fq,
    uint8_t* fused_area = nullptr, const CUtensorMap* map_k = nullptr, const CUtensorMap* map_v = nullptr,
    uint64_t* bars = nullptr, int* status = nullptr) {

  constexpr int ROWS_BYTES = DC_KEYS * D * 2;                  // one warp's 16 keys of K (or V)
  constexpr int WARP_BYTES = STAGES * 2 * ROWS_BYTES;          // a warp's private ring
  const int lane = tid & 31, warp = tid >> 5;
  uint8_t* ring = smem + warp * WARP_BYTES;

  const int seq = dec_seq[dec];
  const int g = nq / nkv;
  const int token = cu_q[seq];
  const int kvlen = kv_lens[seq];
  const int pos = kvlen - 1;
  const int kv_lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int kv_hi = FUSED ? pos : kvlen;     // fused: the token's own key is not in the cache yet
  const int* bt = block_tables + (size_t)seq * bt_stride;

  const int kt0 = (kv_lo / DC_TILE) * DC_TILE;
  const int total_tiles = max(0, (kv_hi - kt0 + DC_TILE - 1) / DC_TILE);
  const int tps = (total_tiles + splits - 1) / splits;
  const int t_begin = z * tps, t_end = min(total_tiles, t_begin + tps);
  const int n_tiles = max(0, t_end - t_begin);

  // Row-major form: Q fragments with the query heads of the group as rows, O as [16 heads][D].
  // Transposed form: Q^T fragments (heads as columns), O^T as [D][8 heads]; m and l then belong to
  // the thread's two head columns 2 (lane % 4) and + 1.
  uint32_t qf[TR ? 1 : D / 16][4];
  float o[TR ? 1 : D / 8][4];
  uint32_t qb[TR ? D / 16 : 1][2];
  float ot[TR ? D / 16 : 1][4];
  if constexpr (TR) {
#pragma unroll
    for (int t = 0; t < D / 16; ++t) ot[t][0] = ot[t][1] = ot[t][2] = ot[t][3] = 0.f;
  } else {
#pragma unroll
    for (int t = 0; t < D / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  // Lane r (r < 16) looks up the page of key r of a tile one iteration before the tile's
  // copies are issued, so the block-table load is never waited for inside the loop.
  auto lookup = [&](int t) -> int {
    const int j = kt0 + (t_begin + t) * DC_TILE + warp * DC_KEYS + (lane & 15);
    if (t >= n_tiles || j < kv_lo || j >= kv_hi) return -1;
    return __ldg(bt + (page_shift >= 0 ? (j >> page_shift) : (j / page_size)));
  };
  uint64_t* my_bars = TMA ? bars + warp * STAGES : nullptr;
  if (TMA) {
    if (lane == 0) {
#pragma unroll
      for (int st = 0; st < STAGES; ++st) mbar_init(&my_bars[st], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
  }
  auto issue = [&](int t, int pg) {   // this warp's 16 keys of tile t into stage t % STAGES
    uint8_t* ks = ring + (t % STAGES) * 2 * ROWS_BYTES;
    const int key0 = kt0 + (t_begin + t) * DC_TILE + warp * DC_KEYS;
    if constexpr (TMA)
      tma_kv_tile<D>(ks, ks + ROWS_BYTES, &my_bars[t % STAGES], key0, pg, map_k, map_v, nkv, kvh, page_size, lane);
    else
      load_kv_rows_pg<D>(ks, ks + ROWS_BYTES, key0, pg, kcache, vcache, nkv, kvh, page_size, page_shift, lane);
  };
  // Not fused: the kernel before this one wrote the newest token's key and value (and q).  The first
  // tiles are asked for before the wait for it unless they may hold that key.
  const bool early = !FUSED && kt0 + (t_begin + STAGES - 1) * DC_TILE <= pos;
  if (!FUSED && !early) pdl_wait();
  int pg_next = lookup(0);
#pragma unroll
  for (int t = 0; t < STAGES - 1; ++t) {
    const int pg = pg_next;
    pg_next = lookup(t + 1);
    if (t < n_tiles) issue(t, pg);
    if constexpr (!TMA) cp_async_commit();
  }
  if (!FUSED && TR) {
    if (early) pdl_wait();
    const int hq = lane >> 2;   // the head (column of Q^T) this lane holds
    const bf16* qp = q + (size_t)token * q_stride + (size_t)(kvh * g + hq) * D + 2 * (lane & 3);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      qb[kk][0] = hq < g ? *reinterpret_cast<const uint32_t*>(qp + kk * 16) : 0u;
      qb[kk][1] = hq < g ? *reinterpret_cast<const uint32_t*>(qp + kk * 16 + 8) : 0u;
    }
  }
  if (!FUSED && !TR) {
    if (early) pdl_wait();
    const int r0 = lane >> 2, r1 = r0 + 8;
    const bf16* q0p = q + (size_t)token * q_stride + (size_t)(kvh * g + r0) * D + 2 * (lane & 3);
    const bf16* q1p = q + (size_t)token * q_stride + (size_t)(kvh * g + r1) * D + 2 * (lane & 3);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      qf[kk][0] = r0 < g ? *reinterpret_cast<const uint32_t*>(q0p + kk * 16) : 0u;
      qf[kk][1] = r1 < g ? *reinterpret_cast<const uint32_t*>(q1p + kk * 16) : 0u;
      qf[kk][2] = r0 < g ? *reinterpret_cast<const uint32_t*>(q0p + kk * 16 + 8) : 0u;
      qf[kk][3] = r1 < g ? *reinterpret_cast<const uint32_t*>(q1p + kk * 16 + 8) : 0u;
    }
  }
  // ---- fused: q (all blocks) and the token's own k, v (block of the last split), while the
  // first tiles are on their way
  // q tile [16][D] bf16 (swizzled), then floats: behind the rings unless the caller has another place
  uint8_t* fused_smem = fused_area ? fused_area : smem + DC_WARPS * WARP_BYTES;
  float* knew = reinterpret_cast<float*>(fused_smem + 16 * D * 2);   // [D] own key, as stored (bf16-rounded)
  float* vnew = knew + D;                                            // [D] own value, as stored
  float* snew = vnew + D;                                            // [16] own key's score per head, exp2 domain
  const bool owner = FUSED && z == splits - 1;
  if (FUSED) {
    // Everything above read only the step's own arrays and pages that earlier steps wrote; the
    // projection rows below come from the kernel before this one.
    pdl_wait();
    constexpr int HALF = D / 2, MAXP = HALF / 32 > 0 ? HALF / 32 : 1;
    const int my_pos = min(fq.positions[token], fq.n_table_pos - 1);
    // Heads of this block: g query heads, then (owner only) the key head and the value head.
    // Warp w takes heads w, w + 4, ...: first ALL loads of all its heads (one trip to memory, not
    // one per head), then the norms and rotations.
    constexpr int MAXH = (16 + 2 + DC_WARPS - 1) / DC_WARPS;
    float a[MAXH][MAXP], b[MAXH][MAXP];
    int which[MAXH];   // 0 q head, 1 key, 2 value, -1 nothing
#pragma unroll
    for (int k = 0; k < MAXH; ++k) {
      const int hh = warp + k * DC_WARPS;
      which[k] = hh < g ? 0 : (hh == 16 && owner ? 1 : (hh == 17 && owner ? 2 : -1));
#pragma unroll
      for (int j = 0; j < MAXP; ++j) a[k][j] = b[k][j] = 0.f;
    }
    auto head_col_of = [&](int k) -> int {
      const int hh = warp + k * DC_WARPS;
      return which[k] == 0 ? (kvh * g + hh) * D : (which[k] == 1 ? (nq + kvh) * D : (nq + nkv + kvh) * D);
    };
    if (fq.part) {
      for (int zz = 0; zz < fq.part_splits; ++zz) {
        const float* p = fq.part + (size_t)zz * fq.part_zstride + (size_t)token * fq.width;
#pragma unroll
        for (int k = 0; k < MAXH; ++k) {
          if (which[k] < 0) continue;
          const float* ph = p + head_col_of(k);
#pragma unroll
          for (int j = 0; j < MAXP; ++j) {
            const int i = lane + 32 * j;
            if (i < HALF) {
              a[k][j] += ph[i];
              b[k][j] += ph[i + HALF];
            }
          }
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < MAXH; ++k) {
        if (which[k] < 0) continue;
        const bf16* ph = fq.qkv + (size_t)token * fq.qkv_stride + head_col_of(k);
#pragma unroll
        for (int j = 0; j < MAXP; ++j) {
          const int i = lane + 32 * j;
          if (i < HALF) {
            a[k][j] = __bfloat162float(ph[i]);
            b[k][j] = __bfloat162float(ph[i + HALF]);
          }
        }
      }
    }
    // norm weights and rotation of this lane's elements (the same for every head of a kind)
    float wq[2][MAXP], wk[2][MAXP], cs[MAXP], sn[MAXP];
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
      const int i = lane + 32 * j;
      const bool in = i < HALF;
      wq[0][j] = in && fq.qw ? fq.qw[i] : 1.f;
      wq[1][j] = in && fq.qw ? fq.qw[i + HALF] : 1.f;
      wk[0][j] = in && fq.kw ? fq.kw[i] : 1.f;
      wk[1][j] = in && fq.kw ? fq.kw[i + HALF] : 1.f;
      cs[j] = in && fq.cos_t ? fq.cos_t[(size_t)my_pos * HALF + i] : 1.f;
      sn[j] = in && fq.cos_t ? fq.sin_t[(size_t)my_pos * HALF + i] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < MAXH; ++k) {
      const int hh = warp + k * DC_WARPS;
      if (hh >= g && hh < 16) {   // rows of the q tile beyond the group are zero
        for (int c = lane; c < D / 8; c += 32) *reinterpret_cast<uint4*>(fused_smem + swz<D>(hh, c)) = make_uint4(0, 0, 0, 0);
        continue;
      }
      if (which[k] < 0) continue;
      if (which[k] == 2) {
#pragma unroll
        for (int j = 0; j < MAXP; ++j) {
          const int i = lane + 32 * j;
          if (i < HALF) {
            vnew[i] = __bfloat162float(__float2bfloat16_rn(a[k][j]));
            vnew[i + HALF] = __bfloat162float(__float2bfloat16_rn(b[k][j]));
          }
        }
        continue;
      }
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < MAXP; ++j) {
        ss = sum_squares_step(ss, a[k][j], b[k][j]);   // lanes beyond HALF hold zeros
      }
      const bool normed = which[k] == 0 ? fq.qw != nullptr : fq.kw != nullptr;
      float inv = 1.f;
      if (normed) {
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)D + fq.eps);
      }
#pragma unroll
      for (int j = 0; j < MAXP; ++j) {
        const int i = lane + 32 * j;
        if (i >= HALF) continue;
        float x = a[k][j], y = b[k][j];
        if (normed) {
          x = norm_scale(x, which[k] == 0 ? wq[0][j] : wk[0][j], inv);
          y = norm_scale(y, which[k] == 0 ? wq[1][j] : wk[1][j], inv);
        }
        if (fq.cos_t) rotate_pair(x, y, cs[j], sn[j]);
        if (which[k] == 0) {
          // element i of row hh lies in chunk i / 8 at offset i % 8 of the swizzled tile
          *reinterpret_cast<bf16*>(fused_smem + swz<D>(hh, i >> 3) + (i & 7) * 2) = __float2bfloat16_rn(x);
          *reinterpret_cast<bf16*>(fused_smem + swz<D>(hh, (i + HALF) >> 3) + ((i + HALF) & 7) * 2) = __float2bfloat16_rn(y);
        } else {
          knew[i] = __bfloat162float(__float2bfloat16_rn(x));
          knew[i + HALF] = __bfloat162float(__float2bfloat16_rn(y));
        }
      }
    }
    Sync::sync();
    if (owner) {
      // the token's key and value go to their page; their score against every head of the group
      const int slot = fq.slots[token];
      if (slot >= 0) {
        const size_t off = (((size_t)(slot / page_size) * nkv + kvh) * page_size + (slot % page_size)) * D;
        for (int i = tid; i < D; i += DC_THREADS) {
          fq.kcache_w[off + i] = __float2bfloat16_rn(knew[i]);
          fq.vcache_w[off + i] = __float2bfloat16_rn(vnew[i]);
        }
      }
      for (int r = warp; r < g; r += DC_WARPS) {
        float dot = 0.f;
        for (int i = lane; i < D; i += 32)
          dot += __bfloat162float(*reinterpret_cast<const bf16*>(fused_smem + swz<D>(r, i >> 3) + (i & 7) * 2)) * knew[i];
        dot = warp_sum(dot);
        if (lane == 0) snew[r] = dot * scale_log2;
      }
    }
    if constexpr (TR) {
      // rows 0..7 of the q tile are the heads; matrix i of a load is the 16-byte chunk 2 kk + i
#pragma unroll
      for (int kk = 0; kk < D / 16; kk += 2) {
        uint32_t r[4];
        ldmatrix_x4(r, smem_addr(fused_smem) + swz<D>(lane & 7, kk * 2 + (lane >> 3)));
        qb[kk][0] = r[0];
        qb[kk][1] = r[1];
        qb[kk + 1][0] = r[2];
        qb[kk + 1][1] = r[3];
      }
    } else {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const int mtx = lane >> 3;
        ldmatrix_x4(qf[kk], smem_addr(fused_smem) + swz<D>((mtx & 1) * 8 + (lane & 7), kk * 2 + (mtx >> 1)));
      }
    }
  }

  for (int t = 0; t < n_tiles; ++t) {
    {
      const int tt = t + STAGES - 1;
      const int pg = pg_next;
      pg_next = lookup(tt + 1);
      if (tt < n_tiles) issue(tt, pg);
    }
    if constexpr (TMA) {
      // the tile's bytes have landed when its barrier's phase completes (bounded wait)
      if (!mbar_wait(&my_bars[t % STAGES], (uint32_t)(t / STAGES) & 1u)) {
        if (lane == 0 && status) atomicExch(status, 21);
        for (int i = 0; i < 64; ++i) __nanosleep(10000);   // let copies in flight land before the ring is reused
        break;
      }
    } else {
      cp_async_commit();
      cp_async_wait<STAGES - 1>();
    }
    __syncwarp();
    const int key0 = kt0 + (t_begin + t) * DC_TILE + warp * DC_KEYS;
    if (key0 < kv_hi && key0 + DC_KEYS > kv_lo) {
      const uint32_t ks_addr = smem_addr(ring + (t % STAGES) * 2 * ROWS_BYTES), vs_addr = ks_addr + ROWS_BYTES;
      const bool need_mask = key0 + DC_KEYS > kv_hi || key0 < kv_lo;
      if constexpr (TR) {
        float st[4] = {0.f, 0.f, 0.f, 0.f};   // keys lane/4 (st[0], st[1]) and + 8 (st[2], st[3]) x heads 2 (lane%4), + 1
        qk_16keys_t<D, TMA>(st, qb, ks_addr, lane);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float v = st[c] * scale_log2;
          if (need_mask) {
            const int j = key0 + (lane >> 2) + (c >> 1) * 8;
            if (j >= kv_hi || j < kv_lo) v = -INFINITY;
          }
          st[c] = v;
        }
        // online softmax down the key rows: the maximum of a head's column lies across the 8 lanes
        // that share lane % 4; the sums stay per thread until the end
        float alpha[2];
        bool grew = false;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          float mx = fmaxf(st[i], st[2 + i]);
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
          const float m_new = fmaxf(m[i], mx);
          const float m_use = m_new == -INFINITY ? 0.f : m_new;
          alpha[i] = fast_exp2(m[i] - m_use);
          grew |= m_new != m[i];
          st[i] = fast_exp2(st[i] - m_use);
          st[2 + i] = fast_exp2(st[2 + i] - m_use);
          l[i] = l[i] * alpha[i] + st[i] + st[2 + i];
          m[i] = m_new;
        }
        if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
          for (int np = 0; np < D / 16; ++np) {
            ot[np][0] *= alpha[0];
            ot[np][1] *= alpha[1];
            ot[np][2] *= alpha[0];
            ot[np][3] *= alpha[1];
          }
        }
        const uint32_t pb0 = movmatrix_trans(pack_bf16(st[0], st[1]));   // keys 0..7 of the tile
        const uint32_t pb1 = movmatrix_trans(pack_bf16(st[2], st[3]));   // keys 8..15
        pv_16keys_t<D, TMA>(ot, pb0, pb1, vs_addr, lane);
      } else {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      qk_16keys<D, TMA>(s, qf, ks_addr, 0, lane);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float v = s[nt][c] * scale_log2;
          if (need_mask) {
            const int j = key0 + nt * 8 + 2 * (lane & 3) + (c & 1);
            if (j >= kv_hi || j < kv_lo) v = -INFINITY;
          }
          s[nt][c] = v;
        }
      softmax_step<2, D / 8>(s, o, m, l);
      uint32_t pf[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]), pack_bf16(s[1][0], s[1][1]),
                        pack_bf16(s[1][2], s[1][3])};
      pv_16keys<D, TMA>(o, pf, vs_addr, 0, lane);
      }
    }
    __syncwarp();  // the stage is refilled by this warp's next issue
  }
  if constexpr (!TMA) cp_async_wait<0>();

  // merge the four warps: each writes (o, m, l) of its rows to its own ring, then all combine
  __syncwarp();
  float* wo = reinterpret_cast<float*>(ring);               // [16][D] then m[16], l[16]
  static_assert(WARP_BYTES >= (16 * D + 32) * 4, "a warp's ring must hold its partial result");
  if constexpr (TR) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {   // a head's sum lies across the 8 lanes that share lane % 4
      l[i] += __shfl_xor_sync(0xffffffffu, l[i], 4);
      l[i] += __shfl_xor_sync(0xffffffffu, l[i], 8);
      l[i] += __shfl_xor_sync(0xffffffffu, l[i], 16);
    }
    const int h0 = 2 * (lane & 3), d0 = lane >> 2;
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      wo[h0 * D + np * 16 + d0] = ot[np][0];
      wo[(h0 + 1) * D + np * 16 + d0] = ot[np][1];
      wo[h0 * D + np * 16 + d0 + 8] = ot[np][2];
      wo[(h0 + 1) * D + np * 16 + d0 + 8] = ot[np][3];
    }
    if (lane < 4) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        wo[16 * D + h0 + i] = m[i];
        wo[16 * D + 16 + h0 + i] = l[i];
      }
    }
  } else {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = (lane >> 2) + i * 8;
#pragma unroll
    for (int t = 0; t < D / 8; ++t) {
      wo[r * D + t * 8 + 2 * (lane & 3)] = o[t][2 * i];
      wo[r * D + t * 8 + 2 * (lane & 3) + 1] = o[t][2 * i + 1];
    }
    if ((lane & 3) == 0) {
      wo[16 * D + r] = m[i];
      wo[16 * D + 16 + r] = l[i];
    }
  }
  }
  Sync::sync();
  for (int e = tid; e < g * D; e += DC_THREADS) {
    const int r = e / D, c = e % D;
    float mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) mt = fmaxf(mt, reinterpret_cast<float*>(smem + w * WARP_BYTES)[16 * D + r]);
    if (owner) mt = fmaxf(mt, snew[r]);
    float acc = 0.f, lt = 0.f;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) {
      const float* p = reinterpret_cast<float*>(smem + w * WARP_BYTES);
      const float mw = p[16 * D + r];
      const float sc = mw == -INFINITY ? 0.f : exp2f(mw - mt);
      acc += p[r * D + c] * sc;
      lt += p[16 * D + 16 + r] * sc;
    }
    if (owner) {   // the token's own key: one more partial with sum 1 and its value as output
      const float sc = exp2f(snew[r] - mt);
      acc += vnew[c] * sc;
      lt += sc;
    }
    if (partial) {
      float* dst = partial + ((((size_t)dec * nkv + kvh) * splits + z) * g + r) * (D + 2);
      dst[c] = acc;
      if (c == 0) {
        dst[D] = mt;
        dst[D + 1] = lt;
      }
    } else {
      out[(size_t)token * out_stride + (size_t)(kvh * g + r) * D + c] = __float2bfloat16_rn(lt > 0.f ? acc / lt : 0.f);
    }
  }
}

// Combines the splits of one (request, query head) in split order; `nthreads` threads.
// (`partial` may have been written earlier in the same kernel: no read-only loads of it.)
template <int D>
__device__ __forceinline__ void attn_decode_combine_item(int dec, int h, int tid, int nthreads, bf16* __restrict__ out,
                                                         int out_stride, const float* partial, int token, int nq,
                                                         int nkv, int splits) {
  const int g = nq / nkv, kvh = h / g, r = h % g;
  const float* base = partial + ((((size_t)dec * nkv + kvh) * splits) * g + r) * (D + 2);
  const size_t zstride = (size_t)g * (D + 2);
  if (splits <= 32) {
    // Lane z holds split z's maximum and sum: one trip to memory for all of them, and the loads of
    // the outputs go out eight at a time (a loop that waits for each split in turn costs 0.3 us a split).
    const int lane = tid & 31;
    const float mz = lane < splits ? base[lane * zstride + D] : -INFINITY;
    const float lz = lane < splits ? base[lane * zstride + D + 1] : 0.f;
    float mt = mz;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
    const float sc = mz == -INFINITY ? 0.f : exp2f(mz - mt);
    float lt = 0.f;
    for (int z = 0; z < splits; ++z) lt += __shfl_sync(0xffffffffu, lz * sc, z);   // in split order
    for (int c = tid; c < D; c += nthreads) {   // whole warps run this loop together (D is a multiple of nthreads or the reverse)
      float acc = 0.f;
      for (int z0 = 0; z0 < splits; z0 += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = z0 + j < splits ? base[(z0 + j) * zstride + c] : 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += v[j] * __shfl_sync(0xffffffffu, sc, (z0 + j) & 31);
      }
      out[(size_t)token * out_stride + (size_t)h * D + c] = __float2bfloat16_rn(lt > 0.f ? acc / lt : 0.f);
    }
    return;
  }
  float mt = -INFINITY;
  for (int z = 0; z < splits; ++z) mt = fmaxf(mt, base[z * zstride + D]);
  for (int c = tid; c < D; c += nthreads) {
    float acc = 0.f, lt = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float mz = base[z * zstride + D];
      const float sc = mz == -INFINITY ? 0.f : exp2f(mz - mt);
      acc += base[z * zstride + c] * sc;
      lt += base[z * zstride + D + 1] * sc;
    }
    out[(size_t)token * out_stride + (size_t)h * D + c] = __float2bfloat16_rn(lt > 0.f ? acc / lt : 0.f);
  }
}

inline int log2_or_minus1(int v) {
  for (int s = 0; s < 31; ++s)
    if ((1 << s) == v) return s;
  return -1;
}

}  // namespace
