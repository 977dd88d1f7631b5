// The host side of the engine's hot path, native: page pools, the cache manager's
// bookkeeping (which pages and which state slot each request holds, per group of layers
// with the same need), and the flattening of a step's batch into the one int32 buffer
// that is copied to the device.  Python keeps the interfaces (zinfer_b200/cache,
// zinfer_b200/engine/batch.py) and calls in here through ctypes; nothing in this file
// touches the GPU, so it runs and is tested without one.
//
// The reference has no counterpart for pages (it preallocates one contiguous cache per
// request, src/model/runtime/optimized_kv_cache/cache.zig:38-84) and forwards one token of
// one request at a time (src/model/runtime/optimized_decoder/batch.zig:116-136); its
// runtime around the kernels is native code, which is why this one is too.
//
// Errors: functions return >= 0 on success and a negative code otherwise; the message is
// in zi_last_error().  The Python side turns codes into its exceptions.
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>

extern "C" const char* zi_last_error();
int zi_refuse(const char* fmt, ...);

namespace {

constexpr int ERR_OUT_OF_PAGES = -2;   // not enough free pages or slots; nothing was taken
constexpr int ERR_NOT_LIVE = -3;       // no such request (freed twice?)
constexpr int ERR_ALREADY_LIVE = -4;
constexpr int ERR_BAD_PAGE = -5;       // a page that is not in use (freed twice, or never allocated)
constexpr int ERR_RELEASED = -6;       // a position lies in a page already given back
constexpr int ERR_CHECK = -7;          // the bookkeeping is inconsistent
constexpr int ERR_ARGUMENT = -8;
constexpr int ERR_NAMED_TWICE = -9;   // a page named twice in one free

// A pool of equal pages (or slots) with a free list.  Pages freed last are handed out
// first, so reuse is immediate and a fault from stale contents shows at once.
struct Pool {
  int num_pages = 0;
  std::vector<int> free_list;      // back() is handed out next
  std::vector<uint8_t> used, ever;
  long long n_used = 0, reused = 0;

  void init(int n) {
    num_pages = n;
    free_list.resize(n);
    for (int i = 0; i < n; ++i) free_list[i] = n - 1 - i;   // pops 0, 1, 2, ... first
    used.assign(n, 0);
    ever.assign(n, 0);
    n_used = reused = 0;
  }
  int num_free() const { return (int)free_list.size(); }
  // n pages into out, or false with the pool unchanged
  bool alloc(int n, int* out) {
    if (n < 0 || n > num_free()) return false;
    for (int i = 0; i < n; ++i) {
      const int p = free_list.back();
      free_list.pop_back();
      used[p] = 1;
      reused += ever[p];
      ever[p] = 1;
      out[i] = p;
    }
    n_used += n;
    return true;
  }
  // 0, or the code with the pool unchanged; *bad receives the offending page
  int release(const int* pages, int n, int* bad) {
    for (int i = 0; i < n; ++i) {
      const int p = pages[i];
      const bool in_range = p >= 0 && p < num_pages;
      if (!in_range || used[p] != 1) {          // 0: not in use; 2: named earlier in this call
        const int code = in_range && used[p] == 2 ? ERR_NAMED_TWICE : ERR_BAD_PAGE;
        for (int j = 0; j < i; ++j) used[pages[j]] = 1;
        *bad = p;
        return code;
      }
      used[p] = 2;
    }
    for (int i = 0; i < n; ++i) {
      used[pages[i]] = 0;
      free_list.push_back(pages[i]);
    }
    n_used -= n;
    return 0;
  }
  bool check(std::string* why) const {
    std::vector<uint8_t> seen(num_pages, 0);
    for (int p : free_list) {
      if (p < 0 || p >= num_pages) { *why = "a page outside the pool is on the free list"; return false; }
      if (seen[p]) { *why = "a page is on the free list twice"; return false; }
      if (used[p]) { *why = "a page is both free and in use"; return false; }
      seen[p] = 1;
    }
    long long u = 0;
    for (int p = 0; p < num_pages; ++p) u += used[p] ? 1 : 0;
    if (u != n_used) { *why = "the count of pages in use is wrong"; return false; }
    if ((long long)free_list.size() + u != num_pages) { *why = "a page was lost"; return false; }
    return true;
  }
};

struct Group {
  int window = 0;   // 0: every key stays visible
  Pool pool;
};

struct Request {
  int slot = -1;
  long long length = 0;                    // tokens committed to the cache
  std::vector<std::vector<int>> tables;    // per group: page per block, -1 once released
};

struct Cache {
  int page_size = 16, max_requests = 0;
  std::vector<Group> groups;
  Pool slots;
  std::unordered_map<long long, Request> requests;

  int blocks_for(long long tokens) const { return (int)((tokens + page_size - 1) / page_size); }
  Request* find(long long id) {
    auto it = requests.find(id);
    return it == requests.end() ? nullptr : &it->second;
  }
  // pages each group must still take so that n_new more tokens fit
  void pages_needed(const Request& r, long long n_new, int* out) const {
    const int want = blocks_for(r.length + n_new);
    for (size_t g = 0; g < groups.size(); ++g) out[g] = std::max(0, want - (int)r.tables[g].size());
  }
};

Cache* as_cache(void* h) { return reinterpret_cast<Cache*>(h); }

}  // namespace

// ------------------------------------------------------------------------------- pools
extern "C" void* zi_pool_create(int num_pages) {
  if (num_pages < 0) return nullptr;
  Pool* p = new Pool();
  p->init(num_pages);
  return p;
}
extern "C" void zi_pool_destroy(void* h) { delete reinterpret_cast<Pool*>(h); }
extern "C" int zi_pool_alloc(void* h, int n, int* out) {
  Pool* p = reinterpret_cast<Pool*>(h);
  if (n < 0) return zi_refuse("cannot allocate a negative number of pages"), ERR_ARGUMENT;
  return p->alloc(n, out) ? n : ERR_OUT_OF_PAGES;
}
extern "C" int zi_pool_free(void* h, const int* pages, int n, int* bad) {
  return reinterpret_cast<Pool*>(h)->release(pages, n, bad);
}
// out: pages, free, used, allocations that returned a page used before
extern "C" void zi_pool_stats(void* h, long long* out) {
  Pool* p = reinterpret_cast<Pool*>(h);
  out[0] = p->num_pages;
  out[1] = p->num_free();
  out[2] = p->n_used;
  out[3] = p->reused;
}
extern "C" int zi_pool_check(void* h) {
  std::string why;
  if (!reinterpret_cast<Pool*>(h)->check(&why)) return zi_refuse("%s", why.c_str()), ERR_CHECK;
  return 0;
}
extern "C" int zi_pool_in_use(void* h, int page) {
  Pool* p = reinterpret_cast<Pool*>(h);
  return page >= 0 && page < p->num_pages && p->used[page] ? 1 : 0;
}

// ------------------------------------------------------------------------------- cache
// windows[g]: 0 for a group whose keys all stay visible, else the window in tokens.
extern "C" void* zi_cache_create(int n_groups, const int* windows, const int* num_pages, int page_size,
                                 int max_requests) {
  if (n_groups < 0 || page_size <= 0 || max_requests < 0) return nullptr;
  Cache* c = new Cache();
  c->page_size = page_size;
  c->max_requests = max_requests;
  c->groups.resize(n_groups);
  for (int g = 0; g < n_groups; ++g) {
    c->groups[g].window = windows[g];
    c->groups[g].pool.init(num_pages[g]);
  }
  c->slots.init(max_requests);
  return c;
}
extern "C" void zi_cache_destroy(void* h) { delete as_cache(h); }

// The request's state slot, or a negative code.
extern "C" int zi_cache_add(void* h, long long id) {
  Cache* c = as_cache(h);
  if (c->find(id)) return ERR_ALREADY_LIVE;
  int slot = -1;
  if (!c->slots.alloc(1, &slot)) return ERR_OUT_OF_PAGES;
  Request r;
  r.slot = slot;
  r.tables.resize(c->groups.size());
  c->requests.emplace(id, std::move(r));
  return slot;
}

// Gives back everything the request holds.  released (may be null): up to cap (group, page) pairs.
// Returns the number of pages given back.
extern "C" int zi_cache_free(void* h, long long id, int* released, int cap) {
  Cache* c = as_cache(h);
  Request* r = c->find(id);
  if (!r) return ERR_NOT_LIVE;
  int n_out = 0, bad = -1;
  std::vector<int> pages;
  for (size_t g = 0; g < c->groups.size(); ++g) {
    pages.clear();
    for (int p : r->tables[g])
      if (p >= 0) pages.push_back(p);
    const int rc = c->groups[g].pool.release(pages.data(), (int)pages.size(), &bad);
    if (rc != 0) return zi_refuse("request %lld holds page %d of group %zu, which is not in use", id, bad, g), ERR_CHECK;
    for (int p : pages) {
      if (released && 2 * n_out + 1 < cap) {
        released[2 * n_out] = (int)g;
        released[2 * n_out + 1] = p;
      }
      ++n_out;
    }
  }
  const int slot = r->slot;
  if (c->slots.release(&slot, 1, &bad) != 0) return zi_refuse("request %lld holds slot %d, which is not in use", id, slot), ERR_CHECK;
  c->requests.erase(id);
  return n_out;
}

extern "C" int zi_cache_has(void* h, long long id) { return as_cache(h)->find(id) ? 1 : 0; }
extern "C" long long zi_cache_length(void* h, long long id) {
  Request* r = as_cache(h)->find(id);
  return r ? r->length : (long long)ERR_NOT_LIVE;
}
extern "C" int zi_cache_slot(void* h, long long id) {
  Request* r = as_cache(h)->find(id);
  return r ? r->slot : ERR_NOT_LIVE;
}
extern "C" int zi_cache_num_requests(void* h) { return (int)as_cache(h)->requests.size(); }

extern "C" int zi_cache_pages_needed(void* h, long long id, long long n_new, int* out) {
  Cache* c = as_cache(h);
  Request* r = c->find(id);
  if (!r) return ERR_NOT_LIVE;
  c->pages_needed(*r, n_new, out);
  return 0;
}
extern "C" int zi_cache_can_reserve(void* h, long long id, long long n_new) {
  Cache* c = as_cache(h);
  Request* r = c->find(id);
  if (!r) return ERR_NOT_LIVE;
  const int want = c->blocks_for(r->length + n_new);
  for (size_t g = 0; g < c->groups.size(); ++g)
    if (std::max(0, want - (int)r->tables[g].size()) > c->groups[g].pool.num_free()) return 0;
  return 1;
}
// Pages for positions length .. length + n_new - 1 in every group, or ERR_OUT_OF_PAGES with
// nothing taken (info: the group that ran out, pages wanted there, pages free there).
extern "C" int zi_cache_reserve(void* h, long long id, long long n_new, int* info) {
  Cache* c = as_cache(h);
  Request* r = c->find(id);
  if (!r) return ERR_NOT_LIVE;
  const int want = c->blocks_for(r->length + n_new);
  for (size_t g = 0; g < c->groups.size(); ++g) {
    const int need = std::max(0, want - (int)r->tables[g].size());
    if (need > c->groups[g].pool.num_free()) {
      if (info) {
        info[0] = (int)g;
        info[1] = need;
        info[2] = c->groups[g].pool.num_free();
      }
      return ERR_OUT_OF_PAGES;
    }
  }
  for (size_t g = 0; g < c->groups.size(); ++g) {
    const int need = std::max(0, want - (int)r->tables[g].size());
    const size_t old = r->tables[g].size();
    r->tables[g].resize(old + need);
    c->groups[g].pool.alloc(need, r->tables[g].data() + old);
  }
  return 0;
}
// All-or-nothing over several requests: counts first, then takes.  info as above.
extern "C" int zi_cache_reserve_all(void* h, int n, const long long* ids, const long long* n_new, int* info) {
  Cache* c = as_cache(h);
  std::vector<long long> need(c->groups.size(), 0);
  for (int i = 0; i < n; ++i) {
    Request* r = c->find(ids[i]);
    if (!r) return ERR_NOT_LIVE;
    const int want = c->blocks_for(r->length + n_new[i]);
    for (size_t g = 0; g < c->groups.size(); ++g) need[g] += std::max(0, want - (int)r->tables[g].size());
  }
  for (size_t g = 0; g < c->groups.size(); ++g)
    if (need[g] > c->groups[g].pool.num_free()) {
      if (info) {
        info[0] = (int)g;
        info[1] = (int)need[g];
        info[2] = c->groups[g].pool.num_free();
      }
      return ERR_OUT_OF_PAGES;
    }
  for (int i = 0; i < n; ++i) zi_cache_reserve(h, ids[i], n_new[i], nullptr);
  return 0;
}
// The step wrote n_new tokens.  Gives back the pages that every window has passed; released (may be
// null) receives up to cap (group, page) pairs.  Returns how many pages were given back.
extern "C" int zi_cache_commit(void* h, long long id, long long n_new, int* released, int cap) {
  Cache* c = as_cache(h);
  Request* r = c->find(id);
  if (!r) return ERR_NOT_LIVE;
  r->length += n_new;
  int n_out = 0, bad = -1;
  for (size_t g = 0; g < c->groups.size(); ++g) {
    const int window = c->groups[g].window;
    if (window <= 0) continue;
    // the next query sits at position `length`; it reads keys > length - window
    const long long first_needed = r->length - window + 1;
    const long long n_dead = first_needed > 0 ? first_needed / c->page_size : 0;
    std::vector<int>& table = r->tables[g];
    for (long long b = 0; b < n_dead && b < (long long)table.size(); ++b) {
      if (table[b] < 0) continue;
      const int p = table[b];
      if (c->groups[g].pool.release(&p, 1, &bad) != 0) return zi_refuse("page %d of group %zu is not in use", p, g), ERR_CHECK;
      if (released && 2 * n_out + 1 < cap) {
        released[2 * n_out] = (int)g;
        released[2 * n_out + 1] = p;
      }
      ++n_out;
      table[b] = -1;
    }
  }
  return n_out;
}
extern "C" int zi_cache_table_len(void* h, long long id, int group) {
  Cache* c = as_cache(h);
  Request* r = c->find(id);
  if (!r) return ERR_NOT_LIVE;
  if (group < 0 || group >= (int)c->groups.size()) return ERR_ARGUMENT;
  return (int)r->tables[group].size();
}
extern "C" int zi_cache_table(void* h, long long id, int group, int* out, int cap) {
  Cache* c = as_cache(h);
  Request* r = c->find(id);
  if (!r) return ERR_NOT_LIVE;
  if (group < 0 || group >= (int)c->groups.size()) return ERR_ARGUMENT;
  const int n = std::min(cap, (int)r->tables[group].size());
  if (n > 0) memcpy(out, r->tables[group].data(), (size_t)n * sizeof(int));
  return (int)r->tables[group].size();
}
// Flat slot (page * page_size + offset) of positions start .. start + n - 1.
extern "C" int zi_cache_slots_for(void* h, long long id, int group, long long start, int n, int* out) {
  Cache* c = as_cache(h);
  Request* r = c->find(id);
  if (!r) return ERR_NOT_LIVE;
  if (group < 0 || group >= (int)c->groups.size()) return ERR_ARGUMENT;
  const std::vector<int>& table = r->tables[group];
  for (int i = 0; i < n; ++i) {
    const long long pos = start + i;
    const long long b = pos / c->page_size;
    if (b >= (long long)table.size()) return zi_refuse("position %lld has no page yet", pos), ERR_ARGUMENT;
    if (table[b] < 0) return zi_refuse("position %lld lies in a page already given back", pos), ERR_RELEASED;
    out[i] = table[b] * c->page_size + (int)(pos % c->page_size);
  }
  return 0;
}
// group >= 0: that group's page pool; -1: the request slots.  out as zi_pool_stats.
extern "C" int zi_cache_pool_stats(void* h, int group, long long* out) {
  Cache* c = as_cache(h);
  if (group >= (int)c->groups.size()) return ERR_ARGUMENT;
  zi_pool_stats(group < 0 ? (void*)&c->slots : (void*)&c->groups[group].pool, out);
  return 0;
}
// No page lost, held twice or freed twice; no slot either.
extern "C" int zi_cache_check(void* h) {
  Cache* c = as_cache(h);
  std::string why;
  if (!c->slots.check(&why)) return zi_refuse("request slots: %s", why.c_str()), ERR_CHECK;
  for (size_t g = 0; g < c->groups.size(); ++g) {
    const Pool& pool = c->groups[g].pool;
    if (!pool.check(&why)) return zi_refuse("group %zu: %s", g, why.c_str()), ERR_CHECK;
    std::vector<uint8_t> held(pool.num_pages, 0);
    long long n_held = 0;
    for (const auto& kv : c->requests)
      for (int p : kv.second.tables[g]) {
        if (p < 0) continue;
        if (p >= pool.num_pages || held[p]) return zi_refuse("group %zu: a page is held by two block tables", g), ERR_CHECK;
        if (!pool.used[p]) return zi_refuse("group %zu: a block table holds a page that is not in use", g), ERR_CHECK;
        held[p] = 1;
        ++n_held;
      }
    if (n_held != pool.n_used) return zi_refuse("group %zu: pages in use and pages in block tables differ", g), ERR_CHECK;
  }
  std::vector<uint8_t> slot_held(c->slots.num_pages, 0);
  for (const auto& kv : c->requests) {
    const int s = kv.second.slot;
    if (s < 0 || s >= c->slots.num_pages || slot_held[s] || !c->slots.used[s])
      return zi_refuse("request slots are inconsistent"), ERR_CHECK;
    slot_held[s] = 1;
  }
  if ((long long)c->requests.size() != c->slots.n_used) return zi_refuse("request slots are inconsistent"), ERR_CHECK;
  return 0;
}

// ------------------------------------------------------------------------- step builder
// Flattens a step's entries into one int32 buffer.  Arrays, each padded to a multiple of four
// words so that it starts on a 16-byte boundary, in this order (sizes in words):
//   0 token_ids [T]      1 positions [T]     2 cu_q [n+1]        3 kv_lens [n]      4 state_slots [n]
//   5 tile_seq [tiles]   6 tile_q0 [tiles]   7 logit_rows [R]    8 dec_seq [n_dec]
//   9 pf_tile_seq [pf]  10 pf_tile_q0 [pf]  11 patch_dst [P]    12 patch_src [P]
//  13 + 2g slots_g [T]  14 + 2g block_table_g [n * width_g]
// n = max(n_entries, static_batch): with static_batch > 0 (a decode step replayed from a CUDA graph)
// the batch is padded with requests of one key in no page whose key/value write is skipped and whose
// state slot is the spare one behind the requests' slots (index max_requests), every
// entry brings one token, logits are wanted for all n rows, block tables have static_width columns and
// P = n.  Otherwise width_g is the longest block table of the entries in group g (at least 1).
// The pages of the entries' tokens must have been reserved.
//
// layout (out): for each of the 13 + 2 * n_groups arrays its offset and size in words, then
// [total words, n, T, R, n_dec, n_pf_tiles, n_tiles, n_patch, max_q, max_kv, width_0, width_1, ...].
// With buf == null only the layout is computed (to size the buffer); returns total words or a code.
extern "C" long long zi_step_build(void* h, int n_entries, const long long* ids, const int* q_lens,
                                   const int* tokens /* all entries' tokens, flat */, const int* want_counts,
                                   const int* want /* flat, indices into each entry's tokens */,
                                   const int* token_src /* per entry, -1: none */, int static_batch, int static_width,
                                   int tile_rows, int pf_tile_rows, int* buf, long long capacity, long long* layout) {
  Cache* c = as_cache(h);
  const int G = (int)c->groups.size();
  if (n_entries <= 0 || tile_rows <= 0 || pf_tile_rows <= 0) return zi_refuse("step_build: nothing to build"), ERR_ARGUMENT;
  const bool is_static = static_batch > 0;
  if (is_static && n_entries > static_batch) return zi_refuse("step_build: %d entries in a bucket of %d", n_entries, static_batch), ERR_ARGUMENT;
  const int n = is_static ? static_batch : n_entries;
  std::vector<Request*> reqs(n_entries);
  std::vector<long long> ctx(n, 0);
  std::vector<int> ql(n, 1);
  for (int i = 0; i < n_entries; ++i) {
    reqs[i] = c->find(ids[i]);
    if (!reqs[i]) return zi_refuse("step_build: entry %d names a request that is not live", i), ERR_NOT_LIVE;
    if (q_lens[i] <= 0 || (is_static && q_lens[i] != 1)) return zi_refuse("step_build: entry %d brings %d tokens", i, q_lens[i]), ERR_ARGUMENT;
    ctx[i] = reqs[i]->length;
    ql[i] = q_lens[i];
  }
  long long T = 0;
  int n_tiles = 0, n_dec = 0, n_pf = 0, n_patch = 0, max_q = 0;
  long long R = 0, max_kv = 0;
  for (int i = 0; i < n; ++i) {
    T += ql[i];
    n_tiles += (ql[i] + tile_rows - 1) / tile_rows;
    if (ql[i] == 1) ++n_dec;
    else n_pf += (ql[i] + pf_tile_rows - 1) / pf_tile_rows;
  }
  for (int i = 0; i < n_entries; ++i) {
    R += want_counts ? want_counts[i] : 0;
    if (token_src && token_src[i] >= 0) ++n_patch;
    max_q = std::max(max_q, ql[i]);
    max_kv = std::max(max_kv, ctx[i] + ql[i]);
  }
  if (is_static) R = n;
  const int P = is_static ? n : n_patch;
  std::vector<int> width(G, 1);
  for (int g = 0; g < G; ++g) {
    if (is_static) {
      width[g] = static_width;
      for (int i = 0; i < n_entries; ++i)
        if ((int)reqs[i]->tables[g].size() > static_width)
          return zi_refuse("step_build: a request is longer than its bucket's block tables"), ERR_ARGUMENT;
    } else {
      for (int i = 0; i < n_entries; ++i) width[g] = std::max(width[g], (int)reqs[i]->tables[g].size());
    }
  }
  const int n_arrays = 13 + 2 * G;
  std::vector<long long> size(n_arrays), off(n_arrays);
  size[0] = size[1] = T;
  size[2] = n + 1;
  size[3] = size[4] = n;
  size[5] = size[6] = n_tiles;
  size[7] = R;
  size[8] = n_dec;
  size[9] = size[10] = n_pf;
  size[11] = size[12] = P;
  for (int g = 0; g < G; ++g) {
    size[13 + 2 * g] = T;
    size[14 + 2 * g] = (long long)n * width[g];
  }
  long long total = 0;
  for (int a = 0; a < n_arrays; ++a) {
    off[a] = total;
    total += (size[a] + 3) / 4 * 4;
  }
  if (layout) {
    for (int a = 0; a < n_arrays; ++a) {
      layout[2 * a] = off[a];
      layout[2 * a + 1] = size[a];
    }
    long long* tail = layout + 2 * n_arrays;
    tail[0] = total; tail[1] = n; tail[2] = T; tail[3] = R; tail[4] = n_dec; tail[5] = n_pf; tail[6] = n_tiles;
    tail[7] = n_patch; tail[8] = max_q; tail[9] = max_kv;
    for (int g = 0; g < G; ++g) tail[10 + g] = width[g];
  }
  if (!buf) return total;
  if (capacity < total) return zi_refuse("step_build: the buffer holds %lld words, %lld are needed", capacity, total), ERR_ARGUMENT;

  int* tok = buf + off[0];
  int* pos = buf + off[1];
  int* cu = buf + off[2];
  int* kv = buf + off[3];
  int* ss = buf + off[4];
  int* tseq = buf + off[5];
  int* tq0 = buf + off[6];
  int* rows = buf + off[7];
  int* dec = buf + off[8];
  int* pfs = buf + off[9];
  int* pfq = buf + off[10];
  int* pdst = buf + off[11];
  int* psrc = buf + off[12];
  long long t = 0, src = 0;
  int ti = 0, di = 0, ri = 0, pi = 0, wi = 0;
  std::vector<std::pair<long long, std::pair<int, int>>> pf_tiles;   // (keys read, (request, first token))
  cu[0] = 0;
  for (int i = 0; i < n; ++i) {
    const bool real = i < n_entries;
    for (int j = 0; j < ql[i]; ++j) {
      // placeholders (negative: sampled on the device, not yet read by the host) are patched on the device
      tok[t + j] = real ? std::max(tokens[src + j], 0) : 0;
      pos[t + j] = real ? (int)(ctx[i] + j) : 0;
    }
    if (real) {
      const int nw = want_counts ? want_counts[i] : 0;
      if (!is_static)
        for (int w = 0; w < nw; ++w) {
          const int idx = want[wi + w];
          if (idx < 0 || idx >= ql[i]) return zi_refuse("step_build: a wanted place lies outside the entry's tokens"), ERR_ARGUMENT;
          rows[ri++] = (int)t + idx;
        }
      wi += nw;
      if (token_src && token_src[i] >= 0) {
        pdst[pi] = (int)t;
        psrc[pi] = token_src[i];
        ++pi;
      }
      src += ql[i];
    }
    kv[i] = real ? (int)(ctx[i] + ql[i]) : 1;
    ss[i] = real ? reqs[i]->slot : c->max_requests;   // padding rows: the spare slot that belongs to no request
    for (int q0 = 0; q0 < ql[i]; q0 += tile_rows) {
      tseq[ti] = i;
      tq0[ti] = q0;
      ++ti;
    }
    if (ql[i] == 1) dec[di++] = i;
    else
      for (int q0 = 0; q0 < ql[i]; q0 += pf_tile_rows)
        pf_tiles.push_back({(real ? ctx[i] : 0) + std::min(ql[i], q0 + pf_tile_rows), {i, q0}});
    t += ql[i];
    cu[i + 1] = (int)t;
  }
  if (is_static)
    for (int i = 0; i < n; ++i) rows[i] = i;
  for (int i = pi; i < P; ++i) {
    pdst[i] = -1;
    psrc[i] = 0;
  }
  // the tiles that read the most keys come first: blocks are handed out in this order, so the long
  // ones do not end up alone at the tail
  std::stable_sort(pf_tiles.begin(), pf_tiles.end(), [](const auto& a, const auto& b) { return a.first > b.first; });
  for (size_t k = 0; k < pf_tiles.size(); ++k) {
    pfs[k] = pf_tiles[k].second.first;
    pfq[k] = pf_tiles[k].second.second;
  }
  for (int g = 0; g < G; ++g) {
    int* sl = buf + off[13 + 2 * g];
    int* bt = buf + off[14 + 2 * g];
    const int W = width[g];
    std::fill(bt, bt + (long long)n * W, -1);
    std::fill(sl, sl + T, -1);
    for (int i = 0; i < n_entries; ++i) {
      const std::vector<int>& table = reqs[i]->tables[g];
      if (!table.empty()) memcpy(bt + (long long)i * W, table.data(), table.size() * sizeof(int));
      for (int j = 0; j < ql[i]; ++j) {
        const long long p = ctx[i] + j;
        const long long b = p / c->page_size;
        if (b >= (long long)table.size()) return zi_refuse("step_build: entry %d: no page was reserved for position %lld", i, p), ERR_ARGUMENT;
        if (table[b] < 0) return zi_refuse("step_build: entry %d: a token would be written to a page already given back", i), ERR_RELEASED;
        sl[cu[i] + j] = table[b] * c->page_size + (int)(p % c->page_size);
      }
    }
  }
  return total;
}
