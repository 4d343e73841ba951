// The engine's host runtime in C++: the page pools, the cache manager (block tables, layer
// groups, state slots) and the scheduler's decisions. Python holds the requests' tokens and
// drives the device; what is decided every step is decided here.
//
// In the manner of the reference's BlockManager (src/block_manager.h:25-57,
// src/block_manager.cpp:21-59), of how its engine uses it (src/engine.cpp:146-174) and of its
// scheduling loop (src/engine.cpp:304-377). The reference's prefix cache (hash chain, LRU of
// unreferenced pages) is left out; the reference count and a fork stay. Beyond the
// reference: layer groups (every key, or a window of the last W keys, each with a pool and a
// block table per request of its own; a window group gives a page back as soon as no later
// query can reach into it) and state slots (one per live request).
//
// C interface, opaque handles, requests named by 64-bit keys. Every function that can fail
// returns a negative number and leaves a message for bw_host_last_error().
#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#define BW_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_error;

int fail(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_error = buf;
  return -1;
}

constexpr int kFreed = -1;  // table entry of a page that a window has passed

// Reference-counted pages of one group, handed out low ids first.
struct PagePool {
  int num_pages = 0;
  std::vector<int> ref;
  std::vector<int> free_list;  // back() is handed out next

  explicit PagePool(int n) : num_pages(n), ref(n, 0) {
    free_list.reserve(n);
    for (int p = n - 1; p >= 0; --p) free_list.push_back(p);
  }
  int available() const { return static_cast<int>(free_list.size()); }
  int allocate() {
    if (free_list.empty()) return -1;
    const int p = free_list.back();
    free_list.pop_back();
    ref[p] = 1;
    return p;
  }
  bool fork(int page) {
    if (page < 0 || page >= num_pages || ref[page] <= 0) return false;
    ++ref[page];
    return true;
  }
  bool release(int page) {
    if (page < 0 || page >= num_pages || ref[page] <= 0) return false;
    if (--ref[page] == 0) free_list.push_back(page);
    return true;
  }
};

struct RequestCache {
  std::vector<std::vector<int>> tables;  // per group: page ids by block index (kFreed where passed)
  std::vector<int> first_live;           // per group: first block index not yet given back
  int length = 0;                        // tokens whose keys/values are in the cache
  int slot = -1;
  int epoch = 0;                         // a number no other table generation of this manager has had
};

struct CacheManager {
  std::vector<int> windows;  // per group: -1 keeps every key
  int page_size;
  std::vector<PagePool> pools;
  int num_slots;
  std::vector<int> free_slots;  // back() is handed out next
  std::unordered_map<int64_t, RequestCache> requests;
  int next_epoch = 1;  // every begin and every emptying of tables takes a fresh one

  CacheManager(int groups, const int* win, const int* pages, int page, int slots) : page_size(page), num_slots(slots) {
    for (int g = 0; g < groups; ++g) {
      windows.push_back(win[g]);
      pools.emplace_back(pages[g]);
    }
    for (int s = slots - 1; s >= 0; --s) free_slots.push_back(s);
  }
  RequestCache* find(int64_t rid) {
    auto it = requests.find(rid);
    return it == requests.end() ? nullptr : &it->second;
  }
  int begin(int64_t rid) {
    if (requests.count(rid)) return fail("request is already live");
    if (free_slots.empty()) return fail("no free state slot (more live requests than slots)");
    RequestCache rc;
    rc.tables.resize(pools.size());
    rc.first_live.assign(pools.size(), 0);
    rc.slot = free_slots.back();
    rc.epoch = next_epoch++;
    free_slots.pop_back();
    requests.emplace(rid, std::move(rc));
    return 0;
  }
  // Make every group's table cover positions 0 .. tokens-1. Pages are taken one at a time; on
  // failure what was gained is kept (src/engine.cpp:146-153) and 0 is returned.
  int ensure(int64_t rid, int tokens) {
    RequestCache* rc = find(rid);
    if (!rc) return fail("request is not live");
    const int need = (tokens + page_size - 1) / page_size;
    for (size_t g = 0; g < pools.size(); ++g) {
      std::vector<int>& table = rc->tables[g];
      while (static_cast<int>(table.size()) < need) {
        const int p = pools[g].allocate();
        if (p < 0) return 0;
        table.push_back(p);
      }
    }
    return 1;
  }
  // Record that `length` tokens are now cached; window groups give back the pages that no later
  // query can reach: the next query sits at position >= length and reads keys from
  // length - window + 1 on.
  int advance(int64_t rid, int length) {
    RequestCache* rc = find(rid);
    if (!rc) return fail("request is not live");
    if (length < rc->length) return fail("length goes back from %d to %d", rc->length, length);
    if (!rc->tables.empty()) {
      size_t shortest = rc->tables[0].size();
      for (const auto& t : rc->tables) shortest = std::min(shortest, t.size());
      if (length > static_cast<long long>(shortest) * page_size) return fail("%d tokens exceed the pages the request holds", length);
    }
    rc->length = length;
    for (size_t g = 0; g < pools.size(); ++g) {
      if (windows[g] < 0) continue;
      const int first_needed = length - windows[g] + 1;
      std::vector<int>& table = rc->tables[g];
      int& fl = rc->first_live[g];
      while (fl < static_cast<int>(table.size()) && (fl + 1) * page_size <= first_needed) {
        pools[g].release(table[fl]);
        table[fl] = kFreed;
        ++fl;
      }
    }
    return 0;
  }
  // Give back every page of the request (finish, cancel, preemption: src/engine.cpp:155-164)
  // and, unless keep_slot, its state slot.
  int release(int64_t rid, bool keep_slot) {
    RequestCache* rc = find(rid);
    if (!rc) return fail("request is not live");
    for (size_t g = 0; g < pools.size(); ++g) {
      for (int p : rc->tables[g])
        if (p != kFreed) pools[g].release(p);
      rc->tables[g].clear();
      rc->first_live[g] = 0;
    }
    rc->length = 0;
    rc->epoch = next_epoch++;
    if (!keep_slot) {
      free_slots.push_back(rc->slot);
      requests.erase(rid);
    }
    return 0;
  }
  int fork(int64_t src, int64_t dst) {
    if (!find(src)) return fail("request is not live");
    if (begin(dst) < 0) return -1;
    RequestCache* a = find(src);  // begin() may have moved the map's storage
    RequestCache* b = find(dst);
    for (size_t g = 0; g < pools.size(); ++g) {
      for (int p : a->tables[g])
        if (p != kFreed) pools[g].fork(p);
      b->tables[g] = a->tables[g];
      b->first_live[g] = a->first_live[g];
    }
    b->length = a->length;
    return 0;
  }
  bool all_free() const {
    for (const auto& p : pools)
      if (p.available() != p.num_pages) return false;
    return static_cast<int>(free_slots.size()) == num_slots;
  }
  // No page lost, none held twice without a matching count, none both free and held.
  int check() {
    for (size_t g = 0; g < pools.size(); ++g) {
      const PagePool& pool = pools[g];
      std::vector<int> held(pool.num_pages, 0), free_count(pool.num_pages, 0);
      for (const auto& kv : requests)
        for (int p : kv.second.tables[g])
          if (p != kFreed) {
            if (p < 0 || p >= pool.num_pages) return fail("group %zu: a table holds page %d, which does not exist", g, p);
            ++held[p];
          }
      for (int p : pool.free_list) {
        if (++free_count[p] > 1) return fail("group %zu: a page is on the free list twice", g);
      }
      for (int p = 0; p < pool.num_pages; ++p) {
        if (pool.ref[p] != held[p]) return fail("group %zu: page %d has count %d but %d holders", g, p, pool.ref[p], held[p]);
        if ((free_count[p] == 1) != (pool.ref[p] == 0))
          return fail("group %zu: page %d is %s with count %d", g, p, free_count[p] ? "free" : "missing", pool.ref[p]);
      }
    }
    std::vector<int> slot_use(num_slots, 0);
    for (const auto& kv : requests) {
      const int s = kv.second.slot;
      if (s < 0 || s >= num_slots || ++slot_use[s] > 1) return fail("a state slot is held twice");
    }
    for (int s : free_slots)
      if (s < 0 || s >= num_slots || ++slot_use[s] > 1) return fail("a state slot is held twice");
    if (static_cast<int>(requests.size() + free_slots.size()) != num_slots) return fail("a state slot is lost");
    return 0;
  }
};

// One request as the scheduler sees it (src/engine.cpp:82-98): how many tokens it has
// (prompt + generated) and how many of them are in the cache.
struct Seq {
  int64_t id;          // the cache manager's key of the request
  long long order = 0; // its age: smaller is older (the caller's request id)
  int tokens = 0;
  int computed = 0;
  bool running = false;
};

// Continuous batching above the step function. The policy is the reference's
// (src/engine.cpp:304-377), decision for decision:
// 1. Running requests are served oldest first (by id). A request needs tokens - computed rows;
//    if that exceeds what is left of the step's budget it gets the rest of the budget (a
//    portion), or nothing when the budget is spent; it stays running.
// 2. Its pages are taken one at a time. When the pool runs dry the YOUNGEST running request
//    that is neither already scheduled in this step nor the asker is preempted: all its pages
//    go back, computed = 0, and it returns to the waiting queue in id order, ahead of newer
//    arrivals. With no such victim the asker preempts itself. (src/engine.cpp:166-174,233-237,335-347)
// 3. Then waiting requests are admitted first-in first-out, only the head of the queue, while
//    fewer than max_num_seqs run and budget is left. A head that cannot get its pages gives
//    back what it took and admission stops for this step. (src/engine.cpp:354-376)
struct Scheduler {
  CacheManager* manager;
  int max_batched_tokens, max_num_seqs;
  std::unordered_map<int64_t, Seq> seqs;
  std::vector<int64_t> running;  // sorted by age
  std::deque<int64_t> waiting;
  long long preemptions = 0, admitted = 0;
  // what the last plan() did, for the caller to mirror
  std::vector<int64_t> plan_ids;
  std::vector<int> plan_rows;
  std::vector<int64_t> preempted_ids;
  std::vector<int> preempted_slots;

  Scheduler(CacheManager* m, int budget, int max_seqs) : manager(m), max_batched_tokens(budget), max_num_seqs(max_seqs) {}

  void release_pages(Seq& s) {
    if (manager->find(s.id)) manager->release(s.id, false);
    s.computed = 0;
  }
  void preempt(Seq& s) {
    const RequestCache* rc = manager->find(s.id);
    preempted_ids.push_back(s.id);
    preempted_slots.push_back(rc ? rc->slot : -1);
    release_pages(s);
    s.running = false;
    running.erase(std::find(running.begin(), running.end(), s.id));
    size_t pos = 0;
    while (pos < waiting.size() && seqs[waiting[pos]].order < s.order) ++pos;
    waiting.insert(waiting.begin() + pos, s.id);
    ++preemptions;
  }
  int finish(int64_t id) {
    auto it = seqs.find(id);
    if (it == seqs.end()) return fail("the scheduler does not know request %lld", static_cast<long long>(id));
    Seq& s = it->second;
    release_pages(s);
    if (s.running) {
      running.erase(std::find(running.begin(), running.end(), id));
    } else {
      auto w = std::find(waiting.begin(), waiting.end(), id);
      if (w != waiting.end()) waiting.erase(w);
    }
    seqs.erase(it);
    return 0;
  }
  void plan() {
    plan_ids.clear(), plan_rows.clear(), preempted_ids.clear(), preempted_slots.clear();
    int budget = max_batched_tokens;
    std::vector<int64_t> scheduled;
    const std::vector<int64_t> snapshot = running;
    for (int64_t id : snapshot) {
      Seq& s = seqs[id];
      if (!s.running) continue;  // preempted earlier in this loop
      int n = s.tokens - s.computed;
      if (n == 0) continue;
      if (n > budget) {
        if (budget <= 0) continue;
        n = budget;
      }
      bool ok = manager->ensure(id, s.computed + n) == 1;
      while (!ok) {
        int64_t victim = -1;
        bool found = false;
        for (auto it = running.rbegin(); it != running.rend(); ++it) {
          if (*it == id || std::find(scheduled.begin(), scheduled.end(), *it) != scheduled.end()) continue;
          victim = *it, found = true;
          break;
        }
        if (!found) break;
        preempt(seqs[victim]);
        ok = manager->ensure(id, s.computed + n) == 1;
      }
      if (!ok) {
        preempt(s);
        continue;
      }
      plan_ids.push_back(id), plan_rows.push_back(n);
      scheduled.push_back(id);
      budget -= n;
    }
    while (!waiting.empty() && static_cast<int>(running.size()) < max_num_seqs) {
      if (budget <= 0) break;
      Seq& s = seqs[waiting.front()];
      const int need = s.tokens - s.computed;
      const int n = std::min(need, budget);
      if (!manager->find(s.id)) {
        if (manager->free_slots.empty()) break;
        manager->begin(s.id);
      }
      if (manager->ensure(s.id, s.computed + n) != 1) {
        release_pages(s);
        break;
      }
      waiting.pop_front();
      s.running = true;
      running.insert(std::lower_bound(running.begin(), running.end(), s.id,
                                      [this](int64_t a, int64_t b) { return seqs[a].order < seqs[b].order; }),
                     s.id);
      ++admitted;
      if (n > 0) {
        plan_ids.push_back(s.id), plan_rows.push_back(n);
        budget -= n;
      }
    }
  }
};

template <typename T>
int copy_out(const std::vector<T>& v, T* out, int cap) {
  const int n = static_cast<int>(v.size());
  for (int i = 0; i < n && i < cap; ++i) out[i] = v[i];
  return n;
}

}  // namespace

BW_HOST_API const char* bw_host_last_error() { return g_error.c_str(); }

// ---- page pool (on its own, for tests and tools) -------------------------------------------
BW_HOST_API void* bw_pool_create(int num_pages) {
  if (num_pages < 0) {
    fail("a pool cannot have a negative number of pages");
    return nullptr;
  }
  return new PagePool(num_pages);
}
BW_HOST_API void bw_pool_destroy(void* h) { delete static_cast<PagePool*>(h); }
BW_HOST_API int bw_pool_available(void* h) { return static_cast<PagePool*>(h)->available(); }
BW_HOST_API int bw_pool_allocate(void* h) { return static_cast<PagePool*>(h)->allocate(); }
BW_HOST_API int bw_pool_fork(void* h, int page) {
  return static_cast<PagePool*>(h)->fork(page) ? 0 : fail("fork of page %d, which nobody holds", page);
}
BW_HOST_API int bw_pool_release(void* h, int page) {
  return static_cast<PagePool*>(h)->release(page) ? 0 : fail("release of page %d, which nobody holds", page);
}
BW_HOST_API int bw_pool_refcount(void* h, int page) {
  PagePool* p = static_cast<PagePool*>(h);
  return (page < 0 || page >= p->num_pages) ? fail("page %d does not exist", page) : p->ref[page];
}

// ---- cache manager -------------------------------------------------------------------------
BW_HOST_API void* bw_cm_create(int groups, const int* windows, const int* pages_per_group, int page_size, int num_slots) {
  if (page_size <= 0) {
    fail("page size must be positive");
    return nullptr;
  }
  for (int g = 0; g < groups; ++g)
    if (pages_per_group[g] < 0) {
      fail("a pool cannot have a negative number of pages");
      return nullptr;
    }
  return new CacheManager(groups, windows, pages_per_group, page_size, num_slots);
}
BW_HOST_API void bw_cm_destroy(void* h) { delete static_cast<CacheManager*>(h); }
BW_HOST_API int bw_cm_begin(void* h, int64_t rid) { return static_cast<CacheManager*>(h)->begin(rid); }
BW_HOST_API int bw_cm_has(void* h, int64_t rid) { return static_cast<CacheManager*>(h)->find(rid) ? 1 : 0; }
BW_HOST_API int bw_cm_ensure(void* h, int64_t rid, int tokens) { return static_cast<CacheManager*>(h)->ensure(rid, tokens); }
BW_HOST_API int bw_cm_advance(void* h, int64_t rid, int length) { return static_cast<CacheManager*>(h)->advance(rid, length); }
BW_HOST_API int bw_cm_release(void* h, int64_t rid, int keep_slot) {
  return static_cast<CacheManager*>(h)->release(rid, keep_slot != 0);
}
BW_HOST_API int bw_cm_fork(void* h, int64_t src, int64_t dst) { return static_cast<CacheManager*>(h)->fork(src, dst); }
// length, slot, epoch of a request, and per group the table's length and first live block:
// info[0..2], then (len, first_live) per group
BW_HOST_API int bw_cm_info(void* h, int64_t rid, int* info) {
  CacheManager* m = static_cast<CacheManager*>(h);
  RequestCache* rc = m->find(rid);
  if (!rc) return fail("request is not live");
  info[0] = rc->length, info[1] = rc->slot, info[2] = rc->epoch;
  for (size_t g = 0; g < m->pools.size(); ++g) {
    info[3 + 2 * g] = static_cast<int>(rc->tables[g].size());
    info[4 + 2 * g] = rc->first_live[g];
  }
  return 0;
}
// Copies table entries [begin, end) of a group into out (kFreed entries as `freed_as`);
// returns the table's length.
BW_HOST_API int bw_cm_table(void* h, int64_t rid, int group, int begin, int* out, int cap, int freed_as) {
  CacheManager* m = static_cast<CacheManager*>(h);
  RequestCache* rc = m->find(rid);
  if (!rc) return fail("request is not live");
  if (group < 0 || group >= static_cast<int>(m->pools.size())) return fail("group %d does not exist", group);
  const std::vector<int>& t = rc->tables[group];
  for (int i = begin; i < static_cast<int>(t.size()) && i - begin < cap; ++i) out[i - begin] = t[i] == kFreed ? freed_as : t[i];
  return static_cast<int>(t.size());
}
// What the step function does for every request of a step, in one call: take the pages the
// request needs for `counts[i]` more tokens and bring its rows of the block tables (one per
// group, at dst[table_offset[g] + i * max_blocks[g]]) up to date. `rows` remembers what each
// row holds, so a request that sits in the same row as in the step before only adds the pages
// it gained. Outputs per request: tokens already cached, state slot. Returns 0, or -1 with a
// message, or 1 + i when request i found no free page (requests before it keep what they
// got), or -(2 + i) when request i would outgrow its row of the block table.
struct RowState {
  int epoch = -1, len = 0, first_live = 0;
};
struct Rows {
  int max_seqs, groups;
  std::vector<RowState> state;
  Rows(int m, int g) : max_seqs(m), groups(g), state(static_cast<size_t>(m) * g) {}
};
BW_HOST_API void* bw_rows_create(int max_seqs, int groups) { return new Rows(max_seqs, groups); }
BW_HOST_API void bw_rows_destroy(void* h) { delete static_cast<Rows*>(h); }
BW_HOST_API int bw_cm_prepare(void* h, void* rows_h, int n, const int64_t* keys, const int* counts, int* dst,
                              const int* table_offset, const int* max_blocks, int* starts, int* slots) {
  CacheManager* m = static_cast<CacheManager*>(h);
  Rows* rows = static_cast<Rows*>(rows_h);
  const int groups = static_cast<int>(m->pools.size());
  if (n > rows->max_seqs || groups != rows->groups) return fail("%d requests in one step; the rows were made for %d", n, rows->max_seqs);
  for (int i = 0; i < n; ++i) {
    RequestCache* rc = m->find(keys[i]);
    if (!rc) return fail("request is not live");
    const int start = rc->length, total = start + counts[i];
    const int need = (total + m->page_size - 1) / m->page_size;
    for (int g = 0; g < groups; ++g)
      if (need > max_blocks[g]) return -(2 + i);
    if (m->ensure(keys[i], total) != 1) return 1 + i;
    starts[i] = start, slots[i] = rc->slot;
    for (int g = 0; g < groups; ++g) {
      RowState& was = rows->state[static_cast<size_t>(i) * groups + g];
      const std::vector<int>& table = rc->tables[g];
      const int len = static_cast<int>(table.size()), first_live = rc->first_live[g];
      const int begin = (was.epoch == rc->epoch && was.first_live == first_live && was.len <= len) ? was.len : 0;
      int* row = dst + table_offset[g] + static_cast<size_t>(i) * max_blocks[g];
      for (int b = begin; b < len; ++b) row[b] = table[b] == kFreed ? 0 : table[b];
      was.epoch = rc->epoch, was.len = len, was.first_live = first_live;
    }
  }
  return 0;
}
BW_HOST_API int bw_cm_pages_needed(void* h, int64_t rid, int tokens, int* out) {
  CacheManager* m = static_cast<CacheManager*>(h);
  RequestCache* rc = m->find(rid);
  if (!rc) return fail("request is not live");
  const int need = (tokens + m->page_size - 1) / m->page_size;
  for (size_t g = 0; g < m->pools.size(); ++g) out[g] = std::max(0, need - static_cast<int>(rc->tables[g].size()));
  return 0;
}
BW_HOST_API int bw_cm_available(void* h, int group) {
  CacheManager* m = static_cast<CacheManager*>(h);
  if (group < 0 || group >= static_cast<int>(m->pools.size())) return fail("group %d does not exist", group);
  return m->pools[group].available();
}
BW_HOST_API int bw_cm_refcount(void* h, int group, int page) {
  CacheManager* m = static_cast<CacheManager*>(h);
  if (group < 0 || group >= static_cast<int>(m->pools.size())) return fail("group %d does not exist", group);
  if (page < 0 || page >= m->pools[group].num_pages) return fail("page %d does not exist", page);
  return m->pools[group].ref[page];
}
BW_HOST_API int bw_cm_free_slots(void* h) { return static_cast<int>(static_cast<CacheManager*>(h)->free_slots.size()); }
BW_HOST_API int bw_cm_all_free(void* h) { return static_cast<CacheManager*>(h)->all_free() ? 1 : 0; }
BW_HOST_API int bw_cm_live(void* h) { return static_cast<int>(static_cast<CacheManager*>(h)->requests.size()); }
BW_HOST_API int bw_cm_max_blocks(void* h, int group) {
  CacheManager* m = static_cast<CacheManager*>(h);
  if (group < 0 || group >= static_cast<int>(m->pools.size())) return fail("group %d does not exist", group);
  size_t most = 0;
  for (const auto& kv : m->requests) most = std::max(most, kv.second.tables[group].size());
  return static_cast<int>(most);
}
BW_HOST_API int bw_cm_check(void* h) { return static_cast<CacheManager*>(h)->check(); }

// ---- scheduler -----------------------------------------------------------------------------
BW_HOST_API void* bw_sched_create(void* manager, int max_batched_tokens, int max_num_seqs) {
  if (max_batched_tokens <= 0 || max_num_seqs <= 0) {
    fail("max_batched_tokens and max_num_seqs must be positive");
    return nullptr;
  }
  return new Scheduler(static_cast<CacheManager*>(manager), max_batched_tokens, max_num_seqs);
}
BW_HOST_API void bw_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }
BW_HOST_API int bw_sched_add(void* h, int64_t id, long long order, int tokens, int computed) {
  Scheduler* s = static_cast<Scheduler*>(h);
  if (s->seqs.count(id)) return fail("request %lld is already queued", static_cast<long long>(id));
  Seq q;
  q.id = id, q.order = order, q.tokens = tokens, q.computed = computed;
  s->seqs.emplace(id, q);
  s->waiting.push_back(id);
  return 0;
}
// The caller owns the tokens: before a plan it says how many each request has and how many of
// them are computed.
BW_HOST_API int bw_sched_update(void* h, int64_t id, int tokens, int computed) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return fail("the scheduler does not know request %lld", static_cast<long long>(id));
  it->second.tokens = tokens, it->second.computed = computed;
  return 0;
}
BW_HOST_API int bw_sched_update_many(void* h, int n, const int64_t* ids, const int* tokens, const int* computed) {
  Scheduler* s = static_cast<Scheduler*>(h);
  for (int i = 0; i < n; ++i) {
    auto it = s->seqs.find(ids[i]);
    if (it == s->seqs.end()) return fail("the scheduler does not know request %lld", static_cast<long long>(ids[i]));
    it->second.tokens = tokens[i], it->second.computed = computed[i];
  }
  return 0;
}
BW_HOST_API int bw_sched_finish(void* h, int64_t id) { return static_cast<Scheduler*>(h)->finish(id); }
BW_HOST_API int bw_sched_preempt(void* h, int64_t id) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end() || !it->second.running) return fail("request %lld is not running", static_cast<long long>(id));
  s->preempted_ids.clear(), s->preempted_slots.clear();
  s->preempt(it->second);
  return 0;
}
BW_HOST_API int bw_sched_plan(void* h) {
  Scheduler* s = static_cast<Scheduler*>(h);
  s->plan();
  return static_cast<int>(s->plan_ids.size());
}
BW_HOST_API int bw_sched_plan_entries(void* h, int64_t* ids, int* rows, int cap) {
  Scheduler* s = static_cast<Scheduler*>(h);
  copy_out(s->plan_ids, ids, cap);
  return copy_out(s->plan_rows, rows, cap);
}
BW_HOST_API int bw_sched_preempted(void* h, int64_t* ids, int* slots, int cap) {
  Scheduler* s = static_cast<Scheduler*>(h);
  copy_out(s->preempted_ids, ids, cap);
  return copy_out(s->preempted_slots, slots, cap);
}
BW_HOST_API int bw_sched_running(void* h, int64_t* ids, int cap) { return copy_out(static_cast<Scheduler*>(h)->running, ids, cap); }
BW_HOST_API int bw_sched_waiting(void* h, int64_t* ids, int cap) {
  Scheduler* s = static_cast<Scheduler*>(h);
  const std::vector<int64_t> w(s->waiting.begin(), s->waiting.end());
  return copy_out(w, ids, cap);
}
BW_HOST_API int bw_sched_state(void* h, int64_t id, int* computed, int* running) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->seqs.find(id);
  if (it == s->seqs.end()) return fail("the scheduler does not know request %lld", static_cast<long long>(id));
  *computed = it->second.computed, *running = it->second.running ? 1 : 0;
  return 0;
}
BW_HOST_API long long bw_sched_stat(void* h, int which) {
  Scheduler* s = static_cast<Scheduler*>(h);
  return which == 0 ? s->preemptions : s->admitted;
}
