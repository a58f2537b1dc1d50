// The host side of the engine's inner loop, in C++ (no CUDA in here): the cache book, the planner
// and the step layout.
//
//  * CacheBook: which pages every live request holds in every group of layers, what it has
//    reserved and committed, the hash chain of its full pages (prefix reuse), the pages a window
//    has passed, and the request's state slot.  It owns one PagePool per group and the SlotPool.
//  * Planner: continuous batching over a CacheBook.  Every step gives each running request one
//    token if it is decoding, else the next portion of its prompt, oldest first, under a token
//    budget; admits waiting requests first-in first-out; and, when pages run out, preempts the most
//    recently admitted running request (its pages go back, it returns to the head of the queue to
//    be computed again).  The reference schedules one token per lane with capacity reserved up
//    front (crates/coheryn-api/src/scheduler.rs:321-415, scheduler/batching.rs:163-219); this is
//    its counterpart with pages allocated on demand.
//  * layout: the arrays a step needs on the device (ids, positions, request of each token, offsets,
//    lengths, slots, block tables), written into the caller's buffers.
//
// Python faces: cache/manager.py, engine/scheduler.py, engine/step.py.  Every call returns a
// status (0 = fine); nothing changes when a call fails.
#include <algorithm>
#include <deque>
#include <memory>

#include "host_pools.h"
#include "host_sha256.h"

namespace {

enum {
  BOOK_OK = 0,
  BOOK_ALREADY = 6,        // the request is already admitted
  BOOK_NO_SLOT = 7,        // no state slot is free
  BOOK_UNKNOWN = 8,        // no such request
  BOOK_UNCOMMITTED = 9,    // a reservation was not committed
  BOOK_SMALL = 10,         // the caller's buffer is too small
};

struct Held {
  int slot = -1;
  long long serial = 0;
  int length = 0;                          // tokens whose keys and values are committed
  std::vector<int> tokens;                 // committed + reserved token ids
  std::vector<std::vector<int>> tables;    // per group: page per block, -1 once given back
  int unknown_at = -1;                     // index of a token whose id is not known yet
  int hashed_blocks = 0;
  std::string last_hash;
  int reused = 0;
};

struct CacheBook {
  int page_size, num_pages, max_requests;
  bool prefix_reuse;
  std::vector<int> windows;                // per group, 0: none
  std::vector<std::unique_ptr<PagePool>> pools;
  SlotPool slots;
  std::unordered_map<std::string, Held> held;
  long long admissions = 0;

  CacheBook(int ps, int np, int mr, bool reuse, int groups, const int* win)
      : page_size(ps), num_pages(np), max_requests(mr), prefix_reuse(reuse), slots(mr) {
    for (int g = 0; g < groups; ++g) {
      windows.push_back(win ? win[g] : 0);
      pools.emplace_back(new PagePool(np));
      if (windows.back() > 0) prefix_reuse = false;    // pages behind a window cannot be found again
    }
  }

  Held* find(const std::string& id) {
    auto it = held.find(id);
    return it == held.end() ? nullptr : &it->second;
  }

  std::string block_hash(const std::string& prev, const int* tokens, int n) const {
    std::string msg(prev);
    for (int i = 0; i < n; ++i) {
      const uint32_t v = (uint32_t)tokens[i];
      const char b[4] = {(char)(v & 255), (char)((v >> 8) & 255), (char)((v >> 16) & 255), (char)((v >> 24) & 255)};
      msg.append(b, 4);
    }
    unsigned char out[32];
    sha256(reinterpret_cast<const unsigned char*>(msg.data()), msg.size(), out);
    return std::string(reinterpret_cast<const char*>(out), 32);
  }

  // A state slot and, with a prompt and prefix reuse, the leading full pages that are already
  // cached (never the page with the last prompt token: crates/coheryn-engine/src/inference/
  // generation.rs:189-198 always computes that token again).
  int admit(const std::string& id, const int* prompt, int n_prompt, int* reused) {
    if (held.count(id)) return BOOK_ALREADY;
    const int slot = slots.acquire();
    if (slot < 0) return BOOK_NO_SLOT;
    Held r;
    r.slot = slot;
    r.serial = ++admissions;
    r.tables.resize(pools.size());
    if (prompt && prefix_reuse && !pools.empty() && n_prompt > 1) {
      const int limit = (n_prompt - 1) / page_size;
      std::string h;
      std::vector<std::vector<int>> found;
      for (int b = 0; b < limit; ++b) {
        h = block_hash(h, prompt + (size_t)b * page_size, page_size);
        std::vector<int> pages;
        for (auto& pool : pools) pages.push_back(pool->lookup(reinterpret_cast<const unsigned char*>(h.data()), 32));
        if (std::find(pages.begin(), pages.end(), -1) != pages.end()) break;
        found.push_back(pages);
        r.last_hash = h;
      }
      for (auto& pages : found)
        for (size_t g = 0; g < pools.size(); ++g) {
          pools[g]->retain(pages[g]);
          r.tables[g].push_back(pages[g]);
        }
      const int n = (int)found.size() * page_size;
      r.length = r.reused = n;
      r.tokens.assign(prompt, prompt + n);
      r.hashed_blocks = (int)found.size();
    }
    *reused = r.reused;
    held.emplace(id, std::move(r));
    return BOOK_OK;
  }

  void pages_needed(const Held& r, int n, int* out) const {
    const int blocks = (r.length + n + page_size - 1) / page_size;
    for (size_t g = 0; g < pools.size(); ++g) out[g] = std::max(0, blocks - (int)r.tables[g].size());
  }

  // Pages for n more tokens after what the request holds.  All groups or none.
  int reserve(Held& r, const int* tokens, int n) {
    if ((int)r.tokens.size() != r.length) return BOOK_UNCOMMITTED;
    std::vector<int> need(pools.size());
    pages_needed(r, n, need.data());
    for (size_t g = 0; g < pools.size(); ++g)
      if (need[g] > pools[g]->available()) return POOL_NOT_ENOUGH;
    for (size_t g = 0; g < pools.size(); ++g) {
      std::vector<int> got(std::max(need[g], 1));
      pools[g]->allocate(need[g], got.data());
      r.tables[g].insert(r.tables[g].end(), got.begin(), got.begin() + need[g]);
    }
    r.tokens.insert(r.tokens.end(), tokens, tokens + n);
    return BOOK_OK;
  }

  int first_needed_block(int g, int next_position) const {
    if (windows[g] <= 0) return 0;
    return std::max(0, next_position - windows[g] + 1) / page_size;
  }

  // The reserved tokens' keys and values are written: advance the length, hash the pages that
  // became full, give back the pages a window has passed.
  void commit(Held& r) {
    r.length = (int)r.tokens.size();
    if (prefix_reuse) {
      const int known = r.unknown_at < 0 ? r.length : std::min(r.length, r.unknown_at);   // hashing waits for the id
      while ((r.hashed_blocks + 1) * page_size <= known) {
        const int b = r.hashed_blocks;
        r.last_hash = block_hash(r.last_hash, r.tokens.data() + (size_t)b * page_size, page_size);
        for (size_t g = 0; g < pools.size(); ++g)
          pools[g]->set_hash(r.tables[g][b], reinterpret_cast<const unsigned char*>(r.last_hash.data()), 32);
        ++r.hashed_blocks;
      }
    }
    for (size_t g = 0; g < pools.size(); ++g) {
      if (windows[g] <= 0) continue;
      const int upto = std::min(first_needed_block((int)g, r.length), (int)r.tables[g].size());
      for (int b = 0; b < upto; ++b)
        if (r.tables[g][b] >= 0) {
          pools[g]->release(r.tables[g][b]);
          r.tables[g][b] = -1;
        }
    }
  }

  // Drop a reservation that was not committed (pages beyond the committed length go back).
  void rollback(Held& r) {
    r.tokens.resize(r.length);
    const size_t keep = (size_t)((r.length + page_size - 1) / page_size);
    for (size_t g = 0; g < pools.size(); ++g) {
      auto& t = r.tables[g];
      for (size_t b = keep; b < t.size(); ++b)
        if (t[b] >= 0) pools[g]->release(t[b]);
      if (t.size() > keep) t.resize(keep);
    }
  }

  int release_all(const std::string& id) {
    auto it = held.find(id);
    if (it == held.end()) return BOOK_UNKNOWN;
    for (size_t g = 0; g < pools.size(); ++g)
      for (int p : it->second.tables[g])
        if (p >= 0) pools[g]->release(p);
    slots.release(it->second.slot);
    held.erase(it);
    return BOOK_OK;
  }
};

// ------------------------------------------------------------------------------------ planner
enum { REASON_NONE = 0, REASON_STOP = 1, REASON_LENGTH = 2, REASON_CANCELLED = 3 };
enum {
  PLAN_OK = 0,
  PLAN_EMPTY_PROMPT = 20,
  PLAN_NEGATIVE = 21,
  PLAN_CONTEXT = 22,
  PLAN_POOL = 23,
  PLAN_UNKNOWN = 24,
  PLAN_DUPLICATE = 25,
};

struct Job {
  std::string id;
  std::vector<int> prompt, output, stop_ids;
  int max_tokens = 0;
  int computed = 0;              // tokens whose keys and values are in the cache
  int reused = 0;                // prompt tokens found in the cache at the first admission
  int preemptions = 0;
  int reason = REASON_NONE;
  long long arrival = 0;
  bool penalised = false;
  bool running = false;
  int total() const { return (int)(prompt.size() + output.size()); }
  int token(int i) const { return i < (int)prompt.size() ? prompt[i] : output[i - (int)prompt.size()]; }
};

struct PlanEntry { int job; int start; int count; int samples; };

struct Planner {
  CacheBook* book;
  int context, max_num_seqs, max_num_batched_tokens;
  std::vector<std::unique_ptr<Job>> jobs;         // by handle; finished jobs stay until forgotten
  std::unordered_map<std::string, int> by_id;
  std::deque<int> waiting;
  std::vector<int> running;
  long long arrivals = 0;
  long long steps = 0, preemptions = 0, admitted = 0, finished = 0, scheduled_tokens = 0;
  int max_batch_width = 0;
  std::vector<PlanEntry> plan;
  std::vector<int> preempted_now, admitted_now;

  Planner(CacheBook* b, int ctx, int seqs, int budget)
      : book(b), context(ctx), max_num_seqs(std::min(seqs, b->max_requests)), max_num_batched_tokens(budget) {}

  int add(const std::string& id, const int* prompt, int n, int max_tokens, const int* stops, int n_stops, bool penalised,
          int* handle) {
    if (n <= 0) return PLAN_EMPTY_PROMPT;
    if (max_tokens < 0) return PLAN_NEGATIVE;
    if (n + max_tokens > context) return PLAN_CONTEXT;
    const int need = (n + std::max(max_tokens - 1, 0) + book->page_size - 1) / book->page_size;
    if (!book->pools.empty() && need > book->num_pages) return PLAN_POOL;
    auto it = by_id.find(id);
    if (it != by_id.end() && jobs[it->second]->reason == REASON_NONE) return PLAN_DUPLICATE;
    std::unique_ptr<Job> j(new Job);
    j->id = id;
    j->prompt.assign(prompt, prompt + n);
    j->stop_ids.assign(stops, stops + n_stops);
    j->max_tokens = max_tokens;
    j->arrival = arrivals++;
    j->penalised = penalised;
    jobs.push_back(std::move(j));
    *handle = (int)jobs.size() - 1;
    by_id[id] = *handle;
    waiting.push_back(*handle);
    return PLAN_OK;
  }

  void tokens_of(const Job& j, int start, int count, std::vector<int>& out) const {
    out.resize(count);
    for (int i = 0; i < count; ++i) out[i] = j.token(start + i);
  }

  bool fits(const Job& j, int n, const std::vector<int>& reserved) const {
    const Held* r = book->find(j.id);
    std::vector<int> need(book->pools.size());
    book->pages_needed(*r, n, need.data());
    for (size_t g = 0; g < need.size(); ++g)
      if (need[g] && reserved[g] + need[g] > book->pools[g]->available()) return false;
    return true;
  }

  // The most tokens (at most n) of the job that the free pages can take.
  int largest_fit(const Job& j, int n, const std::vector<int>& reserved) const {
    const Held* r = book->find(j.id);
    for (size_t g = 0; g < book->pools.size(); ++g) {
      const int blocks = (int)r->tables[g].size() + book->pools[g]->available() - reserved[g];
      n = std::min(n, blocks * book->page_size - r->length);
    }
    return std::max(n, 0);
  }

  void take(int h, int n, std::vector<int>& reserved) {
    Job& j = *jobs[h];
    const Held* r = book->find(j.id);
    std::vector<int> need(book->pools.size());
    book->pages_needed(*r, n, need.data());
    for (size_t g = 0; g < need.size(); ++g) reserved[g] += need[g];
    plan.push_back({h, j.computed, n, j.computed + n == j.total() ? 1 : 0});
  }

  void preempt(int h) {
    Job& j = *jobs[h];
    running.erase(std::find(running.begin(), running.end(), h));
    book->release_all(j.id);
    j.computed = 0;
    j.running = false;
    ++j.preemptions;
    ++preemptions;
    waiting.push_front(h);
    preempted_now.push_back(h);
  }

  void schedule() {
    plan.clear();
    preempted_now.clear();
    admitted_now.clear();
    int budget = max_num_batched_tokens;
    std::vector<int> reserved(book->pools.size(), 0);     // pages promised to earlier entries of this step
    std::vector<int> order(running);
    std::sort(order.begin(), order.end(), [&](int a, int b) { return jobs[a]->arrival < jobs[b]->arrival; });
    for (int h : order) {
      if (budget == 0 || !jobs[h]->running) continue;      // nothing left, or preempted below
      Job& j = *jobs[h];
      int n = std::min(j.total() - j.computed, budget);
      while (!fits(j, n, reserved)) {
        int victim = -1;
        for (int v : running) {
          if (v == h) continue;
          bool planned = false;
          for (auto& e : plan) planned = planned || e.job == v;
          if (!planned && (victim < 0 || jobs[v]->arrival > jobs[victim]->arrival)) victim = v;
        }
        if (victim < 0) {                                   // nobody left to preempt: what fits of the portion
          n = largest_fit(j, n, reserved);
          break;
        }
        preempt(victim);
      }
      if (n == 0) continue;
      take(h, n, reserved);
      budget -= n;
    }
    // admissions, first in first out; stop at the first that does not fit; none in a step that
    // had to preempt (the pool is short)
    while (preempted_now.empty() && !waiting.empty() && budget > 0 && (int)running.size() < max_num_seqs) {
      const int h = waiting.front();
      Job& j = *jobs[h];
      std::vector<int> all;
      tokens_of(j, 0, j.total(), all);
      int reused = 0;
      if (book->admit(j.id, all.data(), (int)all.size(), &reused) != BOOK_OK) break;
      j.computed = reused;
      int n = std::min(j.total() - j.computed, budget);
      if (!fits(j, n, reserved))
        // Beside running requests a newcomer waits for room for its whole first portion; alone it
        // starts with what fits.
        n = (!running.empty() || !plan.empty()) ? 0 : largest_fit(j, n, reserved);
      if (n == 0) {
        book->release_all(j.id);
        j.computed = 0;
        break;
      }
      if (j.preemptions == 0) j.reused = reused;
      waiting.pop_front();
      running.push_back(h);
      j.running = true;
      ++admitted;
      admitted_now.push_back(h);
      take(h, n, reserved);
      budget -= n;
    }
    count_step();
  }

  void count_step() {
    ++steps;
    for (auto& e : plan) scheduled_tokens += e.count;
    max_batch_width = std::max(max_batch_width, (int)plan.size());
  }

  // The plan of the step AFTER `prev` when that can be said before prev's tokens are known: prev
  // decodes every running request, nobody waits, none of the requests can end by length or context
  // with the token prev yields, and the pages are there.  Call after advance(prev).
  bool lookahead(const std::vector<PlanEntry>& prev) {
    if (!waiting.empty() || prev.empty() || prev.size() != running.size() || (int)prev.size() > max_num_batched_tokens)
      return false;
    std::vector<int> reserved(book->pools.size(), 0), need(book->pools.size());
    std::vector<PlanEntry> out;
    for (auto& e : prev) {
      Job& j = *jobs[e.job];
      if (j.reason != REASON_NONE || !e.samples || e.count != 1 || !j.running) return false;
      if ((int)j.output.size() + 2 > j.max_tokens || j.total() + 2 > context) return false;
      if (j.penalised) return false;     // the penalties of the next step need this step's id
      book->pages_needed(*book->find(j.id), 1, need.data());
      for (size_t g = 0; g < need.size(); ++g) reserved[g] += need[g];
      out.push_back({e.job, j.computed, 1, 1});
    }
    for (size_t g = 0; g < reserved.size(); ++g)
      if (reserved[g] > book->pools[g]->available()) return false;
    plan = out;
    preempted_now.clear();
    admitted_now.clear();
    count_step();
    return true;
  }

  void finish(int h, int reason) {
    Job& j = *jobs[h];
    j.reason = reason;
    auto r = std::find(running.begin(), running.end(), h);
    if (r != running.end()) {
      running.erase(r);
      j.running = false;
      book->release_all(j.id);
      ++finished;
    } else {
      auto w = std::find(waiting.begin(), waiting.end(), h);
      if (w != waiting.end()) {
        waiting.erase(w);
        ++finished;
      }
    }
    std::vector<int>().swap(j.prompt);      // a finished job keeps its numbers, not its tokens
    std::vector<int>().swap(j.output);
  }

  // Record a sampled token; the reason the job ended with it, or REASON_NONE.  The last sampled
  // token is not run through the model (crates/coheryn-engine/src/inference/generation.rs:386-388).
  int append_token(int h, int token) {
    Job& j = *jobs[h];
    j.output.push_back(token);
    int reason = REASON_NONE;
    if (std::find(j.stop_ids.begin(), j.stop_ids.end(), token) != j.stop_ids.end()) reason = REASON_STOP;   // the stop token stays in the ids
    else if ((int)j.output.size() >= j.max_tokens) reason = REASON_LENGTH;
    if (reason != REASON_NONE) finish(h, reason);
    return reason;
  }
};

std::string str(const char* s) { return std::string(s ? s : ""); }

}  // namespace

// ---------------------------------------------------------------------------- C interface: book
HOST_EXPORT void* coheryn_book_new(int page_size, int num_pages, int max_requests, int prefix_reuse, int groups,
                                   const int* windows) {
  if (page_size < 1 || num_pages < 0 || max_requests < 0 || groups < 0) return nullptr;
  return new CacheBook(page_size, num_pages, max_requests, prefix_reuse != 0, groups, windows);
}
HOST_EXPORT void coheryn_book_delete(void* h) { delete static_cast<CacheBook*>(h); }
HOST_EXPORT int coheryn_book_prefix_reuse(void* h) { return static_cast<CacheBook*>(h)->prefix_reuse ? 1 : 0; }
HOST_EXPORT void coheryn_book_set_prefix_reuse(void* h, int on) { static_cast<CacheBook*>(h)->prefix_reuse = on != 0; }
// The pools stay the book's: the handles serve the pool interface of host_pages.cpp (never delete them).
HOST_EXPORT void* coheryn_book_pool(void* h, int group) {
  CacheBook* b = static_cast<CacheBook*>(h);
  return group >= 0 && group < (int)b->pools.size() ? b->pools[group].get() : nullptr;
}
HOST_EXPORT void* coheryn_book_slots(void* h) { return &static_cast<CacheBook*>(h)->slots; }
HOST_EXPORT int coheryn_book_count(void* h) { return (int)static_cast<CacheBook*>(h)->held.size(); }
HOST_EXPORT int coheryn_book_has(void* h, const char* id) { return static_cast<CacheBook*>(h)->held.count(str(id)) ? 1 : 0; }

// n_prompt < 0: no prompt.  *reused, *slot, *serial describe the admission.
HOST_EXPORT int coheryn_book_admit(void* h, const char* id, const int* prompt, int n_prompt, int* reused, int* slot,
                                   long long* serial) {
  CacheBook* b = static_cast<CacheBook*>(h);
  int got = 0;
  const int rc = b->admit(str(id), n_prompt >= 0 ? prompt : nullptr, n_prompt, &got);
  if (rc != BOOK_OK) return rc;
  const Held* r = b->find(str(id));
  *reused = got;
  *slot = r->slot;
  *serial = r->serial;
  return BOOK_OK;
}
// what: 0 committed length, 1 tokens held (committed + reserved), 2 state slot, 3 hashed blocks,
// 4 tokens reused at admission; -1 for a request that is not admitted.
HOST_EXPORT long long coheryn_book_number(void* h, const char* id, int what) {
  const Held* r = static_cast<CacheBook*>(h)->find(str(id));
  if (!r) return -1;
  switch (what) {
    case 0: return r->length;
    case 1: return (long long)r->tokens.size();
    case 2: return r->slot;
    case 3: return r->hashed_blocks;
    case 4: return r->reused;
    case 5: return r->serial;
    default: return -1;
  }
}
HOST_EXPORT int coheryn_book_pages_needed(void* h, const char* id, int n, int* out) {
  CacheBook* b = static_cast<CacheBook*>(h);
  const Held* r = b->find(str(id));
  if (!r) return BOOK_UNKNOWN;
  b->pages_needed(*r, n, out);
  return BOOK_OK;
}
HOST_EXPORT int coheryn_book_reserve(void* h, const char* id, const int* tokens, int n) {
  CacheBook* b = static_cast<CacheBook*>(h);
  Held* r = b->find(str(id));
  return r ? b->reserve(*r, tokens, n) : BOOK_UNKNOWN;
}
HOST_EXPORT int coheryn_book_commit(void* h, const char* id) {
  CacheBook* b = static_cast<CacheBook*>(h);
  Held* r = b->find(str(id));
  if (!r) return BOOK_UNKNOWN;
  b->commit(*r);
  return BOOK_OK;
}
HOST_EXPORT int coheryn_book_rollback(void* h, const char* id) {
  CacheBook* b = static_cast<CacheBook*>(h);
  Held* r = b->find(str(id));
  if (!r) return BOOK_UNKNOWN;
  b->rollback(*r);
  return BOOK_OK;
}
HOST_EXPORT int coheryn_book_free(void* h, const char* id) { return static_cast<CacheBook*>(h)->release_all(str(id)); }
HOST_EXPORT int coheryn_book_mark_unknown(void* h, const char* id, int index) {
  Held* r = static_cast<CacheBook*>(h)->find(str(id));
  if (!r) return BOOK_UNKNOWN;
  r->unknown_at = index;
  return BOOK_OK;
}
HOST_EXPORT int coheryn_book_patch_token(void* h, const char* id, int index, int token) {
  Held* r = static_cast<CacheBook*>(h)->find(str(id));
  if (!r) return BOOK_UNKNOWN;
  if (index < 0 || index >= (int)r->tokens.size()) return POOL_BAD_ARGUMENT;
  r->tokens[index] = token;
  if (r->unknown_at == index) r->unknown_at = -1;
  return BOOK_OK;
}
// The block table of a group into out[0..cap): returns its length (also when cap is too small), or -1.
HOST_EXPORT int coheryn_book_table(void* h, const char* id, int group, int* out, int cap) {
  CacheBook* b = static_cast<CacheBook*>(h);
  const Held* r = b->find(str(id));
  if (!r || group < 0 || group >= (int)r->tables.size()) return -1;
  const auto& t = r->tables[group];
  for (int i = 0; i < (int)t.size() && i < cap; ++i) out[i] = t[i];
  return (int)t.size();
}
// Cache slot (page * page_size + offset) of every reserved, uncommitted token: returns their number, or -1.
HOST_EXPORT int coheryn_book_slot_ids(void* h, const char* id, int group, int* out, int cap) {
  CacheBook* b = static_cast<CacheBook*>(h);
  const Held* r = b->find(str(id));
  if (!r || group < 0 || group >= (int)r->tables.size()) return -1;
  const auto& t = r->tables[group];
  const int n = (int)r->tokens.size() - r->length;
  for (int i = 0; i < n && i < cap; ++i) {
    const int p = r->length + i;
    out[i] = t[p / b->page_size] * b->page_size + p % b->page_size;
  }
  return n;
}
HOST_EXPORT void coheryn_book_available(void* h, int* out) {
  CacheBook* b = static_cast<CacheBook*>(h);
  for (size_t g = 0; g < b->pools.size(); ++g) out[g] = b->pools[g]->available();
}
// No page lost, held twice or freed twice; no slot lost or shared.  0, or: 1..4 a pool's complaint
// (see PagePool::check) with the group in *group; 5 the slot pool lost a slot; 6 two requests share one.
HOST_EXPORT int coheryn_book_check(void* h, int* group, int* bad_page, int* info) {
  CacheBook* b = static_cast<CacheBook*>(h);
  for (size_t g = 0; g < b->pools.size(); ++g) {
    std::vector<int> held(std::max(b->num_pages, 1), 0);
    for (auto& kv : b->held)
      for (int p : kv.second.tables[g])
        if (p >= 0 && p < b->num_pages) ++held[p];
    *group = (int)g;
    const int rc = b->pools[g]->check(held.data(), bad_page, info);
    if (rc) return rc;
  }
  int in_use = 0;
  for (char c : b->slots.held) in_use += c ? 1 : 0;
  if (in_use + (int)b->slots.free_stack.size() != b->slots.num_slots) return 5;
  std::vector<char> seen(std::max(b->slots.num_slots, 1), 0);
  for (auto& kv : b->held) {
    const int s = kv.second.slot;
    if (s < 0 || s >= b->slots.num_slots || seen[s]) return 6;
    seen[s] = 1;
  }
  return 0;
}

// The arrays of a step for n requests (ids[i], counts[i] reserved tokens each): writes, per token,
// position, request index and (per group g) slot into pos / req / slots[g * T ..]; per request
// cu (n + 1), kv_lens, state slots, serials; returns the number of tokens T, or -1 (unknown request
// or a count that is not the request's reservation).  Block tables are fetched with coheryn_book_table.
HOST_EXPORT int coheryn_book_layout(void* h, int n, const char* const* ids, int* pos, int* req, int* slots, int cap_tokens,
                                    int* cu, int* kv_lens, int* state_slots, long long* serials) {
  CacheBook* b = static_cast<CacheBook*>(h);
  int T = 0;
  std::vector<const Held*> rs(n);
  for (int i = 0; i < n; ++i) {
    rs[i] = b->find(str(ids[i]));
    if (!rs[i]) return -1;
    T += (int)rs[i]->tokens.size() - rs[i]->length;
  }
  if (T > cap_tokens) return -1;
  int o = 0;
  cu[0] = 0;
  for (int i = 0; i < n; ++i) {
    const Held& r = *rs[i];
    const int cnt = (int)r.tokens.size() - r.length;
    for (int k = 0; k < cnt; ++k) {
      const int p = r.length + k;
      pos[o + k] = p;
      req[o + k] = i;
      for (size_t g = 0; g < b->pools.size(); ++g)
        slots[g * (size_t)T + o + k] = r.tables[g][p / b->page_size] * b->page_size + p % b->page_size;
    }
    o += cnt;
    cu[i + 1] = o;
    kv_lens[i] = r.length + cnt;
    state_slots[i] = r.slot;
    serials[i] = r.serial;
  }
  return T;
}

// The block tables of n requests for one group: row i of out (width entries, -1 beyond the table)
// and lens[i]; returns the longest table's length (nothing is written when it exceeds width), or -1.
HOST_EXPORT int coheryn_book_tables(void* h, int n, const char* const* ids, int group, int* out, int width, int* lens) {
  CacheBook* b = static_cast<CacheBook*>(h);
  int longest = 0;
  std::vector<const Held*> rs(n);
  for (int i = 0; i < n; ++i) {
    rs[i] = b->find(str(ids[i]));
    if (!rs[i] || group < 0 || group >= (int)rs[i]->tables.size()) return -1;
    longest = std::max(longest, (int)rs[i]->tables[group].size());
  }
  if (longest > width) return longest;
  for (int i = 0; i < n; ++i) {
    const auto& t = rs[i]->tables[group];
    int* row = out + (size_t)i * width;
    for (int k = 0; k < width; ++k) row[k] = k < (int)t.size() ? t[k] : -1;
    lens[i] = (int)t.size();
  }
  return longest;
}

// ------------------------------------------------------------------------- C interface: planner
HOST_EXPORT void* coheryn_planner_new(void* book, int context, int max_num_seqs, int max_num_batched_tokens) {
  if (!book || max_num_seqs < 1 || max_num_batched_tokens < 1) return nullptr;
  return new Planner(static_cast<CacheBook*>(book), context, max_num_seqs, max_num_batched_tokens);
}
HOST_EXPORT void coheryn_planner_delete(void* h) { delete static_cast<Planner*>(h); }
HOST_EXPORT int coheryn_planner_max_seqs(void* h) { return static_cast<Planner*>(h)->max_num_seqs; }
// 0 and the job's handle, or 20 empty prompt, 21 negative max_tokens, 22 beyond the context, 23 more
// pages than the pool has, 25 the id is in use.
HOST_EXPORT int coheryn_planner_add(void* h, const char* id, const int* prompt, int n, int max_tokens, const int* stops,
                                    int n_stops, int penalised, int* handle) {
  return static_cast<Planner*>(h)->add(str(id), prompt, n, max_tokens, stops, n_stops, penalised != 0, handle);
}
// A job that runs already (its pages are in the book, `computed` tokens of its prompt committed): for
// callers that fill the cache by other means.  Same refusals as add.
HOST_EXPORT int coheryn_planner_adopt(void* h, const char* id, const int* prompt, int n, int max_tokens, int computed,
                                      int* handle) {
  Planner* p = static_cast<Planner*>(h);
  const int rc = p->add(str(id), prompt, n, max_tokens, nullptr, 0, false, handle);
  if (rc != PLAN_OK) return rc;
  p->waiting.pop_back();
  p->running.push_back(*handle);
  p->jobs[*handle]->running = true;
  p->jobs[*handle]->computed = computed;
  return PLAN_OK;
}
HOST_EXPORT int coheryn_planner_has_work(void* h) {
  Planner* p = static_cast<Planner*>(h);
  return (!p->waiting.empty() || !p->running.empty()) ? 1 : 0;
}
HOST_EXPORT int coheryn_planner_schedule(void* h) {
  Planner* p = static_cast<Planner*>(h);
  p->schedule();
  return (int)p->plan.size();
}
// The plan after `n` entries (job handles with one sampled token each) of the step before: 1 and the
// new plan, or 0 when the ordinary schedule has to decide.
HOST_EXPORT int coheryn_planner_lookahead(void* h, int n, const int* jobs, const int* counts, const int* samples) {
  Planner* p = static_cast<Planner*>(h);
  std::vector<PlanEntry> prev(n);
  for (int i = 0; i < n; ++i) prev[i] = {jobs[i], 0, counts[i], samples[i]};
  return p->lookahead(prev) ? 1 : 0;
}
// The plan of the last schedule / lookahead: per entry job handle, first token, number of tokens,
// whether its last token yields a sampled one.
HOST_EXPORT int coheryn_planner_plan(void* h, int* jobs, int* starts, int* counts, int* samples, int cap) {
  Planner* p = static_cast<Planner*>(h);
  const int n = (int)p->plan.size();
  for (int i = 0; i < n && i < cap; ++i) {
    jobs[i] = p->plan[i].job; starts[i] = p->plan[i].start; counts[i] = p->plan[i].count; samples[i] = p->plan[i].samples;
  }
  return n;
}
// which: 0 preempted, 1 admitted by the last schedule; 2 running (in order of admission), 3 waiting (queue order).
HOST_EXPORT int coheryn_planner_list(void* h, int which, int* out, int cap) {
  Planner* p = static_cast<Planner*>(h);
  std::vector<int> tmp;
  const std::vector<int>* src = &tmp;
  if (which == 0) src = &p->preempted_now;
  else if (which == 1) src = &p->admitted_now;
  else if (which == 2) src = &p->running;
  else tmp.assign(p->waiting.begin(), p->waiting.end());
  for (int i = 0; i < (int)src->size() && i < cap; ++i) out[i] = (*src)[i];
  return (int)src->size();
}
// The tokens [start, start + count) of a job (prompt, then output) into out.
HOST_EXPORT int coheryn_planner_tokens(void* h, int job, int start, int count, int* out) {
  Planner* p = static_cast<Planner*>(h);
  if (job < 0 || job >= (int)p->jobs.size()) return PLAN_UNKNOWN;
  const Job& j = *p->jobs[job];
  if (start < 0 || count < 0 || start + count > j.total()) return POOL_BAD_ARGUMENT;
  for (int i = 0; i < count; ++i) out[i] = j.token(start + i);
  return PLAN_OK;
}
// what: 0 computed, 1 reused prompt tokens, 2 preemptions, 3 reason, 4 output length, 5 running.
HOST_EXPORT long long coheryn_planner_job(void* h, int job, int what) {
  Planner* p = static_cast<Planner*>(h);
  if (job < 0 || job >= (int)p->jobs.size()) return -1;
  const Job& j = *p->jobs[job];
  switch (what) {
    case 0: return j.computed;
    case 1: return j.reused;
    case 2: return j.preemptions;
    case 3: return j.reason;
    case 4: return (long long)j.output.size();
    case 5: return j.running ? 1 : 0;
    default: return -1;
  }
}
HOST_EXPORT void coheryn_planner_set_computed(void* h, int job, int computed) {
  Planner* p = static_cast<Planner*>(h);
  if (job >= 0 && job < (int)p->jobs.size()) p->jobs[job]->computed = computed;
}
// After a step: every planned job has its tokens in the cache.
HOST_EXPORT void coheryn_planner_advance(void* h, int n, const int* jobs, const int* counts) {
  Planner* p = static_cast<Planner*>(h);
  for (int i = 0; i < n; ++i)
    if (jobs[i] >= 0 && jobs[i] < (int)p->jobs.size()) p->jobs[jobs[i]]->computed += counts[i];
}
// A sampled token: returns the reason the job ended with it (1 stop, 2 length) or 0.
HOST_EXPORT int coheryn_planner_append_token(void* h, int job, int token) {
  Planner* p = static_cast<Planner*>(h);
  if (job < 0 || job >= (int)p->jobs.size()) return -1;
  return p->append_token(job, token);
}
HOST_EXPORT int coheryn_planner_finish(void* h, int job, int reason) {
  Planner* p = static_cast<Planner*>(h);
  if (job < 0 || job >= (int)p->jobs.size()) return PLAN_UNKNOWN;
  p->finish(job, reason);
  return PLAN_OK;
}
// steps, preemptions, admitted, finished, scheduled tokens, widest batch
HOST_EXPORT void coheryn_planner_stats(void* h, long long* out) {
  Planner* p = static_cast<Planner*>(h);
  out[0] = p->steps; out[1] = p->preemptions; out[2] = p->admitted; out[3] = p->finished; out[4] = p->scheduled_tokens;
  out[5] = p->max_batch_width;
}
