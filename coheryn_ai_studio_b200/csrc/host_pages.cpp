// Host-side bookkeeping of cache pages and of per-request state slots (no CUDA in here).
//
// A page pool owns num_pages page ids.  Every page is free, or held with a reference count
// >= 1 (several holders when requests share a prefix), or idle: it was filled completely,
// carries a content hash and has no holder left.  Idle pages stay findable by their hash and
// are wiped, least recently used first, only when no plain free page is left.  Freed pages are
// handed out again last-in first-out, so reuse happens at once.
//
// The reference keeps whole sessions with byte budgets (crates/coheryn-api/src/memory.rs:125-178);
// this is the page-granular counterpart.  Every function returns a status (0 = fine) instead
// of throwing, and nothing changes when a call fails.
#include <cstdint>
#include <cstring>
#include <list>
#include <string>
#include <unordered_map>
#include <vector>

#define HOST_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

struct PagePool {
  int num_pages;
  std::vector<int> free_stack;                       // back = next out
  std::vector<int> refs;
  std::vector<char> hashed, idle;
  std::vector<std::string> hash_of;                  // valid where hashed
  std::unordered_map<std::string, int> page_of;      // content hash -> page
  std::list<int> idle_lru;                           // front = least recently used
  std::vector<std::list<int>::iterator> idle_at;     // valid where idle

  explicit PagePool(int n) : num_pages(n), refs(n, 0), hashed(n, 0), idle(n, 0), hash_of(n), idle_at(n) {
    free_stack.reserve(n);
    for (int p = n - 1; p >= 0; --p) free_stack.push_back(p);   // page 0 first out
  }
  bool known(int p) const { return p >= 0 && p < num_pages; }
  int available() const { return (int)free_stack.size() + (int)idle_lru.size(); }
  void forget(int p) {
    if (hashed[p]) {
      page_of.erase(hash_of[p]);
      hash_of[p].clear();
      hashed[p] = 0;
    }
  }
};

struct SlotPool {
  int num_slots;
  std::vector<int> free_stack;
  std::vector<char> held;
  explicit SlotPool(int n) : num_slots(n), held(n, 0) {
    for (int s = n - 1; s >= 0; --s) free_stack.push_back(s);
  }
};

}  // namespace

// Status codes shared by the calls below.
enum { POOL_OK = 0, POOL_UNKNOWN_PAGE = 1, POOL_NOT_HELD = 2, POOL_FREE_PAGE = 3, POOL_NOT_ENOUGH = 4, POOL_BAD_ARGUMENT = 5 };

HOST_EXPORT void* coheryn_pool_new(int num_pages) { return num_pages < 0 ? nullptr : new PagePool(num_pages); }
HOST_EXPORT void coheryn_pool_delete(void* h) { delete static_cast<PagePool*>(h); }
HOST_EXPORT int coheryn_pool_available(void* h) { return static_cast<PagePool*>(h)->available(); }
HOST_EXPORT int coheryn_pool_refcount(void* h, int page) {
  PagePool* p = static_cast<PagePool*>(h);
  return p->known(page) ? p->refs[page] : -1;
}

// n pages with reference count 1 into out[0..n), or POOL_NOT_ENOUGH and no change.
HOST_EXPORT int coheryn_pool_allocate(void* h, int n, int* out) {
  PagePool* p = static_cast<PagePool*>(h);
  if (n < 0) return POOL_BAD_ARGUMENT;
  if (n > p->available()) return POOL_NOT_ENOUGH;
  for (int i = 0; i < n; ++i) {
    int page;
    if (!p->free_stack.empty()) {
      page = p->free_stack.back();
      p->free_stack.pop_back();
    } else {                                     // evict the least recently used idle page
      page = p->idle_lru.front();
      p->idle_lru.pop_front();
      p->idle[page] = 0;
      p->forget(page);
    }
    p->refs[page] = 1;
    out[i] = page;
  }
  return POOL_OK;
}

// One more holder of a page (a shared prefix); revives an idle hashed page.
HOST_EXPORT int coheryn_pool_retain(void* h, int page) {
  PagePool* p = static_cast<PagePool*>(h);
  if (!p->known(page)) return POOL_UNKNOWN_PAGE;
  if (p->refs[page] == 0) {
    if (!p->idle[page]) return POOL_FREE_PAGE;
    p->idle_lru.erase(p->idle_at[page]);
    p->idle[page] = 0;
  }
  ++p->refs[page];
  return POOL_OK;
}

HOST_EXPORT int coheryn_pool_release(void* h, int page) {
  PagePool* p = static_cast<PagePool*>(h);
  if (!p->known(page)) return POOL_UNKNOWN_PAGE;
  if (p->refs[page] <= 0) return POOL_NOT_HELD;
  if (--p->refs[page] == 0) {
    if (p->hashed[page]) {
      p->idle_lru.push_back(page);
      p->idle_at[page] = std::prev(p->idle_lru.end());
      p->idle[page] = 1;
    } else {
      p->free_stack.push_back(page);
    }
  }
  return POOL_OK;
}

// Record that `page` holds the full block identified by the digest.  If another page already
// carries that digest, or the page a digest, the older record stays.
HOST_EXPORT int coheryn_pool_set_hash(void* h, int page, const unsigned char* digest, int len) {
  PagePool* p = static_cast<PagePool*>(h);
  if (!p->known(page)) return POOL_UNKNOWN_PAGE;
  if (p->refs[page] <= 0) return POOL_NOT_HELD;
  if (len <= 0 || !digest) return POOL_BAD_ARGUMENT;
  std::string key(reinterpret_cast<const char*>(digest), (size_t)len);
  if (p->hashed[page] || p->page_of.count(key)) return POOL_OK;
  p->hash_of[page] = key;
  p->hashed[page] = 1;
  p->page_of.emplace(std::move(key), page);
  return POOL_OK;
}

// The page that carries the digest, or -1.
HOST_EXPORT int coheryn_pool_lookup(void* h, const unsigned char* digest, int len) {
  PagePool* p = static_cast<PagePool*>(h);
  if (len <= 0 || !digest) return -1;
  auto it = p->page_of.find(std::string(reinterpret_cast<const char*>(digest), (size_t)len));
  return it == p->page_of.end() ? -1 : it->second;
}

// Forget every content hash (idle pages become plain free pages, least recently used first).
HOST_EXPORT void coheryn_pool_drop_hashes(void* h) {
  PagePool* p = static_cast<PagePool*>(h);
  for (int page : p->idle_lru) {
    p->free_stack.push_back(page);
    p->idle[page] = 0;
  }
  p->idle_lru.clear();
  for (int page = 0; page < p->num_pages; ++page) {
    p->hash_of[page].clear();
    p->hashed[page] = 0;
  }
  p->page_of.clear();
}

// Invariants: every page is in exactly one place (free / idle / held); an idle page has a hash;
// with `held` (the holders of each page as the caller counts them, num_pages entries) the
// reference counts agree.  Returns 0, or a code with the page in *bad_page and a number in *info:
//   1 negative reference count; 2 the page is in *info places; 3 an idle page without a hash;
//   4 the pool counts *info holders where the caller counts held[page].
HOST_EXPORT int coheryn_pool_check(void* h, const int* held, int* bad_page, int* info) {
  PagePool* p = static_cast<PagePool*>(h);
  std::vector<int> seen(p->num_pages, 0);
  for (int page : p->free_stack) ++seen[page];
  for (int page : p->idle_lru) ++seen[page];
  for (int page = 0; page < p->num_pages; ++page) {
    *bad_page = page;
    if (p->refs[page] < 0) return 1;
    if (p->refs[page] > 0) ++seen[page];
    if (seen[page] != 1) { *info = seen[page]; return 2; }
    if (p->idle[page] && !p->hashed[page]) return 3;
    if (held && p->refs[page] != held[page]) { *info = p->refs[page]; return 4; }
  }
  return 0;
}

// ---- slots for per-request state of fixed size -----------------------------------------
HOST_EXPORT void* coheryn_slots_new(int num_slots) { return num_slots < 0 ? nullptr : new SlotPool(num_slots); }
HOST_EXPORT void coheryn_slots_delete(void* h) { delete static_cast<SlotPool*>(h); }
HOST_EXPORT int coheryn_slots_available(void* h) { return (int)static_cast<SlotPool*>(h)->free_stack.size(); }
// A free slot (lowest index first from a fresh pool), or -1.
HOST_EXPORT int coheryn_slots_acquire(void* h) {
  SlotPool* s = static_cast<SlotPool*>(h);
  if (s->free_stack.empty()) return -1;
  const int slot = s->free_stack.back();
  s->free_stack.pop_back();
  s->held[slot] = 1;
  return slot;
}
// 0, or 1 for a slot that is not in the pool, 2 for one that is not held.
HOST_EXPORT int coheryn_slots_release(void* h, int slot) {
  SlotPool* s = static_cast<SlotPool*>(h);
  if (slot < 0 || slot >= s->num_slots) return 1;
  if (!s->held[slot]) return 2;
  s->held[slot] = 0;
  s->free_stack.push_back(slot);
  return 0;
}
HOST_EXPORT int coheryn_slots_held(void* h, int slot) {
  SlotPool* s = static_cast<SlotPool*>(h);
  return slot >= 0 && slot < s->num_slots ? s->held[slot] : -1;
}
