// Host-side bookkeeping of cache pages and of per-request state slots (no CUDA in here): the two
// pools as C++ classes, used by the C interface of host_pages.cpp and by the cache book and the
// planner of host_engine.cpp.
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
#pragma once
#include <cstdint>
#include <cstring>
#include <list>
#include <string>
#include <unordered_map>
#include <vector>

#define HOST_EXPORT extern "C" __attribute__((visibility("default")))

// Status codes shared by the calls of both files.
enum { POOL_OK = 0, POOL_UNKNOWN_PAGE = 1, POOL_NOT_HELD = 2, POOL_FREE_PAGE = 3, POOL_NOT_ENOUGH = 4, POOL_BAD_ARGUMENT = 5 };

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

  // n pages with reference count 1 into out[0..n), or POOL_NOT_ENOUGH and no change.
  int allocate(int n, int* out) {
    if (n < 0) return POOL_BAD_ARGUMENT;
    if (n > available()) return POOL_NOT_ENOUGH;
    for (int i = 0; i < n; ++i) {
      int page;
      if (!free_stack.empty()) {
        page = free_stack.back();
        free_stack.pop_back();
      } else {                                     // evict the least recently used idle page
        page = idle_lru.front();
        idle_lru.pop_front();
        idle[page] = 0;
        forget(page);
      }
      refs[page] = 1;
      out[i] = page;
    }
    return POOL_OK;
  }

  // One more holder of a page (a shared prefix); revives an idle hashed page.
  int retain(int page) {
    if (!known(page)) return POOL_UNKNOWN_PAGE;
    if (refs[page] == 0) {
      if (!idle[page]) return POOL_FREE_PAGE;
      idle_lru.erase(idle_at[page]);
      idle[page] = 0;
    }
    ++refs[page];
    return POOL_OK;
  }

  int release(int page) {
    if (!known(page)) return POOL_UNKNOWN_PAGE;
    if (refs[page] <= 0) return POOL_NOT_HELD;
    if (--refs[page] == 0) {
      if (hashed[page]) {
        idle_lru.push_back(page);
        idle_at[page] = std::prev(idle_lru.end());
        idle[page] = 1;
      } else {
        free_stack.push_back(page);
      }
    }
    return POOL_OK;
  }

  // Record that `page` holds the full block identified by the digest.  If another page already
  // carries that digest, or the page a digest, the older record stays.
  int set_hash(int page, const unsigned char* digest, int len) {
    if (!known(page)) return POOL_UNKNOWN_PAGE;
    if (refs[page] <= 0) return POOL_NOT_HELD;
    if (len <= 0 || !digest) return POOL_BAD_ARGUMENT;
    std::string key(reinterpret_cast<const char*>(digest), (size_t)len);
    if (hashed[page] || page_of.count(key)) return POOL_OK;
    hash_of[page] = key;
    hashed[page] = 1;
    page_of.emplace(std::move(key), page);
    return POOL_OK;
  }

  // The page that carries the digest, or -1.
  int lookup(const unsigned char* digest, int len) const {
    if (len <= 0 || !digest) return -1;
    auto it = page_of.find(std::string(reinterpret_cast<const char*>(digest), (size_t)len));
    return it == page_of.end() ? -1 : it->second;
  }

  // Forget every content hash (idle pages become plain free pages, least recently used first).
  void drop_hashes() {
    for (int page : idle_lru) {
      free_stack.push_back(page);
      idle[page] = 0;
    }
    idle_lru.clear();
    for (int page = 0; page < num_pages; ++page) {
      hash_of[page].clear();
      hashed[page] = 0;
    }
    page_of.clear();
  }

  // Invariants: every page is in exactly one place (free / idle / held); an idle page has a hash;
  // with `held` (the holders of each page as the caller counts them, num_pages entries) the
  // reference counts agree.  Returns 0, or a code with the page in *bad_page and a number in *info:
  //   1 negative reference count; 2 the page is in *info places; 3 an idle page without a hash;
  //   4 the pool counts *info holders where the caller counts held[page].
  int check(const int* held, int* bad_page, int* info) const {
    std::vector<int> seen(num_pages, 0);
    for (int page : free_stack) ++seen[page];
    for (int page : idle_lru) ++seen[page];
    for (int page = 0; page < num_pages; ++page) {
      *bad_page = page;
      if (refs[page] < 0) return 1;
      if (refs[page] > 0) ++seen[page];
      if (seen[page] != 1) { *info = seen[page]; return 2; }
      if (idle[page] && !hashed[page]) return 3;
      if (held && refs[page] != held[page]) { *info = refs[page]; return 4; }
    }
    return 0;
  }
};

struct SlotPool {
  int num_slots;
  std::vector<int> free_stack;
  std::vector<char> held;
  explicit SlotPool(int n) : num_slots(n), held(n, 0) {
    for (int s = n - 1; s >= 0; --s) free_stack.push_back(s);
  }
  // A free slot (lowest index first from a fresh pool), or -1.
  int acquire() {
    if (free_stack.empty()) return -1;
    const int slot = free_stack.back();
    free_stack.pop_back();
    held[slot] = 1;
    return slot;
  }
  // 0, or 1 for a slot that is not in the pool, 2 for one that is not held.
  int release(int slot) {
    if (slot < 0 || slot >= num_slots) return 1;
    if (!held[slot]) return 2;
    held[slot] = 0;
    free_stack.push_back(slot);
    return 0;
  }
};
