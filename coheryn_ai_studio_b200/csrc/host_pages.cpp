// The C interface of the page pool and the slot pool (host_pools.h): handles for a caller that keeps
// its own books (the Python face of the pools, and their tests).  Every function returns a status
// (0 = fine) instead of throwing, and nothing changes when a call fails.
#include "host_pools.h"

HOST_EXPORT void* coheryn_pool_new(int num_pages) { return num_pages < 0 ? nullptr : new PagePool(num_pages); }
HOST_EXPORT void coheryn_pool_delete(void* h) { delete static_cast<PagePool*>(h); }
HOST_EXPORT int coheryn_pool_available(void* h) { return static_cast<PagePool*>(h)->available(); }
HOST_EXPORT int coheryn_pool_refcount(void* h, int page) {
  PagePool* p = static_cast<PagePool*>(h);
  return p->known(page) ? p->refs[page] : -1;
}
HOST_EXPORT int coheryn_pool_allocate(void* h, int n, int* out) { return static_cast<PagePool*>(h)->allocate(n, out); }
HOST_EXPORT int coheryn_pool_retain(void* h, int page) { return static_cast<PagePool*>(h)->retain(page); }
HOST_EXPORT int coheryn_pool_release(void* h, int page) { return static_cast<PagePool*>(h)->release(page); }
HOST_EXPORT int coheryn_pool_set_hash(void* h, int page, const unsigned char* digest, int len) {
  return static_cast<PagePool*>(h)->set_hash(page, digest, len);
}
HOST_EXPORT int coheryn_pool_lookup(void* h, const unsigned char* digest, int len) {
  return static_cast<PagePool*>(h)->lookup(digest, len);
}
HOST_EXPORT void coheryn_pool_drop_hashes(void* h) { static_cast<PagePool*>(h)->drop_hashes(); }
HOST_EXPORT int coheryn_pool_check(void* h, const int* held, int* bad_page, int* info) {
  return static_cast<PagePool*>(h)->check(held, bad_page, info);
}

HOST_EXPORT void* coheryn_slots_new(int num_slots) { return num_slots < 0 ? nullptr : new SlotPool(num_slots); }
HOST_EXPORT void coheryn_slots_delete(void* h) { delete static_cast<SlotPool*>(h); }
HOST_EXPORT int coheryn_slots_available(void* h) { return (int)static_cast<SlotPool*>(h)->free_stack.size(); }
HOST_EXPORT int coheryn_slots_acquire(void* h) { return static_cast<SlotPool*>(h)->acquire(); }
HOST_EXPORT int coheryn_slots_release(void* h, int slot) { return static_cast<SlotPool*>(h)->release(slot); }
HOST_EXPORT int coheryn_slots_held(void* h, int slot) {
  SlotPool* s = static_cast<SlotPool*>(h);
  return slot >= 0 && slot < s->num_slots ? s->held[slot] : -1;
}
