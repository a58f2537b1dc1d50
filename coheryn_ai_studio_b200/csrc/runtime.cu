// Error channel and identification of the kernel library.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

static thread_local char g_error[1024];

void co_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

CO_EXPORT const char* coheryn_last_error() { return g_error; }

// Compiled-for architecture, so the loader can refuse a library built for another GPU.
CO_EXPORT int coheryn_arch() {
#ifdef CO_TARGET_ARCH
  return CO_TARGET_ARCH;
#else
  return 0;
#endif
}

// Number of kernel launches made through this library since load (a claim for
// benchmarks that must show that these kernels, not a fallback, did the work).
static unsigned long long g_launches = 0;
void co_count_launch() { __atomic_add_fetch(&g_launches, 1ull, __ATOMIC_RELAXED); }
CO_EXPORT unsigned long long coheryn_launch_count() {
  return __atomic_load_n(&g_launches, __ATOMIC_RELAXED);
}

bool co_pdl_enabled() {
  static int state = -1;
  if (state < 0) {
    const char* e = getenv("COHERYN_PDL");
    state = (e && e[0] == '0') ? 0 : 1;
  }
  return state == 1;
}
