// Shared helpers of the sm_100a kernels: dtype codes, conversions, reductions and the
// error channel of the C entry points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

// dtype codes shared with the Python side (ops.py).
#define CO_F32 0
#define CO_BF16 1

#define CO_EXPORT extern "C" __attribute__((visibility("default")))

// Error channel: every entry point returns 0 on success; otherwise a message is left
// in a thread-local buffer that coheryn_last_error() hands out.
void co_set_error(const char* fmt, ...);
#define CO_FAIL(...)                 \
  do {                               \
    co_set_error(__VA_ARGS__);       \
    return 1;                        \
  } while (0)
void co_count_launch();
#define CO_CHECK_LAUNCH(name)                                                        \
  do {                                                                               \
    co_count_launch();                                                               \
    cudaError_t e__ = cudaGetLastError();                                            \
    if (e__ != cudaSuccess) CO_FAIL("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
  } while (0)

// Programmatic dependent launch: a kernel launched with co_launch() may begin while its
// predecessor in the stream is still running.  It must call co_pdl_wait() before it reads
// or writes anything a predecessor touches (weights and other constants may be fetched
// earlier), and it calls co_pdl_launch_dependents() to let its own successor start its
// preamble.  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void co_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void co_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool co_pdl_enabled();   // COHERYN_PDL=0 in the environment switches the launch attribute off

// Kernels ask for the largest shared-memory carve-out, whatever they use themselves: an SM
// changes its split between L1 and shared memory only when it is empty, so kernels with
// different preferences cannot share an SM, and a dependent launch cannot take its place
// early on an SM that its predecessor still occupies.  A kernel that lives on L1 hits is
// launched with keep_l1 = true and keeps the default split.  COHERYN_CARVEOUT=0 in the
// environment leaves every kernel's default.
inline void co_prefer_max_shared(const void* kernel) {
  static const void* seen[128];
  static int n = 0;
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("COHERYN_CARVEOUT");
    enabled = (e && e[0] == '0') ? 0 : 1;
  }
  if (!enabled) return;
  for (int i = 0; i < n; ++i)
    if (seen[i] == kernel) return;
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
  if (n < 128) seen[n++] = kernel;
}

template <typename... KArgs, typename... Args>
inline cudaError_t co_launch_ex(bool keep_l1, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t stream, Args... args) {
  if (!keep_l1) co_prefer_max_shared((const void*)kernel);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = co_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
// The same for a kernel whose CTAs form clusters of `cluster_x` along x (1: no clusters).
template <typename... KArgs, typename... Args>
inline cudaError_t co_launch_cluster(int cluster_x, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args... args) {
  co_prefer_max_shared((const void*)kernel);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (co_pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t co_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
  return co_launch_ex(false, kernel, grid, block, smem, stream, args...);
}

template <typename T>
__device__ __forceinline__ float co_to_float(T v);
template <>
__device__ __forceinline__ float co_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float co_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T>
__device__ __forceinline__ T co_from_float(float v);
template <>
__device__ __forceinline__ float co_from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 co_from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Loads element i of an array whose dtype is only known at run time (small vectors:
// norm weights, biases).
__device__ __forceinline__ float co_load_any(const void* p, int dtype, size_t i) {
  return dtype == CO_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

__device__ __forceinline__ float co_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float co_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed combination order (warp shuffles, then warp 0 adds the
// per-warp partials in order): the result does not depend on scheduling.
__device__ __forceinline__ float co_block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = co_warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = co_warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
