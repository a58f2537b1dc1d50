// Pieces shared by the tcgen05 matrix-product kernels: mbarrier and TMA wrappers, the shared
// memory and instruction descriptors of tcgen05.mma for 128-byte swizzled K-major bfloat16
// tiles, the TMEM read, and the host-side tensor map of a row-major matrix.
#pragma once
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace {
constexpr int BK = 64;           // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr unsigned WAIT_LIMIT = 1u << 26;


__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; false if `limit` tries ran out.
__device__ __forceinline__ bool mbar_wait_limited(unsigned long long* bar, unsigned parity, unsigned limit) {
  const unsigned addr = smem_u32(bar);
  for (unsigned i = 0; i < limit; ++i) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
  return mbar_wait_limited(bar, parity, WAIT_LIMIT);
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

// A tile in shared memory (as the tensor map's box, 128-byte swizzled) to global memory; rows and
// columns beyond the tensor are not written.  The copies of a thread form bulk groups.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's groups still READ their shared memory / are still in flight.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Orders this thread's ordinary shared-memory writes before later copies of the async proxy.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, swizzled in
// 128-byte mode: start address >> 4, leading byte offset 1 (unused with a swizzle), stride
// byte offset 1024 >> 4 between groups of eight rows, descriptor version 1, layout type 2.
__device__ __forceinline__ unsigned long long umma_desc(const void* tile) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_u32(tile) & 0x3ffff) >> 4);
  d |= (unsigned long long)1 << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}

// Instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, N >> 3, M >> 4.
__host__ __device__ constexpr unsigned umma_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long da, unsigned long long db,
                                          unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The same read without the wait: several reads can be in flight before tmem_wait_ld().
__device__ __forceinline__ void tmem_ld32_nowait(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Thirty-two columns of this thread's lane are written from registers.
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// Descriptor of a 128-byte swizzled tile with explicit leading and stride byte offsets.
__device__ __forceinline__ unsigned long long umma_desc_offsets(const void* tile, unsigned lbo, unsigned sbo) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_u32(tile) & 0x3ffff) >> 4);
  d |= (unsigned long long)((lbo >> 4) & 0x3fff) << 16;
  d |= (unsigned long long)((sbo >> 4) & 0x3fff) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
// Instruction descriptor with operand B stored MN-major (its N index contiguous in memory).
__host__ __device__ constexpr unsigned umma_idesc_b_mn(int m, int n) { return umma_idesc(m, n) | (1u << 16); }
// The MMA with operand A read from tensor memory (bfloat16 pairs, one column per two k).
__device__ __forceinline__ void umma_bf16_a_tmem(unsigned tmem_d, unsigned tmem_a, unsigned long long db,
                                                 unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled)p;
  }
  return fn;
}

// Encoded tensor maps are kept: a map is a function of the address, the extents, the strides and
// the box alone, the same few dozen (weights, the step's activation buffers) come back every step,
// and encoding one costs the host about as much as launching a kernel.  Direct-mapped, 512 entries.
struct MapKey {
  const void* base;
  unsigned long long dims[3], strides[2];
  unsigned box[3];
  int rank;
  bool operator==(const MapKey& o) const {
    return base == o.base && rank == o.rank && dims[0] == o.dims[0] && dims[1] == o.dims[1] && dims[2] == o.dims[2] &&
           strides[0] == o.strides[0] && strides[1] == o.strides[1] && box[0] == o.box[0] && box[1] == o.box[1] &&
           box[2] == o.box[2];
  }
};
struct MapSlot { MapKey key; CUtensorMap map; bool used; };

bool cached_map(CUtensorMap* map, const MapKey& key) {
  static MapSlot slots[512];
  static std::mutex lock;
  unsigned long long h = (unsigned long long)(uintptr_t)key.base * 0x9E3779B97F4A7C15ull;
  h ^= (key.dims[0] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
  h ^= (key.dims[1] * 31 + key.dims[2] * 131 + key.strides[0] * 17 + key.strides[1] * 257 + key.box[1] * 7 + key.box[0] + key.box[2] * 3 +
        0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
  std::lock_guard<std::mutex> guard(lock);
  MapSlot& slot = slots[(h >> 20) & 511];
  if (slot.used && slot.key == key) { *map = slot.map; return true; }
  EncodeTiled fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {key.dims[0], key.dims[1], key.dims[2]};
  cuuint64_t strides[2] = {key.strides[0], key.strides[1]};
  cuuint32_t box[3] = {key.box[0], key.box[1], key.box[2]};
  cuuint32_t elem[3] = {1, 1, 1};
  if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)key.rank, const_cast<void*>(key.base), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  slot.key = key; slot.map = *map; slot.used = true;
  return true;
}

// A [rows, K] bfloat16 matrix with row stride ld (elements) as a 2-D tensor map whose box is
// box_rows x 64 elements, 128-byte swizzled, zero filled out of bounds.
bool make_map(CUtensorMap* map, const void* base, long rows, long K, long ld, int box_rows) {
  MapKey key = {};
  key.base = base; key.rank = 2;
  key.dims[0] = (unsigned long long)K; key.dims[1] = (unsigned long long)rows;
  key.strides[0] = (unsigned long long)ld * 2;
  key.box[0] = (unsigned)BK; key.box[1] = (unsigned)box_rows;
  return cached_map(map, key);
}

// A bfloat16 tensor of rank 2 or 3 (dims and byte strides innermost first, strides[0] being
// that of dims[1]) whose box is `box`, 128-byte swizzled, zero filled out of bounds.
bool make_map_nd(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                 const cuuint32_t* box) {
  MapKey key = {};
  key.base = base; key.rank = rank;
  for (int i = 0; i < rank; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides[i];
  return cached_map(map, key);
}
}  // namespace
