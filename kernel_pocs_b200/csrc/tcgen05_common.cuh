// Shared pieces of the tcgen05 kernels: mbarrier waits that are bounded in time, tiled bulk loads,
// shared-memory matrix descriptors, TMEM reads, the CTA-pair (cta_group::2) primitives, and the
// host-side tensor-map encoder.  No load here uses cluster multicast.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace swiglu_b200 {
namespace tc {

constexpr long long WAIT_CYCLES = 1000000000LL;  // ~0.5 s of SM clock per wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* b, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the barrier did not flip within `limit` cycles of the SM clock
// or when another thread has already reported a failure; the first failure stores `code` in *status.
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, int* status, int code,
                                          long long limit = WAIT_CYCLES) {
  if (mbar_try_wait(b, parity)) return true;
  const long long t0 = clock64();
  for (int spin = 0;; ++spin) {
    if (mbar_try_wait(b, parity)) return true;
    if ((spin & 63) == 63) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (clock64() - t0 > limit) {
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// The barrier in front of every kernel's teardown.  All threads of the CTA take part in ONE barrier
// that also tells each of them whether any thread saw a failure code in the status word, so the
// whole CTA takes the same branch: reading the word thread by thread could split the CTA between a
// barrier inside the branch and the next barrier after it when another CTA reports at that moment.
// After a failure the CTA lets copies that are still in flight land in its shared memory before the
// memory is handed to another CTA.  (The two CTAs of a pair may decide differently; both reach the
// cluster barrier that follows either way.)
__device__ __forceinline__ void settle_before_teardown(const int* status) {
  if (__syncthreads_or(*reinterpret_cast<const volatile int*>(status) != 0)) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
    __syncthreads();
  }
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor: K-major tile of 128-byte rows, 128-byte swizzle, 8-row groups
// 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}

// Same for K-major tiles whose rows are ROW_BYTES = 32, 64 or 128 bytes long, stored with the swizzle of
// that span (8-row groups 8 * ROW_BYTES apart).  Layout codes: 128-byte swizzle 2, 64-byte 4, 32-byte 6.
template <int ROW_BYTES>
__device__ __forceinline__ uint64_t umma_desc_rows(uint32_t smem_addr) {
  static_assert(ROW_BYTES == 32 || ROW_BYTES == 64 || ROW_BYTES == 128, "swizzle spans are 32, 64 or 128 bytes");
  constexpr uint64_t layout = ROW_BYTES == 128 ? 2 : ROW_BYTES == 64 ? 4 : 6;
  return (uint64_t)((smem_addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)((8 * ROW_BYTES) >> 4) << 32) |
         (1ull << 46) | (layout << 61);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

// Shared-memory matrix descriptor for an operand whose contiguous dimension is M or N ("MN-major"),
// stored as chunks of 64 contiguous elements (128 bytes, 128-byte swizzle) by 8-row groups along K:
// 8-row groups are 1024 bytes apart (stride offset), 64-element chunks `chunk_bytes` apart (leading
// offset).  One MMA (K = 16) consumes two 8-row groups, i.e. 2048 bytes: add 128 address units.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t chunk_bytes) {
  return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)((chunk_bytes >> 4) & 0x3fffu) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// ---- CTA pairs ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive (optionally announcing transaction bytes) on a barrier given by its cluster-window address
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// No cluster-scope release here: the producer has written nothing the leader must see, and a
// cluster-scope release per K block stalled the producer thread.
__device__ __forceinline__ void remote_expect_tx(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool try_wait_cluster(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
  return ok != 0;
}
// SLEEP_NS > 0: pause that long between polls.  For waits that last a whole tile (the epilogue warps waiting for
// an accumulator): every poll is a shared-memory access, and several warps polling flat out take bandwidth from
// the operand traffic of the MMAs they are waiting for.
template <bool CLUSTER_SCOPE, int SLEEP_NS = 0>
__device__ __forceinline__ bool wait(uint64_t* b, uint32_t parity, int* status, int code,
                                     long long limit = WAIT_CYCLES) {
  auto poll = [&] { return CLUSTER_SCOPE ? try_wait_cluster(b, parity) : mbar_try_wait(b, parity); };
  if (poll()) return true;
  const long long t0 = clock64();
  for (int spin = 0;; ++spin) {
    if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
    if (poll()) return true;
    if ((spin & 63) == 63) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (clock64() - t0 > limit) {
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}
// tiled load whose completion bytes are credited to a barrier of the pair's leader CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(leader_bar) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p; }"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this shared-memory offset in BOTH CTAs once the MMAs issued so far are done
__device__ __forceinline__ void commit_both(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}

// ---- host ------------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled encode_fn() {
  static std::once_flag once;
  static EncodeTiled fn = nullptr;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(sym);
  });
  return fn;
}

// [rows, k] bf16 row-major matrix, boxes of `box_rows` rows x 64 elements (128 bytes) along the contiguous
// dimension (`box_cols` = 16 or 32 for narrower boxes), swizzle of the box's row length, zero fill outside
// the matrix.
inline bool make_map_uncached(CUtensorMap* map, const void* base, long long rows, long long k, int box_rows,
                              int box_cols) {
  EncodeTiled enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  // the swizzle span equals the box's row length: 64 elements -> 128 bytes, 32 -> 64, 16 -> 32
  const CUtensorMapSwizzle swizzle = box_cols == 64   ? CU_TENSOR_MAP_SWIZZLE_128B
                                     : box_cols == 32 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                      : CU_TENSOR_MAP_SWIZZLE_32B;
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A descriptor depends on nothing but these arguments, and encoding one costs about a microsecond of host
// time, nine times per LoRA launch; training loops present the same buffers again and again (a caching
// allocator hands the same addresses back), so each host thread keeps the last descriptors it built.
inline bool make_map(CUtensorMap* map, const void* base, long long rows, long long k, int box_rows = 128,
                     int box_cols = 64) {
  struct Entry {
    CUtensorMap map;
    const void* base;
    long long rows, k;
    int box_rows, box_cols;
    bool valid;
  };
  constexpr int kEntries = 64;
  thread_local Entry cache[kEntries] = {};
  const unsigned long long a = (unsigned long long)(uintptr_t)base;
  const unsigned long long hsh = (a >> 9) ^ (a >> 21) ^ ((unsigned long long)rows * 0x9e3779b97f4a7c15ull) ^
                                 ((unsigned long long)k << 7) ^ (unsigned long long)(box_rows * 31 + box_cols);
  Entry& slot = cache[hsh % kEntries];
  if (slot.valid && slot.base == base && slot.rows == rows && slot.k == k && slot.box_rows == box_rows &&
      slot.box_cols == box_cols) {
    *map = slot.map;
    return true;
  }
  if (!make_map_uncached(map, base, rows, k, box_rows, box_cols)) return false;
  slot.map = *map;
  slot.base = base;
  slot.rows = rows;
  slot.k = k;
  slot.box_rows = box_rows;
  slot.box_cols = box_cols;
  slot.valid = true;
  return true;
}

}  // namespace tc
}  // namespace swiglu_b200
