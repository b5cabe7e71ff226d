// LoRA + SwiGLU epilogue for sm_100a:
//
//     e = E + s_gate * (XAg . Bg^T)      g = G + s_up * (XAu . Bu^T)      h = silu(e) * g
//
// E, G [M, N]: outputs of the frozen gate / up projections; XAg, XAu [M, r]: x . A^T of the two adapters;
// Bg, Bu [N, r]: the adapters' second factors; all bf16, r a multiple of 8 up to 64.  Optionally e and g
// (with the adapter terms added) are written out for a backward pass.  This is the step the reference
// performs with _fused_lora_swiglu_kernel (kernels/lora_mlp/experiments/v3/lora_mlp_kernel_v3.py:45-138),
// launched from fused_lora_swiglu (:141-200): a Triton tile kernel with two small tl.dot per tile.
//
// The operator streams 3 (or 5) M x N matrices, so it is bound by HBM bandwidth, but the rank-r products
// cost 4*r flops per output, too many for the fp32 pipes at that rate (64 flop per 6 bytes at r = 16); they
// go to the tcgen05 tensor cores, and all the traffic goes through the TMA engine:
//
//   * A CTA owns 128 token rows and walks a range of 64-column tiles.  XAg / XAu tiles (128 rows, rank
//     padded to 16, 32 or 64 by the loads' zero fill) are loaded once per range.
//   * Per tile the producer warp loads E, G (128 x 64) and Bg, Bu (64 rows) into a 3- or 4-stage ring.  One
//     thread issues two M=128, N=64 MMAs per 16 ranks into TMEM (double buffered), which yield the adapter
//     terms in the row-per-thread layout the epilogue reads.
//   * Sixteen epilogue warps, as two groups of eight that take alternate tiles (two warps per TMEM lane
//     quarter, 32 columns each), add the terms to E and G taken from the swizzled shared-memory tiles, apply
//     SwiGLU in fp32, write h (and e, g in place over the staged tiles) back to shared memory, and one
//     thread per group stores the tiles with bulk tensor stores, which also clip at the matrix edge.
// No load uses cluster multicast.  Every mbarrier wait is bounded; a wait that gives up records its code
// in the status word, the other waits then leave, and the CTA drains its copies, frees TMEM and returns.
#include "swiglu_b200.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>

#include "swiglu_kernels.cuh"
#include "tcgen05_common.cuh"

namespace {

using namespace swiglu_b200::tc;
using swiglu_b200::Consts;
using swiglu_b200::Math;

constexpr int TM = 128;                         // token rows per CTA tile
constexpr int TN = 64;                          // output columns per tile (one 128-byte swizzle span)
#ifndef SWIGLU_LORA_TILES_PER_RANGE
#define SWIGLU_LORA_TILES_PER_RANGE 4  // finer items balance the SMs better (16 -> 4: +3..6 %)
#endif
constexpr int TILES_PER_RANGE = SWIGLU_LORA_TILES_PER_RANGE;  // 64-column tiles per work item
constexpr int EG_BYTES = TM * TN * 2;           // 16 KiB
#ifndef SWIGLU_LORA_OUT_BUFS
#define SWIGLU_LORA_OUT_BUFS 2
#endif
constexpr int OUT_BUFS_PER_GROUP = SWIGLU_LORA_OUT_BUFS;  // h tiles of one epilogue group waiting for their bulk store
#ifndef SWIGLU_LORA_EPI_WARPS
#define SWIGLU_LORA_EPI_WARPS 16
#endif
constexpr int EPI_WARPS = SWIGLU_LORA_EPI_WARPS;  // EPI_WARPS / 4 warps share a TMEM lane quarter
#ifndef SWIGLU_LORA_GROUPS
#define SWIGLU_LORA_GROUPS 2
#endif
constexpr int THREADS = 64 + 32 * EPI_WARPS;
// accumulator buffers in TMEM, (64 gate + 64 up) fp32 columns each: one per epilogue group, at least two
constexpr int ACC_BUFS = SWIGLU_LORA_GROUPS > 2 ? SWIGLU_LORA_GROUPS : 2;
constexpr int TMEM_COLS = ACC_BUFS * 128 <= 256 ? 256 : 512;
#ifndef SWIGLU_LORA_STAGES16
#define SWIGLU_LORA_STAGES16 4
#endif
// kind::f16, D fp32, A and B bf16 K-major, M = 128, N = 64
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);

// Shared-memory layout for a rank padded to RK (16, 32 or 64): the narrower the adapter tiles, the more
// stages of E / G tiles fit, and bytes in flight are what this kernel's bandwidth comes from.
//
// GROUPS: the epilogue warps work as this many independent groups, each covering all four TMEM lane quarters
// and taking every GROUPS-th tile, so that one group's waits, barrier and store issue overlap the other's
// arithmetic, and a thread handles twice the columns per tile (half the per-tile bookkeeping per element).
template <int RK>
struct Cfg {
  static constexpr int XA_BYTES = TM * RK * 2;
  static constexpr int B_BYTES = TN * RK * 2;
  static constexpr int STAGE_BYTES = 2 * EG_BYTES + 2 * B_BYTES;
  static constexpr int GROUPS = RK == 64 ? 1 : SWIGLU_LORA_GROUPS;
  static constexpr int STAGES = RK == 16 ? SWIGLU_LORA_STAGES16 : 3;
  static constexpr int OUT_BUFS = GROUPS * OUT_BUFS_PER_GROUP;
  static constexpr int GROUP_WARPS = EPI_WARPS / GROUPS;
  static constexpr int CW = 64 / (GROUP_WARPS / 4);  // columns of a tile handled by one warp
  static constexpr int SMEM_BYTES = 2 * XA_BYTES + STAGES * STAGE_BYTES + OUT_BUFS * EG_BYTES + 1024 + 256;
  static_assert(GROUPS >= 1 && GROUPS <= 3 && EPI_WARPS % (4 * GROUPS) == 0, "one to three epilogue groups");
  static_assert(CW == 16 || CW == 32, "a warp reads 16 or 32 TMEM columns per accumulator");
  static_assert(SMEM_BYTES <= 227 * 1024, "exceeds the shared memory of an SM");
};

struct LoraParams {
  int* status;
  long long m, n;
  int r;
  int save;  // also store e and g
  float s_gate, s_up;
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, const void* smem_src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y),
               "r"(smem_u32(smem_src)) : "memory");
}
// barrier `id` over the `threads` threads of one epilogue group that also ANDs a predicate across them
__device__ __forceinline__ bool epilogue_all(bool ok, int id, int threads) {
  uint32_t all;
  asm volatile("{ .reg .pred p, q; setp.ne.u32 q, %1, 0; bar.red.and.pred p, %2, %3, q; selp.u32 %0, 1, 0, p; }"
               : "=r"(all) : "r"((uint32_t)ok), "r"(id), "r"(threads) : "memory");
  return all != 0;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}

template <int RK, bool SAVE>
__global__ void __launch_bounds__(THREADS, 1)
lora_swiglu_kernel(const __grid_constant__ CUtensorMap map_e, const __grid_constant__ CUtensorMap map_g,
                   const __grid_constant__ CUtensorMap map_xag, const __grid_constant__ CUtensorMap map_xau,
                   const __grid_constant__ CUtensorMap map_bg, const __grid_constant__ CUtensorMap map_bu,
                   const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_eo,
                   const __grid_constant__ CUtensorMap map_go, const LoraParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int XA_BYTES = Cfg<RK>::XA_BYTES, B_BYTES = Cfg<RK>::B_BYTES, STAGE_BYTES = Cfg<RK>::STAGE_BYTES,
                STAGES = Cfg<RK>::STAGES, GROUPS = Cfg<RK>::GROUPS, GROUP_WARPS = Cfg<RK>::GROUP_WARPS,
                CW = Cfg<RK>::CW, OUT_BUFS = Cfg<RK>::OUT_BUFS;
  unsigned char* xa_g = smem;
  unsigned char* xa_u = smem + XA_BYTES;
  unsigned char* ring = smem + 2 * XA_BYTES;
  unsigned char* outs = ring + STAGES * STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(outs + OUT_BUFS * EG_BYTES);
  uint64_t* empty = full + STAGES;        // MMA commit + one epilogue thread
  uint64_t* acc_full = empty + STAGES;            // [ACC_BUFS]
  uint64_t* acc_empty = acc_full + ACC_BUFS;      // [ACC_BUFS], every warp of the group that reads the buffer
  uint64_t* xa_full = acc_empty + ACC_BUFS;
  uint64_t* xa_empty = xa_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xa_empty + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long tiles_n = (p.n + TN - 1) / TN;
  const long long ranges_n = (tiles_n + TILES_PER_RANGE - 1) / TILES_PER_RANGE;
  const long long items = ((p.m + TM - 1) / TM) * ranges_n;
  const int k_steps = (p.r + 15) / 16;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 2);
    }
    for (int b = 0; b < ACC_BUFS; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], GROUP_WARPS);  // with several groups, buffer b is read by group b only
    }
    mbar_init(xa_full, 1);
    mbar_init(xa_empty, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  // Every role walks the same sequence: items (row tile, column range), tiles within the range.
  if (warp == 0) {
    if (lane == 0) {
      long long it = 0, item_no = 0;
      bool ok = true;
      for (long long item = blockIdx.x; item < items && ok; item += gridDim.x, ++item_no) {
        const int m0 = (int)(item / ranges_n) * TM;
        const long long t_lo = (item % ranges_n) * TILES_PER_RANGE;
        const long long t_hi = (t_lo + TILES_PER_RANGE) < tiles_n ? (t_lo + TILES_PER_RANGE) : tiles_n;
        if (item_no > 0) {
          ok = mbar_wait(xa_empty, (uint32_t)((item_no - 1) & 1), p.status, 500);
          if (!ok) break;
        }
        mbar_expect_tx(xa_full, 2 * XA_BYTES);
        tma_load_2d(xa_g, &map_xag, 0, m0, xa_full);
        tma_load_2d(xa_u, &map_xau, 0, m0, xa_full);
        for (long long t = t_lo; t < t_hi; ++t, ++it) {
          const int s = (int)(it % STAGES);
          if (it >= STAGES) {
            ok = mbar_wait(&empty[s], (uint32_t)((it / STAGES - 1) & 1), p.status, 100 + s);
            if (!ok) break;
          }
          unsigned char* stage = ring + s * STAGE_BYTES;
          const int n0 = (int)(t * TN);
          mbar_expect_tx(&full[s], STAGE_BYTES);
          tma_load_2d(stage, &map_e, n0, m0, &full[s]);
          tma_load_2d(stage + EG_BYTES, &map_g, n0, m0, &full[s]);
          tma_load_2d(stage + 2 * EG_BYTES, &map_bg, 0, n0, &full[s]);
          tma_load_2d(stage + 2 * EG_BYTES + B_BYTES, &map_bu, 0, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      long long it = 0, item_no = 0;
      bool ok = true;
      const uint64_t ag_desc = umma_desc_rows<RK * 2>(smem_u32(xa_g));
      const uint64_t au_desc = umma_desc_rows<RK * 2>(smem_u32(xa_u));
      for (long long item = blockIdx.x; item < items && ok; item += gridDim.x, ++item_no) {
        const long long t_lo = (item % ranges_n) * TILES_PER_RANGE;
        const long long t_hi = (t_lo + TILES_PER_RANGE) < tiles_n ? (t_lo + TILES_PER_RANGE) : tiles_n;
        ok = mbar_wait(xa_full, (uint32_t)(item_no & 1), p.status, 510);
        if (!ok) break;
        for (long long t = t_lo; t < t_hi; ++t, ++it) {
          const int s = (int)(it % STAGES);
          const int b = (int)(it % ACC_BUFS);
          if (it >= ACC_BUFS) {
            ok = mbar_wait(&acc_empty[b], (uint32_t)((it / ACC_BUFS - 1) & 1), p.status, 400 + b);
            if (!ok) break;
          }
          ok = mbar_wait(&full[s], (uint32_t)((it / STAGES) & 1), p.status, 200 + s);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t b_addr = smem_u32(ring + s * STAGE_BYTES + 2 * EG_BYTES);
          const uint64_t bg_desc = umma_desc_rows<RK * 2>(b_addr);
          const uint64_t bu_desc = umma_desc_rows<RK * 2>(b_addr + B_BYTES);
          const uint32_t d_gate = tmem_base + (uint32_t)b * 128u;
          for (int kk = 0; kk < k_steps; ++kk) {
            umma_bf16(d_gate, ag_desc + 2 * kk, bg_desc + 2 * kk, IDESC, kk != 0);
            umma_bf16(d_gate + 64, au_desc + 2 * kk, bu_desc + 2 * kk, IDESC, kk != 0);
          }
          umma_commit(&acc_full[b]);  // adapter terms of this tile are in TMEM
          umma_commit(&empty[s]);     // ... and the Bg / Bu tiles of the stage have been read
        }
        if (ok) umma_commit(xa_empty);  // the XA tiles may be replaced once these MMAs are done
      }
    }
  } else {
    const int quarter = warp & 3;                   // TMEM lane quarter this warp may read
    const int slot = (warp - 2) >> 2;               // 0 .. EPI_WARPS/4 - 1
    const int group = slot % GROUPS;                // epilogue group: takes the tiles with it % GROUPS == group
    const int part = slot / GROUPS;                 // which CW of the tile's 64 columns this warp handles
    const int row = quarter * 32 + lane;            // row of the tile owned by this thread
    const bool elected = (part == 0 && quarter == ((2 + 4 * group) & 3) && lane == 0);  // one thread per group
    const Consts one(1.0f, 1.0f);
    long long it = 0;
    int mine = 0;                                   // tiles this group has handled
    bool ok = true;
    for (long long item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int m0 = (int)(item / ranges_n) * TM;
      const long long t_lo = (item % ranges_n) * TILES_PER_RANGE;
      const long long t_hi = (t_lo + TILES_PER_RANGE) < tiles_n ? (t_lo + TILES_PER_RANGE) : tiles_n;
      for (long long t = t_lo; t < t_hi; ++t, ++it) {
        if (GROUPS > 1 && (int)(it % GROUPS) != group) continue;
        const int s = (int)(it % STAGES);
        const int b = (int)(it % ACC_BUFS);
        unsigned char* e_tile = ring + s * STAGE_BYTES;
        unsigned char* g_tile = e_tile + EG_BYTES;
        // Two h buffers per group: before the group's barrier of this tile its storing thread has waited for
        // the store of the previous tile to finish reading, so the next tile may overwrite that buffer.
        unsigned char* h_tile = outs + (group * OUT_BUFS_PER_GROUP + (mine % OUT_BUFS_PER_GROUP)) * EG_BYTES;
        ++mine;
        ok = mbar_wait(&full[s], (uint32_t)((it / STAGES) & 1), p.status, 600 + s) &&
             mbar_wait(&acc_full[b], (uint32_t)((it / ACC_BUFS) & 1), p.status, 300 + b);
        if (!__all_sync(0xffffffffu, ok)) ok = false;  // warp-uniform, for the warp-wide TMEM loads
        if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)b * 128u + (uint32_t)(part * CW);
        uint32_t lg[CW], lu[CW];
        if constexpr (CW == 32) {
          tmem_ld32(t_row, lg);
          tmem_ld32(t_row + 64, lu);
        } else {
          tmem_ld16(t_row, lg);
          tmem_ld16(t_row + 64, lu);
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        // the adapter terms are in registers: TMEM buffer b can take the MMAs of the tile after next
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[b]);
#pragma unroll
        for (int c = 0; c < CW; c += 8) {
          // 16-byte chunk (part*CW + c)/8 of this row inside the 128-byte-swizzled tile
          const int off = row * 128 + ((((part * CW + c) >> 3) ^ (row & 7)) << 4);
          const uint4 e4 = *reinterpret_cast<const uint4*>(e_tile + off);
          const uint4 g4 = *reinterpret_cast<const uint4*>(g_tile + off);
          const uint32_t ew[4] = {e4.x, e4.y, e4.z, e4.w}, gw[4] = {g4.x, g4.y, g4.z, g4.w};
          uint32_t hw[4], eo[4], go[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float e0 = fmaf(p.s_gate, __uint_as_float(lg[c + 2 * j]), __uint_as_float(ew[j] << 16));
            const float e1 = fmaf(p.s_gate, __uint_as_float(lg[c + 2 * j + 1]), __uint_as_float(ew[j] & 0xffff0000u));
            const float g0 = fmaf(p.s_up, __uint_as_float(lu[c + 2 * j]), __uint_as_float(gw[j] << 16));
            const float g1 = fmaf(p.s_up, __uint_as_float(lu[c + 2 * j + 1]), __uint_as_float(gw[j] & 0xffff0000u));
            __nv_bfloat162 hb = __floats2bfloat162_rn(Math<true>::fwd(e0, g0, one), Math<true>::fwd(e1, g1, one));
            hw[j] = *reinterpret_cast<uint32_t*>(&hb);
            if constexpr (SAVE) {
              __nv_bfloat162 eb = __floats2bfloat162_rn(e0, e1);
              __nv_bfloat162 gb = __floats2bfloat162_rn(g0, g1);
              eo[j] = *reinterpret_cast<uint32_t*>(&eb);
              go[j] = *reinterpret_cast<uint32_t*>(&gb);
            }
          }
          *reinterpret_cast<uint4*>(h_tile + off) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
          if constexpr (SAVE) {
            *reinterpret_cast<uint4*>(e_tile + off) = make_uint4(eo[0], eo[1], eo[2], eo[3]);
            *reinterpret_cast<uint4*>(g_tile + off) = make_uint4(go[0], go[1], go[2], go[3]);
          }
        }
        }
        // The shared-memory tiles are complete: make them visible to the bulk stores.  The threads of the
        // group meet here once per tile and agree on the outcome of their waits, so that none is left at a
        // later barrier waiting for a thread whose wait gave up.
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // the group's previous store has finished reading its h buffer, which the next tile overwrites
        if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        ok = epilogue_all(ok, 1 + group, 32 * GROUP_WARPS);
        if (!ok) break;
        if (elected) {
          const int n0 = (int)(t * TN);
          tma_store_2d(&map_h, n0, m0, h_tile);
          if constexpr (SAVE) {
            tma_store_2d(&map_eo, n0, m0, e_tile);
            tma_store_2d(&map_go, n0, m0, g_tile);
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          // the stage may be refilled once nothing reads it any more
          if constexpr (SAVE) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          mbar_arrive(&empty[s]);
        }
      }
    }
    if (elected) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  settle_before_teardown(p.status);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

std::atomic<uint64_t> g_lora_launches{0};

}  // namespace

extern "C" {

uint64_t swiglu_b200_lora_launch_count(void) { return g_lora_launches.load(std::memory_order_relaxed); }

int swiglu_b200_lora_swiglu_fwd(void* h, void* e_out, void* g_out, const void* e_base, const void* g_base,
                                const void* xa_gate, const void* xa_up, const void* b_gate, const void* b_up,
                                int64_t m, int64_t n, int64_t r, float s_gate, float s_up, void* status, int device,
                                void* stream) {
  if (m < 0 || n < 0 || r < 0) return SWIGLU_B200_ERR_SHAPE;
  if (m == 0 || n == 0) return SWIGLU_B200_OK;
  if (r == 0 || r > 64 || r % 8 != 0 || n % 8 != 0) return SWIGLU_B200_ERR_SHAPE;
  if (m > 0x7fffff00LL || n > 0x7fffff00LL) return SWIGLU_B200_ERR_SHAPE;
  if (!h || !e_base || !g_base || !xa_gate || !xa_up || !b_gate || !b_up || !status) return SWIGLU_B200_ERR_NULL;
  if ((e_out == nullptr) != (g_out == nullptr)) return SWIGLU_B200_ERR_NULL;
  if (((uintptr_t)h | (uintptr_t)e_out | (uintptr_t)g_out | (uintptr_t)e_base | (uintptr_t)g_base | (uintptr_t)xa_gate |
       (uintptr_t)xa_up | (uintptr_t)b_gate | (uintptr_t)b_up) % 16)
    return SWIGLU_B200_ERR_ALIGN;
  if ((uintptr_t)status % 4) return SWIGLU_B200_ERR_ALIGN;

  int prev = -1;
  bool switched = false;
  if (device >= 0) {
    if (cudaGetDevice(&prev) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
    if (prev != device) {
      if (cudaSetDevice(device) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
      switched = true;
    }
  }
  struct Restore {
    bool on;
    int dev;
    ~Restore() {
      if (on) cudaSetDevice(dev);
    }
  } restore{switched, prev};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;

  const bool save = e_out != nullptr;
  const int rk = r <= 16 ? 16 : r <= 32 ? 32 : 64;  // adapter tiles are padded to this rank by the loads' zero fill
  CUtensorMap me, mg, mxg, mxu, mbg, mbu, mh, meo, mgo;
  if (!make_map(&me, e_base, m, n, TM) || !make_map(&mg, g_base, m, n, TM) || !make_map(&mh, h, m, n, TM) ||
      !make_map(&meo, save ? e_out : h, m, n, TM) || !make_map(&mgo, save ? g_out : h, m, n, TM) ||
      !make_map(&mxg, xa_gate, m, r, TM, rk) || !make_map(&mxu, xa_up, m, r, TM, rk) ||
      !make_map(&mbg, b_gate, n, r, TN, rk) || !make_map(&mbu, b_up, n, r, TN, rk))
    return SWIGLU_B200_ERR_DEVICE;

  static std::atomic<int> sms[64];
  int n_sm = dev < 64 ? sms[dev].load(std::memory_order_acquire) : 0;
  if (n_sm == 0) {
    bool attr_ok = true;
    auto set = [&](auto kernel, int bytes) {
      attr_ok = attr_ok && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
    };
    set(lora_swiglu_kernel<16, false>, Cfg<16>::SMEM_BYTES);
    set(lora_swiglu_kernel<16, true>, Cfg<16>::SMEM_BYTES);
#ifndef SWIGLU_LORA_ONLY16  // (tuning builds compile the rank-16 layout alone)
    set(lora_swiglu_kernel<32, false>, Cfg<32>::SMEM_BYTES);
    set(lora_swiglu_kernel<32, true>, Cfg<32>::SMEM_BYTES);
    set(lora_swiglu_kernel<64, false>, Cfg<64>::SMEM_BYTES);
    set(lora_swiglu_kernel<64, true>, Cfg<64>::SMEM_BYTES);
#endif
    if (!attr_ok) return SWIGLU_B200_ERR_DEVICE;
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm < 1)
      return SWIGLU_B200_ERR_DEVICE;
    if (dev < 64) sms[dev].store(n_sm, std::memory_order_release);
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(status, 0, sizeof(int), st) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
  const long long tiles_n = (n + TN - 1) / TN;
  const long long items = ((m + TM - 1) / TM) * ((tiles_n + TILES_PER_RANGE - 1) / TILES_PER_RANGE);
  const unsigned grid = (unsigned)(items < n_sm ? items : n_sm);
  LoraParams p{static_cast<int*>(status), m, n, (int)r, save ? 1 : 0, s_gate, s_up};
  auto launch = [&](auto kernel, int bytes) {
    kernel<<<grid, THREADS, bytes, st>>>(me, mg, mxg, mxu, mbg, mbu, mh, meo, mgo, p);
  };
  if (rk == 16)
    save ? launch(lora_swiglu_kernel<16, true>, Cfg<16>::SMEM_BYTES) : launch(lora_swiglu_kernel<16, false>, Cfg<16>::SMEM_BYTES);
#ifndef SWIGLU_LORA_ONLY16
  else if (rk == 32)
    save ? launch(lora_swiglu_kernel<32, true>, Cfg<32>::SMEM_BYTES) : launch(lora_swiglu_kernel<32, false>, Cfg<32>::SMEM_BYTES);
  else
    save ? launch(lora_swiglu_kernel<64, true>, Cfg<64>::SMEM_BYTES) : launch(lora_swiglu_kernel<64, false>, Cfg<64>::SMEM_BYTES);
#else
  else
    return SWIGLU_B200_ERR_SHAPE;
#endif
  if (cudaGetLastError() != cudaSuccess) return SWIGLU_B200_ERR_LAUNCH;
  g_lora_launches.fetch_add(1, std::memory_order_relaxed);
  return SWIGLU_B200_OK;
}

}  // extern "C"
