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
//   * Work is cut into tiles of 128 token rows x 64 columns, numbered along the rows of the matrix.  The CTAs
//     (one per SM) take short runs of consecutive tiles in turn, so that together they read and write one
//     contiguous band of E, G and h at any moment: the order of the work alone is worth 10 % of bandwidth.
//   * Per tile one thread loads E, G (128 x 64) and Bg, Bu (64 rows) into a ring of stages that takes all the
//     shared memory left (3 to 5 stages); XAg / XAu tiles (128 rows, rank padded to 16, 32 or 64 by the loads'
//     zero fill) change with the row tile and have a small ring of their own.  One thread issues two M=128,
//     N=64 MMAs per 16 ranks into TMEM (double buffered), which yield the adapter terms in the
//     row-per-thread layout the epilogue reads.
//   * Sixteen epilogue warps (four per TMEM lane quarter; all on one tile, or two sets of eight on alternate
//     tiles) add the terms to E and G taken from the swizzled shared-memory tiles, apply SwiGLU in fp32 and
//     write the results back into the stage: h over E, or, when e and g are wanted, e and g over E and G and
//     h into a third tile of the stage.  Each warp reports its part of a tile on the stage's mbarrier; the
//     warps never wait for one another.
//   * One thread stores finished tiles with bulk tensor stores, which also clip at the matrix edge, and
//     returns a stage to the loads when its stores have read it.
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
constexpr int EG_BYTES = TM * TN * 2;           // 16 KiB
constexpr int EPI_WARPS = 16;
// warps 0..3: loads, MMA issue, stores, idle; the epilogue warps start at a multiple of four so that
// warp & 3 is the TMEM lane quarter a warp may read
constexpr int FIRST_EPI_WARP = 4;
constexpr int THREADS = 32 * (FIRST_EPI_WARP + EPI_WARPS);
constexpr int ACC_BUFS = 2;                     // accumulator buffers in TMEM, (64 gate + 64 up) fp32 columns each
constexpr int TMEM_COLS = 256;
// kind::f16, D fp32, A and B bf16 K-major, M = 128, N = 64
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);

// What was tuned by measurement, per padded rank and per kernel (H: h alone is written; EG: e and g as well).
//   run       Tiles are numbered along the rows of the matrix (row tile major).  CTA b of G takes `run`
//             consecutive tiles, skips the (G - 1) * run that the other CTAs take, and so on, so that at any
//             moment the CTAs together read and write one contiguous band of the matrices.
//   xa_slots  depth of the ring of XA tiles, which change with the row tile: with short runs that is every
//             tile or two, and the loads of E and G run ahead only as far as this ring lets them.
//   lag       After it has issued the stores of a tile, the storing thread waits until all but the stores of
//             its last `lag` tiles have read their shared memory, and returns the stage of the tile `lag`
//             tiles back to the loads: 0 keeps one tile's stores in flight, 1 two, at the price of a stage
//             that stays taken for longer.
//   groups    The epilogue warps work as one set of sixteen on every tile (16 columns per warp) or as two
//             sets of eight on alternate tiles (32 columns per warp).
// Measured on M 16384 x N 14336 (and checked on four smaller shapes): rank 16 H 6.57 TB/s and EG 5.9-6.0 TB/s
// with the settings below; for H run 1 / 4 / 8 give 6.42 / 6.56-6.63 / 6.08, lag 2 6.09, and one long run of
// tiles / G per CTA 5.3-6.0; rank 64 H 5.63 against 4.45 with lag 1.  The response is not monotonic in any of
// the four: what is being tuned is how the reads and writes of 148 SMs meet in DRAM.
struct Tune {
  int run, xa_slots, lag, groups;
};
#ifndef SWIGLU_LORA_TUNE_16_H
#define SWIGLU_LORA_TUNE_16_H {2, 2, 1, 1}
#endif
#ifndef SWIGLU_LORA_TUNE_16_EG
#define SWIGLU_LORA_TUNE_16_EG {1, 3, 0, 2}
#endif
#ifndef SWIGLU_LORA_TUNE_32_H
#define SWIGLU_LORA_TUNE_32_H {2, 2, 0, 1}
#endif
#ifndef SWIGLU_LORA_TUNE_32_EG
#define SWIGLU_LORA_TUNE_32_EG {1, 2, 0, 2}
#endif
#ifndef SWIGLU_LORA_TUNE_64_H
#define SWIGLU_LORA_TUNE_64_H {2, 2, 0, 1}
#endif
#ifndef SWIGLU_LORA_TUNE_64_EG  // (room for one pair of XA tiles only: long runs, few changes of row tile)
#define SWIGLU_LORA_TUNE_64_EG {8, 1, 0, 2}
#endif
template <int RK, bool SAVE>
constexpr Tune tune() {
  if (RK == 16) return SAVE ? Tune SWIGLU_LORA_TUNE_16_EG : Tune SWIGLU_LORA_TUNE_16_H;
  if (RK == 32) return SAVE ? Tune SWIGLU_LORA_TUNE_32_EG : Tune SWIGLU_LORA_TUNE_32_H;
  return SAVE ? Tune SWIGLU_LORA_TUNE_64_EG : Tune SWIGLU_LORA_TUNE_64_H;
}

// Shared-memory layout for a rank padded to RK (16, 32 or 64).  A stage holds the E and G tiles, the two
// adapter tiles and, when e and g are written out (they replace E and G in place), a tile for h; without
// them h replaces E.  The ring of stages takes all the shared memory that the XA tiles leave.
template <int RK, bool SAVE>
struct Cfg {
  static constexpr Tune T = tune<RK, SAVE>();
  static constexpr int RUN = T.run, XA_SLOTS = T.xa_slots, LAG = T.lag, GROUPS = T.groups;
  static constexpr int XA_BYTES = TM * RK * 2;
  static constexpr int B_BYTES = TN * RK * 2;
  static constexpr int H_BYTES = SAVE ? EG_BYTES : 0;
  static constexpr int B_OFFSET = 2 * EG_BYTES + H_BYTES;
  static constexpr int LOAD_BYTES = 2 * EG_BYTES + 2 * B_BYTES;
  static constexpr int STAGE_BYTES = B_OFFSET + 2 * B_BYTES;
  static constexpr int XA_RING_BYTES = XA_SLOTS * 2 * XA_BYTES;
  static constexpr int STAGES = (227 * 1024 - XA_RING_BYTES - 1024 - 512) / STAGE_BYTES;
  static constexpr int SMEM_BYTES = XA_RING_BYTES + STAGES * STAGE_BYTES + 1024 + 512;  // alignment slack, barriers
  static constexpr int GROUP_WARPS = EPI_WARPS / GROUPS;
  static constexpr int CW = 64 / (GROUP_WARPS / 4);  // columns of a tile handled by one warp
  static_assert(RUN >= 1 && XA_SLOTS >= 1 && (GROUPS == 1 || GROUPS == 2), "settings");
  static_assert(STAGES >= 3 && STAGES <= 8, "ring depth");
  static_assert(LAG >= 0 && LAG < STAGES - 1, "stores in flight leave stages for the loads");
  static_assert((2 + 3 * STAGES + 2 * ACC_BUFS + 2 * XA_SLOTS) * 8 + 8 <= 512, "barriers fit their reserve");
};

struct LoraParams {
  int* status;
  long long m, n;
  int r;
  int save;  // also store e and g
  int run;   // consecutive tiles a CTA takes at a time (Tune::run, less for small problems)
  float s_gate, s_up;
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, const void* smem_src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y),
               "r"(smem_u32(smem_src)) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}

// The tiles of one CTA in the order it takes them: runs of `run` consecutive tiles, gridDim.x runs apart.
struct Walk {
  uint32_t tile, tiles, skip;
  int run, j;
  __device__ Walk(uint32_t tiles_, int run_)
      : tile(blockIdx.x * run_), tiles(tiles_), skip((gridDim.x - 1) * run_), run(run_), j(0) {}
  __device__ bool valid() const { return tile < tiles; }
  __device__ void next() {
    ++tile;
    if (++j == run) {
      j = 0;
      tile += skip;
    }
  }
};

template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t* r) {
  if constexpr (N == 32) tmem_ld32(taddr, r);
  else tmem_ld16(taddr, r);
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
  using C = Cfg<RK, SAVE>;
  constexpr int XA_BYTES = C::XA_BYTES, B_BYTES = C::B_BYTES, STAGE_BYTES = C::STAGE_BYTES, STAGES = C::STAGES,
                B_OFFSET = C::B_OFFSET, GROUPS = C::GROUPS, GROUP_WARPS = C::GROUP_WARPS, CW = C::CW;
  constexpr int XA_SLOTS = C::XA_SLOTS;
  unsigned char* xa_ring = smem;                  // slot: XAg tile, XAu tile
  unsigned char* ring = smem + C::XA_RING_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + STAGES * STAGE_BYTES);  // loads of a stage have landed
  uint64_t* done = full + STAGES;                 // every warp of the stage's set has written its results
  uint64_t* empty = done + STAGES;                // the stores of the stage have read it
  uint64_t* acc_full = empty + STAGES;            // [ACC_BUFS]
  uint64_t* acc_empty = acc_full + ACC_BUFS;      // [ACC_BUFS], every warp of the set that reads the buffer
  uint64_t* xa_full = acc_empty + ACC_BUFS;       // [XA_SLOTS]
  uint64_t* xa_empty = xa_full + XA_SLOTS;        // [XA_SLOTS]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xa_empty + XA_SLOTS);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t tiles_n = (uint32_t)((p.n + TN - 1) / TN);
  const uint32_t tiles = (uint32_t)((p.m + TM - 1) / TM) * tiles_n;  // (the host has checked that it fits)
  const Walk walk0(tiles, p.run);
  const int k_steps = (p.r + 15) / 16;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&done[s], GROUP_WARPS);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < ACC_BUFS; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], GROUP_WARPS);  // with several sets, buffer b is read by set b only
    }
    for (int x = 0; x < XA_SLOTS; ++x) {
      mbar_init(&xa_full[x], 1);
      mbar_init(&xa_empty[x], 1);
    }
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

  // Every role walks the same sequence of tiles; `it` counts them for the ring of stages, `xa_n` counts the
  // changes of row tile for the ring of XA tiles.
  if (warp == 0) {
    if (lane == 0) {
      uint32_t xa_n = 0, row_tile = ~0u;
      uint32_t it = 0;
      for (Walk w = walk0; w.valid(); w.next(), ++it) {
        const uint32_t m_tile = w.tile / tiles_n;
        const int m0 = (int)m_tile * TM;
        const int n0 = (int)(w.tile - m_tile * tiles_n) * TN;
        if (m_tile != row_tile) {
          row_tile = m_tile;
          const int x = (int)(xa_n % XA_SLOTS);
          if (xa_n >= XA_SLOTS && !mbar_wait(&xa_empty[x], (uint32_t)((xa_n / XA_SLOTS - 1) & 1), p.status, 500 + x))
            break;
          mbar_expect_tx(&xa_full[x], 2 * XA_BYTES);
          tma_load_2d(xa_ring + x * 2 * XA_BYTES, &map_xag, 0, m0, &xa_full[x]);
          tma_load_2d(xa_ring + x * 2 * XA_BYTES + XA_BYTES, &map_xau, 0, m0, &xa_full[x]);
          ++xa_n;
        }
        const int s = (int)(it % STAGES);
        if (it >= STAGES && !mbar_wait(&empty[s], (uint32_t)((it / STAGES - 1) & 1), p.status, 100 + s)) break;
        unsigned char* stage = ring + s * STAGE_BYTES;
        mbar_expect_tx(&full[s], C::LOAD_BYTES);
        tma_load_2d(stage, &map_e, n0, m0, &full[s]);
        tma_load_2d(stage + EG_BYTES, &map_g, n0, m0, &full[s]);
        tma_load_2d(stage + B_OFFSET, &map_bg, 0, n0, &full[s]);
        tma_load_2d(stage + B_OFFSET + B_BYTES, &map_bu, 0, n0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t xa_n = 0, row_tile = ~0u;
      uint64_t ag_desc = 0, au_desc = 0;
      uint32_t it = 0;
      for (Walk w = walk0; w.valid(); w.next(), ++it) {
        const uint32_t m_tile = w.tile / tiles_n;
        if (m_tile != row_tile) {
          // the XA tiles of the row tile left behind may be replaced once the MMAs issued so far are done
          if (xa_n > 0) umma_commit(&xa_empty[(xa_n - 1) % XA_SLOTS]);
          row_tile = m_tile;
          const int x = (int)(xa_n % XA_SLOTS);
          if (!mbar_wait(&xa_full[x], (uint32_t)((xa_n / XA_SLOTS) & 1), p.status, 510 + x)) break;
          ag_desc = umma_desc_rows<RK * 2>(smem_u32(xa_ring + x * 2 * XA_BYTES));
          au_desc = umma_desc_rows<RK * 2>(smem_u32(xa_ring + x * 2 * XA_BYTES + XA_BYTES));
          ++xa_n;
        }
        const int s = (int)(it % STAGES);
        const int b = (int)(it % ACC_BUFS);
        if (it >= ACC_BUFS && !mbar_wait(&acc_empty[b], (uint32_t)((it / ACC_BUFS - 1) & 1), p.status, 400 + b)) break;
        if (!mbar_wait(&full[s], (uint32_t)((it / STAGES) & 1), p.status, 200 + s)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t b_addr = smem_u32(ring + s * STAGE_BYTES + B_OFFSET);
        const uint64_t bg_desc = umma_desc_rows<RK * 2>(b_addr);
        const uint64_t bu_desc = umma_desc_rows<RK * 2>(b_addr + B_BYTES);
        const uint32_t d_gate = tmem_base + (uint32_t)b * 128u;
        for (int kk = 0; kk < k_steps; ++kk) {
          umma_bf16(d_gate, ag_desc + 2 * kk, bg_desc + 2 * kk, IDESC, kk != 0);
          umma_bf16(d_gate + 64, au_desc + 2 * kk, bu_desc + 2 * kk, IDESC, kk != 0);
        }
        // The adapter terms of this tile are in TMEM.  (The epilogue waits for this before it touches the
        // stage, and the stage is refilled only after the epilogue: the Bg / Bu tiles need no release.)
        umma_commit(&acc_full[b]);
      }
    }
  } else if (warp == 2) {
    // Stores.  One thread issues the bulk tensor stores of a tile once the tile's warps are done with it.
    if (lane == 0) {
      constexpr int LAG = C::LAG;
      uint32_t it = 0;
      for (Walk w = walk0; w.valid(); w.next(), ++it) {
        const uint32_t m_tile = w.tile / tiles_n;
        const int m0 = (int)m_tile * TM;
        const int n0 = (int)(w.tile - m_tile * tiles_n) * TN;
        const int s = (int)(it % STAGES);
        if (!mbar_wait(&done[s], (uint32_t)((it / STAGES) & 1), p.status, 700 + s)) break;
        unsigned char* stage = ring + s * STAGE_BYTES;
        if constexpr (SAVE) {
          tma_store_2d(&map_h, n0, m0, stage + 2 * EG_BYTES);
          tma_store_2d(&map_eo, n0, m0, stage);
          tma_store_2d(&map_go, n0, m0, stage + EG_BYTES);
        } else {
          tma_store_2d(&map_h, n0, m0, stage);
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        if (LAG == 0 || it >= (uint32_t)LAG) {
          asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(LAG) : "memory");
          mbar_arrive(&empty[(it - LAG) % STAGES]);
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
  } else if (warp >= FIRST_EPI_WARP) {
    const int quarter = warp & 3;                   // TMEM lane quarter this warp may read
    const int slot = (warp - FIRST_EPI_WARP) >> 2;  // 0 .. EPI_WARPS/4 - 1
    const int group = slot % GROUPS;                // takes the tiles with it % GROUPS == group
    const int part = slot / GROUPS;                 // which CW of the tile's 64 columns this warp handles
    const int row = quarter * 32 + lane;            // row of the tile owned by this thread
    const Consts one(1.0f, 1.0f);
    bool ok = true;
    {
      uint32_t it = 0;
      for (Walk w = walk0; w.valid(); w.next(), ++it) {
        if (GROUPS > 1 && (int)(it % GROUPS) != group) continue;
        const int s = (int)(it % STAGES);
        const int b = (int)(it % ACC_BUFS);
        unsigned char* e_tile = ring + s * STAGE_BYTES;
        unsigned char* g_tile = e_tile + EG_BYTES;
        unsigned char* h_tile = SAVE ? e_tile + 2 * EG_BYTES : e_tile;  // alone, h takes the place of E
        ok = mbar_wait(&full[s], (uint32_t)((it / STAGES) & 1), p.status, 600 + s) &&
             mbar_wait(&acc_full[b], (uint32_t)((it / ACC_BUFS) & 1), p.status, 300 + b);
        if (!__all_sync(0xffffffffu, ok)) ok = false;  // warp-uniform, for the warp-wide TMEM loads
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)b * 128u + (uint32_t)(part * CW);
        uint32_t lg[CW], lu[CW];
        tmem_ld_cols<CW>(t_row, lg);
        tmem_ld_cols<CW>(t_row + 64, lu);
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
        // This warp's part of the tiles is complete: make it visible to the bulk stores and tell the
        // storing thread.  The warps of a set never wait for one another.
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&done[s]);
      }
    }
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
    set(lora_swiglu_kernel<16, false>, Cfg<16, false>::SMEM_BYTES);
    set(lora_swiglu_kernel<16, true>, Cfg<16, true>::SMEM_BYTES);
#ifndef SWIGLU_LORA_ONLY16  // (tuning builds compile the rank-16 layout alone)
    set(lora_swiglu_kernel<32, false>, Cfg<32, false>::SMEM_BYTES);
    set(lora_swiglu_kernel<32, true>, Cfg<32, true>::SMEM_BYTES);
    set(lora_swiglu_kernel<64, false>, Cfg<64, false>::SMEM_BYTES);
    set(lora_swiglu_kernel<64, true>, Cfg<64, true>::SMEM_BYTES);
#endif
    if (!attr_ok) return SWIGLU_B200_ERR_DEVICE;
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm < 1)
      return SWIGLU_B200_ERR_DEVICE;
    if (dev < 64) sms[dev].store(n_sm, std::memory_order_release);
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(status, 0, sizeof(int), st) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
  const long long tiles_n = (n + TN - 1) / TN;
  const long long tiles = ((m + TM - 1) / TM) * tiles_n;
  if (tiles > 0x7fffffffLL) return SWIGLU_B200_ERR_SHAPE;  // (tens of terabytes per matrix)
  // A CTA takes its tiles in runs of Tune::run, or of that halved (and halved again ...) where the tiles of the
  // busiest CTA would otherwise exceed the best such split by more than 4 %: long runs share their XA tiles, but
  // on a small problem the last wave of long runs leaves most SMs idle.
  int run = rk == 16 ? (save ? Cfg<16, true>::RUN : Cfg<16, false>::RUN)
          : rk == 32 ? (save ? Cfg<32, true>::RUN : Cfg<32, false>::RUN)
                     : (save ? Cfg<64, true>::RUN : Cfg<64, false>::RUN);
  auto busiest = [&](int c) { return ((tiles + c - 1) / c + n_sm - 1) / n_sm * c; };  // tiles of the busiest CTA
  long long least = busiest(run);
  for (int c = run / 2; c >= 1; c /= 2) least = busiest(c) < least ? busiest(c) : least;
  while (run > 1 && busiest(run) * 100 > least * 104) run /= 2;
  const long long runs = (tiles + run - 1) / run;
  const unsigned grid = (unsigned)(runs < n_sm ? runs : n_sm);
  LoraParams p{static_cast<int*>(status), m, n, (int)r, save ? 1 : 0, run, s_gate, s_up};
  auto launch = [&](auto kernel, int bytes) {
    kernel<<<grid, THREADS, bytes, st>>>(me, mg, mxg, mxu, mbg, mbu, mh, meo, mgo, p);
  };
  if (rk == 16)
    save ? launch(lora_swiglu_kernel<16, true>, Cfg<16, true>::SMEM_BYTES) : launch(lora_swiglu_kernel<16, false>, Cfg<16, false>::SMEM_BYTES);
#ifndef SWIGLU_LORA_ONLY16
  else if (rk == 32)
    save ? launch(lora_swiglu_kernel<32, true>, Cfg<32, true>::SMEM_BYTES) : launch(lora_swiglu_kernel<32, false>, Cfg<32, false>::SMEM_BYTES);
  else
    save ? launch(lora_swiglu_kernel<64, true>, Cfg<64, true>::SMEM_BYTES) : launch(lora_swiglu_kernel<64, false>, Cfg<64, false>::SMEM_BYTES);
#else
  else
    return SWIGLU_B200_ERR_SHAPE;
#endif
  if (cudaGetLastError() != cudaSuccess) return SWIGLU_B200_ERR_LAUNCH;
  g_lora_launches.fetch_add(1, std::memory_order_relaxed);
  return SWIGLU_B200_OK;
}

}  // extern "C"
