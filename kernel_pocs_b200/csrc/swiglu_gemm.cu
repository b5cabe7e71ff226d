// Fused gate/up projection + SwiGLU epilogue for sm_100a:
//
//     h[M, N] = silu((X Wg^T) * gm) * (X Wu^T) * dm        X [M, K], Wg, Wu [N, K], all bf16, K contiguous
//
// One kernel replaces two projection GEMMs plus the activation kernel, so the 2*M*N
// pre-activations are never written to or re-read from HBM (unless the caller asks for them for
// a backward pass).  The nearest code in the reference is its Triton dual-GEMM
// (kernels/lora_mlp/experiments/v2/lora_mlp_kernel_v2.py:32-138) and its cuBLASLt call with a
// SWISH epilogue (kernels/lora_mlp/experiments/v4/cublaslt_silu.cu:9-92); this is a dense
// contraction and therefore runs on the tcgen05 tensor cores.
//
// Structure of a CTA (one 128 x 128 tile of h, 192 threads):
//   warp 0      TMA producer: per 64-wide K block, three tiled bulk loads (X tile, Wg tile, Wu tile,
//               each 128 rows x 128 bytes, 128-byte swizzle) into a 4-stage shared-memory ring
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=256, K=16, bf16 -> fp32).  The
//               Wg and Wu tiles sit back to back in shared memory, so ONE instruction produces both
//               accumulators: TMEM columns [0,128) = gate, [128,256) = up.  Also owns TMEM alloc/free.
//   warps 2-5   epilogue: each thread owns one row of the tile, reads 16 gate and 16 up columns at a
//               time from TMEM, applies SwiGLU in fp32 and stores 32 bytes of bf16 h.
// No load uses cluster multicast.  Every mbarrier wait is bounded in time: when a wait gives up it
// records where in the caller's status word, every other wait then leaves at once, the CTA lets
// in-flight copies land, frees its TMEM and returns.
#include "swiglu_b200.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "swiglu_kernels.cuh"
#include "tcgen05_common.cuh"

namespace {

using namespace swiglu_b200::tc;

using swiglu_b200::ACT_GELU_ERF;
using swiglu_b200::ACT_GELU_TANH;
using swiglu_b200::ACT_SILU;
using swiglu_b200::Consts;
using swiglu_b200::Math;

constexpr int BM = 128;           // rows of X / h per tile
constexpr int BN = 128;           // columns of h per tile (gate and up each)
constexpr int BK = 64;            // K elements per stage: 128 bytes, one swizzle atom
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int TILE_BYTES = BM * BK * 2;                  // 16 KiB, same for X, Wg and Wu tiles
constexpr int STAGE_BYTES = 3 * TILE_BYTES;              // 48 KiB
constexpr int TMEM_COLS = 256;                           // 128 gate + 128 up fp32 columns
constexpr int THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

// tcgen05 instruction descriptor, kind::f16: D fp32, A and B bf16, both K-major, M=128, N=256.
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);

struct GemmParams {
  __nv_bfloat16* h;
  __nv_bfloat16* gate_out;  // optional pre-activations for a backward pass
  __nv_bfloat16* up_out;
  int* status;
  long long m, n, k;
  float gm, dm;
  int r;  // rank of the LoRA adapters added to both projections (pair kernel only), 0 for none
};

// Sixteen bf16 results of one row: one 32-byte store (a whole sector) where the outputs allow it, else two of 16.
__device__ __forceinline__ void store_16_results(__nv_bfloat16* dst, const uint32_t (&v)[8], bool aligned32) {
  if (aligned32) {
    asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(v[0]), "r"(v[1]), "r"(v[2]),
                 "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
  } else {
    uint4* d = reinterpret_cast<uint4*>(dst);
    d[0] = make_uint4(v[0], v[1], v[2], v[3]);
    d[1] = make_uint4(v[4], v[5], v[6], v[7]);
  }
}
// n is a multiple of 16, so a group of 16 results starts on a 32-byte boundary whenever the base does
__device__ __forceinline__ bool outputs_aligned32(const void* h, const void* gate_out, const void* up_out) {
  return ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(gate_out) |
           reinterpret_cast<uintptr_t>(up_out)) & 31) == 0;
}

__global__ void __launch_bounds__(THREADS, 1)
swiglu_gemm_fwd_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wg,
                       const __grid_constant__ CUtensorMap map_wu, const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte aligned bases
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_ready = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // m fastest: the CTAs of one wave share a few Wg/Wu tiles and walk down X
  const long long tiles_m = (p.m + BM - 1) / BM;
  const long long tile_m = blockIdx.x % tiles_m;
  const long long tile_n = blockIdx.x / tiles_m;
  const int m0 = (int)(tile_m * BM);
  const int n0 = (int)(tile_n * BN);
  const int k_blocks = (int)((p.k + BK - 1) / BK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_ready, 1);
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

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % STAGES;
        const uint32_t round = kb / STAGES;
        if (kb >= STAGES && !mbar_wait(&empty[s], (round - 1) & 1, p.status, 100 + s)) break;
        unsigned char* stage = smem + s * STAGE_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        tma_load_2d(stage, &map_x, kb * BK, m0, &full[s]);
        tma_load_2d(stage + TILE_BYTES, &map_wg, kb * BK, n0, &full[s]);
        tma_load_2d(stage + 2 * TILE_BYTES, &map_wu, kb * BK, n0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < k_blocks && ok; ++kb) {
        const int s = kb % STAGES;
        ok = mbar_wait(&full[s], (kb / STAGES) & 1, p.status, 200 + s);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t a_desc = umma_desc(a_addr);
        const uint64_t b_desc = umma_desc(a_addr + TILE_BYTES);  // Wg rows 0..127, Wu rows 128..255
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          // 16 K elements = 32 bytes = 2 descriptor address units further along each 128-byte row
          umma_bf16(tmem_base, a_desc + 2 * kk, b_desc + 2 * kk, IDESC, (kb | kk) != 0);
        }
        umma_commit(&empty[s]);  // arrives once these MMAs have finished reading the stage
      }
      if (ok) umma_commit(acc_ready);
    }
  } else {
    // epilogue warps 2..5 read TMEM lane quarters 2, 3, 0, 1
    const int quarter = warp & 3;
    const int row = m0 + quarter * 32 + lane;
    const Consts cst(p.gm, p.dm);
    const bool aligned32 = outputs_aligned32(p.h, p.gate_out, p.up_out);
    const bool ok = mbar_wait(acc_ready, 0, p.status, 300);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        uint32_t g[16], u[16];
        tmem_ld16(t_row + c, g);
        tmem_ld16(t_row + BN + c, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < p.m && n0 + c < p.n) {
          uint32_t hv[8], gv[8], uv[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
            const float u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
            __nv_bfloat162 hb = __floats2bfloat162_rn(Math<true>::fwd(g0, u0, cst), Math<true>::fwd(g1, u1, cst));
            __nv_bfloat162 gb = __floats2bfloat162_rn(g0, g1);
            __nv_bfloat162 ub = __floats2bfloat162_rn(u0, u1);
            hv[j] = *reinterpret_cast<uint32_t*>(&hb);
            gv[j] = *reinterpret_cast<uint32_t*>(&gb);
            uv[j] = *reinterpret_cast<uint32_t*>(&ub);
          }
          const long long off = (long long)row * p.n + n0 + c;
          // n is a multiple of 16 (checked on the host), so a 16-column group is all in or all out
          store_16_results(p.h + off, hv, aligned32);
          if (p.gate_out) {
            store_16_results(p.gate_out + off, gv, aligned32);
            store_16_results(p.up_out + off, uv, aligned32);
          }
        }
      }
    }
  }

  // Teardown.  After a failed wait, give copies that are still in flight time to land in this
  // CTA's shared memory before it is handed to another CTA.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  settle_before_teardown(p.status);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------
// Second kernel: CTA pairs (cta_group::2), persistent, double-buffered accumulators.
//
// A cluster of two CTAs computes a 256 x 128 tile of h.  Each CTA loads its own 128 rows of X and
// ONE of the two weight tiles (rank 0: Wg, rank 1: Wu); the leader's tcgen05.mma.cta_group::2
// (M=256, N=256, K=16) reads X rows from both CTAs' shared memory and treats the two weight tiles
// as the two halves of its N dimension, so each CTA's TMEM again holds gate in columns [0,128) and
// up in [128,256) for its 128 rows.  Per K block a CTA now pulls 32 KiB through L2 instead of
// 48 KiB.  Clusters walk the tiles persistently; TMEM holds two accumulator buffers so the
// epilogue of one tile overlaps the MMAs of the next.  Tiles are visited in bands of 8 row-tiles
// so that the X band and the weight tiles in flight stay in L2.
//
// LoRA adapters (p.r > 0): e = X.Wg^T + s_g (X.Ag^T).Bg^T and g likewise are ONE longer contraction,
//   [X | XA'] . [Wg | Bg']^T   with XA' = [s_g X.Ag^T | s_u X.Au^T]  (M x 2r, prepared by the caller),
// where the gate half of the MMA's N dimension sees Bg' = [Bg | 0] and the up half Bu' = [0 | Bu].  So after the
// K blocks of X come ceil(2r / 64) blocks whose A tile is loaded from XA' and whose B tile is loaded from Bg at
// column 64 j (rank 0) or from Bu at column 64 j - r (rank 1): the tiled loads fill whatever lies outside
// the r columns of the adapter matrix, to the left (negative coordinates) as to the right, with zeros.
namespace pair {

#ifndef SWIGLU_GEMM_PAIR_STAGES
#define SWIGLU_GEMM_PAIR_STAGES 6
#endif
constexpr int STAGES = SWIGLU_GEMM_PAIR_STAGES;
constexpr int STAGE_BYTES = 2 * TILE_BYTES;              // X tile + one weight tile
constexpr int ACC_BUFS = 2;
constexpr int TMEM_COLS = 512;
constexpr int BAND = 8;                                  // row-tiles (of 256 rows) per band
constexpr int EPI_COLS = 16;  // accumulator columns an epilogue thread takes per TMEM wait (32: no faster, the
                              // epilogue hides behind the next tile's MMAs either way)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((256u >> 4) << 24);

struct TileWalk {
  long long tiles_m, tiles_n, total;
  __device__ __forceinline__ TileWalk(long long m, long long n)
      : tiles_m((m + 2 * BM - 1) / (2 * BM)), tiles_n((n + BN - 1) / BN), total(tiles_m * tiles_n) {}
  __device__ __forceinline__ void at(long long t, int& m0, int& n0) const {
    const long long per_band = (long long)BAND * tiles_n;
    const long long band = t / per_band;
    const long long r = t - band * per_band;
    const long long rows_in_band = (tiles_m - band * BAND) < BAND ? (tiles_m - band * BAND) : BAND;
    const long long tn = r / rows_in_band;
    const long long tm = band * BAND + (r - tn * rows_in_band);
    m0 = (int)(tm * 2 * BM);
    n0 = (int)(tn * BN);
  }
};

// ACT: the gate activation of the epilogue (SiLU, or one of the two GELU forms of the GeGLU sibling).
template <int ACT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
swiglu_gemm_fwd_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wg,
                            const __grid_constant__ CUtensorMap map_wu, const __grid_constant__ CUtensorMap map_xa,
                            const __grid_constant__ CUtensorMap map_bg, const __grid_constant__ CUtensorMap map_bu,
                            const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);  // used in the leader only
  uint64_t* empty = full + STAGES;                                            // one copy per CTA
  uint64_t* acc_full = empty + STAGES;                                        // one copy per CTA
  uint64_t* acc_empty = acc_full + ACC_BUFS;                                  // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_BUFS);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cta_rank();
  const long long pair_id = blockIdx.x >> 1;
  const long long n_pairs = gridDim.x >> 1;
  const TileWalk walk(p.m, p.n);
  const int main_blocks = (int)((p.k + BK - 1) / BK);
  const int k_blocks = main_blocks + (p.r > 0 ? (2 * p.r + BK - 1) / BK : 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 2);    // one expect_tx arrival from each CTA's producer
      mbar_init(&empty[s], 1);   // the leader's commit
    }
    for (int b = 0; b < ACC_BUFS; ++b) {
      mbar_init(&acc_full[b], 1);   // the leader's commit
      mbar_init(&acc_empty[b], 8);  // four epilogue warps in each CTA
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before anyone arrives on them remotely
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const CUtensorMap* map_w = rank == 0 ? &map_wg : &map_wu;
      long long it = 0;
      bool ok = true;
      for (long long t = pair_id; t < walk.total && ok; t += n_pairs) {
        int m0, n0;
        walk.at(t, m0, n0);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          if (it >= STAGES) {
            ok = wait<false>(&empty[s], (uint32_t)((it / STAGES - 1) & 1), p.status, 100 + s);
            if (!ok) break;
          }
          const uint32_t leader_full = map_to_rank(smem_u32(&full[s]), 0);
          remote_expect_tx(leader_full, STAGE_BYTES);
          unsigned char* stage = smem + s * STAGE_BYTES;
          if (kb < main_blocks) {
            tma_load_2d_pair(stage, &map_x, kb * BK, m0 + (int)rank * BM, leader_full);
            tma_load_2d_pair(stage + TILE_BYTES, map_w, kb * BK, n0, leader_full);
          } else {
            const int c0 = (kb - main_blocks) * BK;  // column of XA' this block starts at
            tma_load_2d_pair(stage, &map_xa, c0, m0 + (int)rank * BM, leader_full);
            tma_load_2d_pair(stage + TILE_BYTES, rank == 0 ? &map_bg : &map_bu, rank == 0 ? c0 : c0 - p.r, n0,
                             leader_full);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      long long it = 0, i = 0;
      bool ok = true;
      for (long long t = pair_id; t < walk.total && ok; t += n_pairs, ++i) {
        const int b = (int)(i & 1);
        if (i >= ACC_BUFS) {
          ok = wait<true>(&acc_empty[b], (uint32_t)(((i >> 1) - 1) & 1), p.status, 400 + b);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t tmem_d = tmem_base + (uint32_t)b * 256u;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          ok = wait<false>(&full[s], (uint32_t)((it / STAGES) & 1), p.status, 200 + s);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t a_desc = umma_desc(a_addr);
          const uint64_t b_desc = umma_desc(a_addr + TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) umma_pair(tmem_d, a_desc + 2 * kk, b_desc + 2 * kk, IDESC, (kb | kk) != 0);
          commit_both(&empty[s]);
        }
        if (ok) commit_both(&acc_full[b]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const Consts cst(p.gm, p.dm);
    const bool aligned32 = outputs_aligned32(p.h, p.gate_out, p.up_out);
    long long i = 0;
    bool ok = true;
    for (long long t = pair_id; t < walk.total && ok; t += n_pairs, ++i) {
      int m0, n0;
      walk.at(t, m0, n0);
      const int b = (int)(i & 1);
      ok = wait<false, 200>(&acc_full[b], (uint32_t)((i >> 1) & 1), p.status, 300 + b);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = m0 + (int)rank * BM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)b * 256u;
#pragma unroll 1
      for (int c = 0; c < BN; c += EPI_COLS) {
        uint32_t g[EPI_COLS], u[EPI_COLS];
        if constexpr (EPI_COLS == 32) {
          tmem_ld32(t_row + c, g);
          tmem_ld32(t_row + BN + c, u);
        } else {
          tmem_ld16(t_row + c, g);
          tmem_ld16(t_row + BN + c, u);
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int q = 0; q < EPI_COLS / 16; ++q) {
          if (row < p.m && n0 + c + 16 * q < p.n) {  // n is a multiple of 16: a group of 16 columns is in or out
            uint32_t hv[8], gv[8], uv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float g0 = __uint_as_float(g[16 * q + 2 * j]), g1 = __uint_as_float(g[16 * q + 2 * j + 1]);
              const float u0 = __uint_as_float(u[16 * q + 2 * j]), u1 = __uint_as_float(u[16 * q + 2 * j + 1]);
              __nv_bfloat162 hb =
                  __floats2bfloat162_rn(Math<true, ACT>::fwd(g0, u0, cst), Math<true, ACT>::fwd(g1, u1, cst));
              __nv_bfloat162 gb = __floats2bfloat162_rn(g0, g1);
              __nv_bfloat162 ub = __floats2bfloat162_rn(u0, u1);
              hv[j] = *reinterpret_cast<uint32_t*>(&hb);
              gv[j] = *reinterpret_cast<uint32_t*>(&gb);
              uv[j] = *reinterpret_cast<uint32_t*>(&ub);
            }
            const long long off = (long long)row * p.n + n0 + c + 16 * q;
            store_16_results(p.h + off, hv, aligned32);
            if (p.gate_out) {
              store_16_results(p.gate_out + off, gv, aligned32);
              store_16_results(p.up_out + off, uv, aligned32);
            }
          }
        }
      }
      // this warp has drained its quarter of accumulator buffer b: tell the leader's MMA thread
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) remote_arrive(map_to_rank(smem_u32(&acc_empty[b]), 0));
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  settle_before_teardown(p.status);
  cluster_sync();  // the peer's shared memory and TMEM stay alive until the leader's MMAs are done
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace pair

// ------------------------------------------------------------------------------------------
// Third kernel: CTA pairs with a 256 x 256 tile of h (SWIGLU_B200_GEMM_TILE=wide; see forced_tile() below for
// what it gains and loses against the 256 x 128 tile).
//
// Same scheme as the pair kernel above, but per 16 contraction elements the leader issues TWO MMAs of N = 256 that
// share the X operand: one against a 256-row tile of Wg (accumulator columns [0, 256) = gate), one against the same
// rows of Wu (columns [256, 512) = up); each CTA loads its 128 rows of X and its 128-row half of both weight
// tiles.  Per K block a CTA pulls 48 KiB through L2 for twice the flops of the 32 KiB of the 256 x 128 tile (a
// quarter fewer operand bytes per flop: the narrow kernel sits past the knee of what one SM can pull through
// L2).  The price: one 512-column accumulator, so a tile's epilogue no longer hides behind the next tile's MMAs;
// sixteen epilogue warps (four per TMEM lane quarter, 64 columns of h each) keep that exposed part short.
// LoRA adapter blocks work as above: both CTAs load their half of [Bg | 0] for the gate MMA and of [0 | Bu] for
// the up MMA.
namespace wide {

#ifndef SWIGLU_GEMM_WIDE_STAGES
#define SWIGLU_GEMM_WIDE_STAGES 4
#endif
constexpr int STAGES = SWIGLU_GEMM_WIDE_STAGES;
constexpr int STAGE_BYTES = 3 * TILE_BYTES;              // X tile + this CTA's half of the Wg tile + of the Wu tile
constexpr int BNW = 256;                                 // columns of h per pair tile
constexpr int TMEM_COLS = 512;
constexpr int BAND = 8;                                  // row-tiles (of 256 rows) per band
constexpr int EPI_PARTS = 4;                             // epilogue warps per TMEM lane quarter
constexpr int PART_COLS = BNW / EPI_PARTS;               // columns of h one epilogue warp takes
constexpr int EPI_COLS = 16;
constexpr int W_THREADS = 64 + 128 * EPI_PARTS;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
static_assert(SMEM_BYTES <= 227 * 1024, "exceeds the shared memory of an SM");
constexpr uint32_t IDESC = pair::IDESC;                  // M = 256, N = 256, both operands K-major

struct TileWalk {
  long long tiles_m, tiles_n, total;
  __device__ __forceinline__ TileWalk(long long m, long long n)
      : tiles_m((m + 2 * BM - 1) / (2 * BM)), tiles_n((n + BNW - 1) / BNW), total(tiles_m * tiles_n) {}
  __device__ __forceinline__ void at(long long t, int& m0, int& n0) const {
    const long long per_band = (long long)BAND * tiles_n;
    const long long band = t / per_band;
    const long long r = t - band * per_band;
    const long long rows_in_band = (tiles_m - band * BAND) < BAND ? (tiles_m - band * BAND) : BAND;
    const long long tn = r / rows_in_band;
    const long long tm = band * BAND + (r - tn * rows_in_band);
    m0 = (int)(tm * 2 * BM);
    n0 = (int)(tn * BNW);
  }
};

template <int ACT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(W_THREADS, 1)
swiglu_gemm_fwd_wide_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wg,
                            const __grid_constant__ CUtensorMap map_wu, const __grid_constant__ CUtensorMap map_xa,
                            const __grid_constant__ CUtensorMap map_bg, const __grid_constant__ CUtensorMap map_bu,
                            const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);  // used in the leader only
  uint64_t* empty = full + STAGES;                                            // one copy per CTA
  uint64_t* acc_full = empty + STAGES;                                        // one copy per CTA
  uint64_t* acc_empty = acc_full + 1;                                         // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cta_rank();
  const long long pair_id = blockIdx.x >> 1;
  const long long n_pairs = gridDim.x >> 1;
  const TileWalk walk(p.m, p.n);
  const int main_blocks = (int)((p.k + BK - 1) / BK);
  const int k_blocks = main_blocks + (p.r > 0 ? (2 * p.r + BK - 1) / BK : 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 2);    // one expect_tx arrival from each CTA's producer
      mbar_init(&empty[s], 1);   // the leader's commit
    }
    mbar_init(acc_full, 1);                 // the leader's commit
    mbar_init(acc_empty, 8 * EPI_PARTS);    // every epilogue warp of both CTAs
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before anyone arrives on them remotely
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      long long it = 0;
      bool ok = true;
      for (long long t = pair_id; t < walk.total && ok; t += n_pairs) {
        int m0, n0;
        walk.at(t, m0, n0);
        const int w_row = n0 + (int)rank * BM;  // this CTA's 128 rows of both weight tiles
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          if (it >= STAGES) {
            ok = wait<false>(&empty[s], (uint32_t)((it / STAGES - 1) & 1), p.status, 100 + s);
            if (!ok) break;
          }
          const uint32_t leader_full = map_to_rank(smem_u32(&full[s]), 0);
          remote_expect_tx(leader_full, STAGE_BYTES);
          unsigned char* stage = smem + s * STAGE_BYTES;
          if (kb < main_blocks) {
            tma_load_2d_pair(stage, &map_x, kb * BK, m0 + (int)rank * BM, leader_full);
            tma_load_2d_pair(stage + TILE_BYTES, &map_wg, kb * BK, w_row, leader_full);
            tma_load_2d_pair(stage + 2 * TILE_BYTES, &map_wu, kb * BK, w_row, leader_full);
          } else {
            const int c0 = (kb - main_blocks) * BK;  // column of XA' this block starts at
            tma_load_2d_pair(stage, &map_xa, c0, m0 + (int)rank * BM, leader_full);
            tma_load_2d_pair(stage + TILE_BYTES, &map_bg, c0, w_row, leader_full);
            tma_load_2d_pair(stage + 2 * TILE_BYTES, &map_bu, c0 - p.r, w_row, leader_full);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      long long it = 0, i = 0;
      bool ok = true;
      for (long long t = pair_id; t < walk.total && ok; t += n_pairs, ++i) {
        if (i >= 1) {  // the one accumulator must have been drained by every epilogue warp of both CTAs
          ok = wait<true>(acc_empty, (uint32_t)((i - 1) & 1), p.status, 400);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          ok = wait<false>(&full[s], (uint32_t)((it / STAGES) & 1), p.status, 200 + s);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t a_desc = umma_desc(a_addr);
          const uint64_t g_desc = umma_desc(a_addr + TILE_BYTES);
          const uint64_t u_desc = umma_desc(a_addr + 2 * TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            umma_pair(tmem_base, a_desc + 2 * kk, g_desc + 2 * kk, IDESC, (kb | kk) != 0);
            umma_pair(tmem_base + (uint32_t)BNW, a_desc + 2 * kk, u_desc + 2 * kk, IDESC, (kb | kk) != 0);
          }
          commit_both(&empty[s]);
        }
        if (ok) commit_both(acc_full);
      }
    }
  } else {
    const int quarter = warp & 3;           // the TMEM lanes a warp may read: 32 * (warp % 4) ..
    const int part = (warp - 2) >> 2;       // which 64 columns of the tile
    const Consts cst(p.gm, p.dm);
    const bool aligned32 = outputs_aligned32(p.h, p.gate_out, p.up_out);
    long long i = 0;
    bool ok = true;
    for (long long t = pair_id; t < walk.total && ok; t += n_pairs, ++i) {
      int m0, n0;
      walk.at(t, m0, n0);
      ok = wait<false, 200>(acc_full, (uint32_t)(i & 1), p.status, 300);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int row = m0 + (int)rank * BM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = part * PART_COLS; c < (part + 1) * PART_COLS; c += EPI_COLS) {
        uint32_t g[EPI_COLS], u[EPI_COLS];
        tmem_ld16(t_row + c, g);
        tmem_ld16(t_row + BNW + c, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < p.m && n0 + c < p.n) {  // n is a multiple of 16: a group of 16 columns is in or out
          uint32_t hv[8], gv[8], uv[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
            const float u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
            __nv_bfloat162 hb =
                __floats2bfloat162_rn(Math<true, ACT>::fwd(g0, u0, cst), Math<true, ACT>::fwd(g1, u1, cst));
            __nv_bfloat162 gb = __floats2bfloat162_rn(g0, g1);
            __nv_bfloat162 ub = __floats2bfloat162_rn(u0, u1);
            hv[j] = *reinterpret_cast<uint32_t*>(&hb);
            gv[j] = *reinterpret_cast<uint32_t*>(&gb);
            uv[j] = *reinterpret_cast<uint32_t*>(&ub);
          }
          const long long off = (long long)row * p.n + n0 + c;
          store_16_results(p.h + off, hv, aligned32);
          if (p.gate_out) {
            store_16_results(p.gate_out + off, gv, aligned32);
            store_16_results(p.up_out + off, uv, aligned32);
          }
        }
      }
      // this warp has drained its part of the accumulator: tell the leader's MMA thread
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) remote_arrive(map_to_rank(smem_u32(acc_empty), 0));
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  settle_before_teardown(p.status);
  cluster_sync();  // the peer's shared memory and TMEM stay alive until the leader's MMAs are done
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace wide

// ------------------------------------------------------------------------------------------
// Fourth kernel: CTA pairs, 256 x 256 tile of h computed as TWO 256 x 128 half tiles whose contractions run a few
// K blocks apart (SWIGLU_B200_GEMM_TILE=staggered).
//
// The 256 x 256 tile above shares each X tile between two MMAs, which cuts the operand bytes per flop by a quarter,
// but its single 512-column accumulator leaves the epilogue exposed.  Here the tile is two independent streams:
// stream s computes columns [n0 + 128 s, n0 + 128 s + 128) of h exactly as the 256 x 128 kernel does (rank 0 loads
// the Wg rows, rank 1 the Wu rows, TMEM columns [256 s, 256 s + 128) = gate, [256 s + 128, 256 s + 256) = up), each
// issued by a thread of its own in the leader CTA.  Both streams read the same X tiles: X has a ring of its own
// whose slots are released when BOTH streams' MMAs have read them, and the weights of stream 1 are loaded LAG K
// blocks behind those of stream 0, so stream 1 reaches the end of a tile LAG blocks after stream 0.  When a stream
// has finished a tile it waits until the epilogue warps have taken its 256 accumulator columns into registers (a
// fraction of a microsecond); the other stream keeps the tensor pipe fed meanwhile.  No second accumulator buffer
// is needed, and an X tile crosses L2 once for both halves.
namespace stag {

#ifndef SWIGLU_GEMM_STAG_SX
#define SWIGLU_GEMM_STAG_SX 6
#endif
#ifndef SWIGLU_GEMM_STAG_SW
#define SWIGLU_GEMM_STAG_SW 4
#endif
#ifndef SWIGLU_GEMM_STAG_LAG
#define SWIGLU_GEMM_STAG_LAG 2
#endif
constexpr int SX = SWIGLU_GEMM_STAG_SX;                  // X ring: prefetch depth + LAG
constexpr int SW = SWIGLU_GEMM_STAG_SW;                  // each weight ring
constexpr int LAG = SWIGLU_GEMM_STAG_LAG;                // K blocks stream 1's weights are loaded behind stream 0's
constexpr int TMEM_COLS = 512;
constexpr int EPI_WARPS = 16;                            // per CTA: four per TMEM lane quarter, 32 columns of h each
constexpr int FIRST_EPI_WARP = 4;                        // warps 0..3: loads, stream 0, stream 1, idle
constexpr int S_THREADS = 32 * (FIRST_EPI_WARP + EPI_WARPS);
constexpr int RING_BYTES = (SX + 2 * SW) * TILE_BYTES;
constexpr int SMEM_BYTES = RING_BYTES + 1024 + 512;
static_assert(SMEM_BYTES <= 227 * 1024, "exceeds the shared memory of an SM");
static_assert(LAG >= 1 && LAG < SX - 1, "X tiles outlive the lag between the streams");
constexpr uint32_t IDESC = pair::IDESC;                  // M = 256, N = 256, both operands K-major

using TileWalk = wide::TileWalk;

template <int ACT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(S_THREADS, 1)
swiglu_gemm_fwd_staggered_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wg,
                                 const __grid_constant__ CUtensorMap map_wu, const __grid_constant__ CUtensorMap map_xa,
                                 const __grid_constant__ CUtensorMap map_bg, const __grid_constant__ CUtensorMap map_bu,
                                 const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* x_ring = smem;
  unsigned char* w_ring = smem + SX * TILE_BYTES;  // stream 0's SW slots, then stream 1's
  uint64_t* x_full = reinterpret_cast<uint64_t*>(smem + RING_BYTES);  // [SX]  used in the leader only
  uint64_t* x_empty = x_full + SX;                                    // [SX]  one copy per CTA, both streams commit
  uint64_t* w_full = x_empty + SX;                                    // [2][SW]  used in the leader only
  uint64_t* w_empty = w_full + 2 * SW;                                // [2][SW]  one copy per CTA
  uint64_t* acc_full = w_empty + 2 * SW;                              // [2]  one copy per CTA
  uint64_t* acc_empty = acc_full + 2;                                 // [2]  used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cta_rank();
  const long long pair_id = blockIdx.x >> 1;
  const long long n_pairs = gridDim.x >> 1;
  const TileWalk walk(p.m, p.n);
  const int main_blocks = (int)((p.k + BK - 1) / BK);
  const int k_blocks = main_blocks + (p.r > 0 ? (2 * p.r + BK - 1) / BK : 0);  // then the adapter blocks (see above)
  // tiles of this pair: pair_id, pair_id + n_pairs, ...
  const long long my_tiles = walk.total > pair_id ? (walk.total - pair_id + n_pairs - 1) / n_pairs : 0;
  const long long steps = my_tiles * k_blocks;  // K blocks of one stream over all of this pair's tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < SX; ++s) {
      mbar_init(&x_full[s], 2);    // one expect_tx arrival from each CTA's producer
      mbar_init(&x_empty[s], 2);   // the commits of both streams
    }
    for (int s = 0; s < 2 * SW; ++s) {
      mbar_init(&w_full[s], 2);
      mbar_init(&w_empty[s], 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(&acc_full[h], 1);               // the stream's commit
      mbar_init(&acc_empty[h], 2 * EPI_WARPS);  // every epilogue warp of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before anyone arrives on them remotely
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // Step g loads X and the stream-0 weights of K block g (counted over all tiles of the pair) and the
      // stream-1 weights of K block g - LAG.
      const CUtensorMap* map_w = rank == 0 ? &map_wg : &map_wu;
      const CUtensorMap* map_b = rank == 0 ? &map_bg : &map_bu;
      long long t0 = pair_id, t1 = pair_id;  // tiles of the two streams
      int kb0 = 0, kb1 = 0;
      int m0 = 0, n0 = 0, m1 = 0, n1 = 0;
      if (my_tiles > 0) {
        walk.at(t0, m0, n0);
        m1 = m0;
        n1 = n0;
      }
      bool ok = true;
      for (long long g = 0; g < steps + LAG && ok; ++g) {
        if (g < steps) {
          const int xs = (int)(g % SX), ws = (int)(g % SW);
          if (g >= SX) ok = wait<false>(&x_empty[xs], (uint32_t)((g / SX - 1) & 1), p.status, 100 + xs);
          if (ok && g >= SW) ok = wait<false>(&w_empty[ws], (uint32_t)((g / SW - 1) & 1), p.status, 110 + ws);
          if (!ok) break;
          const uint32_t xf = map_to_rank(smem_u32(&x_full[xs]), 0);
          remote_expect_tx(xf, TILE_BYTES);
          const uint32_t wf = map_to_rank(smem_u32(&w_full[ws]), 0);
          remote_expect_tx(wf, TILE_BYTES);
          if (kb0 < main_blocks) {
            tma_load_2d_pair(x_ring + xs * TILE_BYTES, &map_x, kb0 * BK, m0 + (int)rank * BM, xf);
            tma_load_2d_pair(w_ring + ws * TILE_BYTES, map_w, kb0 * BK, n0, wf);
          } else {
            const int c0 = (kb0 - main_blocks) * BK;  // column of XA' this block starts at
            tma_load_2d_pair(x_ring + xs * TILE_BYTES, &map_xa, c0, m0 + (int)rank * BM, xf);
            tma_load_2d_pair(w_ring + ws * TILE_BYTES, map_b, rank == 0 ? c0 : c0 - p.r, n0, wf);
          }
          if (++kb0 == k_blocks) {
            kb0 = 0;
            t0 += n_pairs;
            if (t0 < walk.total) walk.at(t0, m0, n0);
          }
        }
        if (g >= LAG) {
          const long long g1 = g - LAG;
          const int ws = (int)(g1 % SW);
          if (g1 >= SW) ok = wait<false>(&w_empty[SW + ws], (uint32_t)((g1 / SW - 1) & 1), p.status, 120 + ws);
          if (!ok) break;
          const uint32_t wf = map_to_rank(smem_u32(&w_full[SW + ws]), 0);
          remote_expect_tx(wf, TILE_BYTES);
          if (kb1 < main_blocks) {
            tma_load_2d_pair(w_ring + (SW + ws) * TILE_BYTES, map_w, kb1 * BK, n1 + BN, wf);
          } else {
            const int c0 = (kb1 - main_blocks) * BK;
            tma_load_2d_pair(w_ring + (SW + ws) * TILE_BYTES, map_b, rank == 0 ? c0 : c0 - p.r, n1 + BN, wf);
          }
          if (++kb1 == k_blocks) {
            kb1 = 0;
            t1 += n_pairs;
            if (t1 < walk.total) walk.at(t1, m1, n1);
          }
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    if (lane == 0 && rank == 0) {
      const int h = warp - 1;  // the stream this thread issues
      const uint32_t tmem_d = tmem_base + (uint32_t)h * 256u;
      long long it = 0;
      bool ok = true;
      for (long long i = 0; i < my_tiles && ok; ++i) {
        if (i >= 1) {  // the accumulator of this stream must have been taken by every epilogue warp of both CTAs
          ok = wait<true>(&acc_empty[h], (uint32_t)((i - 1) & 1), p.status, 400 + h);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int xs = (int)(it % SX), ws = (int)(it % SW);
          ok = wait<false>(&x_full[xs], (uint32_t)((it / SX) & 1), p.status, 200 + xs) &&
               wait<false>(&w_full[h * SW + ws], (uint32_t)((it / SW) & 1), p.status, 210 + h * SW + ws);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t a_desc = umma_desc(smem_u32(x_ring + xs * TILE_BYTES));
          const uint64_t b_desc = umma_desc(smem_u32(w_ring + (h * SW + ws) * TILE_BYTES));
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) umma_pair(tmem_d, a_desc + 2 * kk, b_desc + 2 * kk, IDESC, (kb | kk) != 0);
          commit_both(&x_empty[xs]);
          commit_both(&w_empty[h * SW + ws]);
        }
        if (ok) commit_both(&acc_full[h]);
      }
    }
  } else if (warp >= FIRST_EPI_WARP) {
    const int quarter = warp & 3;                    // the TMEM lanes a warp may read: 32 * (warp % 4) ..
    const int part = (warp - FIRST_EPI_WARP) >> 2;   // which 32 columns of a half tile
    const Consts cst(p.gm, p.dm);
    const bool aligned32 = outputs_aligned32(p.h, p.gate_out, p.up_out);
    bool ok = true;
    long long t = pair_id;
    for (long long i = 0; i < my_tiles && ok; ++i, t += n_pairs) {
      int m0, n0;
      walk.at(t, m0, n0);
      const int row = m0 + (int)rank * BM + quarter * 32 + lane;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        ok = wait<false, 200>(&acc_full[h], (uint32_t)(i & 1), p.status, 300 + h);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)h * 256u + (uint32_t)(part * 32);
        uint32_t g[32], u[32];
        tmem_ld32(t_row, g);
        tmem_ld32(t_row + BN, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        // this warp's part of the accumulator is in registers: tell the stream's thread in the leader
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) remote_arrive(map_to_rank(smem_u32(&acc_empty[h]), 0));
        const int col0 = n0 + h * BN + part * 32;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          if (row < p.m && col0 + 16 * q < p.n) {  // n is a multiple of 16: a group of 16 columns is in or out
            uint32_t hv[8], gv[8], uv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float g0 = __uint_as_float(g[16 * q + 2 * j]), g1 = __uint_as_float(g[16 * q + 2 * j + 1]);
              const float u0 = __uint_as_float(u[16 * q + 2 * j]), u1 = __uint_as_float(u[16 * q + 2 * j + 1]);
              __nv_bfloat162 hb =
                  __floats2bfloat162_rn(Math<true, ACT>::fwd(g0, u0, cst), Math<true, ACT>::fwd(g1, u1, cst));
              __nv_bfloat162 gb = __floats2bfloat162_rn(g0, g1);
              __nv_bfloat162 ub = __floats2bfloat162_rn(u0, u1);
              hv[j] = *reinterpret_cast<uint32_t*>(&hb);
              gv[j] = *reinterpret_cast<uint32_t*>(&gb);
              uv[j] = *reinterpret_cast<uint32_t*>(&ub);
            }
            const long long off = (long long)row * p.n + col0 + 16 * q;
            store_16_results(p.h + off, hv, aligned32);
            if (p.gate_out) {
              store_16_results(p.gate_out + off, gv, aligned32);
              store_16_results(p.up_out + off, uv, aligned32);
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  settle_before_teardown(p.status);
  cluster_sync();  // the peer's shared memory and TMEM stay alive until the leader's MMAs are done
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace stag

// ------------------------------------------------------------------------------------------ host

std::atomic<uint64_t> g_gemm_launches{0};

// SWIGLU_B200_GEMM=single selects the one-CTA-per-tile kernel; the CTA-pair kernel is the default.
bool use_pair_kernel() {
  static const bool pair_default = [] {
    const char* v = getenv("SWIGLU_B200_GEMM");
    return !(v && v[0] == 's');
  }();
  return pair_default;
}

// Number of 2-CTA clusters of the pair kernel that can be resident at once on `dev` (cached).
int pair_clusters(int dev, int* out) {
  static std::atomic<int> cache[64];
  if (dev < 64) {
    const int c = cache[dev].load(std::memory_order_acquire);
    if (c > 0) {
      *out = c;
      return SWIGLU_B200_OK;
    }
  }
  if (cudaFuncSetAttribute(pair::swiglu_gemm_fwd_pair_kernel<ACT_SILU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           pair::SMEM_BYTES) != cudaSuccess ||
      cudaFuncSetAttribute(pair::swiglu_gemm_fwd_pair_kernel<ACT_GELU_TANH>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES) != cudaSuccess ||
      cudaFuncSetAttribute(pair::swiglu_gemm_fwd_pair_kernel<ACT_GELU_ERF>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES) != cudaSuccess)
    return SWIGLU_B200_ERR_DEVICE;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 148, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = pair::SMEM_BYTES;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, pair::swiglu_gemm_fwd_pair_kernel<ACT_SILU>, &cfg) != cudaSuccess || n < 1)
    return SWIGLU_B200_ERR_DEVICE;
  if (const char* dbg = getenv("SWIGLU_B200_DEBUG")) {
    if (dbg[0] == '1') fprintf(stderr, "swiglu_b200: %d resident 2-CTA clusters on device %d\n", n, dev);
  }
  if (const char* force = getenv("SWIGLU_B200_GEMM_CLUSTERS")) {  // experiments only
    const int f = atoi(force);
    if (f > 0) n = f;
  }
  if (dev < 64) cache[dev].store(n, std::memory_order_release);
  *out = n;
  return SWIGLU_B200_OK;
}

// Same for the 256 x 256 tile kernel.
int wide_clusters(int dev, int* out) {
  static std::atomic<int> cache[64];
  if (dev < 64) {
    const int c = cache[dev].load(std::memory_order_acquire);
    if (c > 0) {
      *out = c;
      return SWIGLU_B200_OK;
    }
  }
  if (cudaFuncSetAttribute(wide::swiglu_gemm_fwd_wide_kernel<ACT_SILU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           wide::SMEM_BYTES) != cudaSuccess ||
      cudaFuncSetAttribute(wide::swiglu_gemm_fwd_wide_kernel<ACT_GELU_TANH>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, wide::SMEM_BYTES) != cudaSuccess ||
      cudaFuncSetAttribute(wide::swiglu_gemm_fwd_wide_kernel<ACT_GELU_ERF>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, wide::SMEM_BYTES) != cudaSuccess)
    return SWIGLU_B200_ERR_DEVICE;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 148, 1, 1);
  cfg.blockDim = dim3(wide::W_THREADS, 1, 1);
  cfg.dynamicSmemBytes = wide::SMEM_BYTES;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, wide::swiglu_gemm_fwd_wide_kernel<ACT_SILU>, &cfg) != cudaSuccess || n < 1)
    return SWIGLU_B200_ERR_DEVICE;
  if (dev < 64) cache[dev].store(n, std::memory_order_release);
  *out = n;
  return SWIGLU_B200_OK;
}

// Same for the staggered two-stream kernel.
int staggered_clusters(int dev, int* out) {
  static std::atomic<int> cache[64];
  if (dev < 64) {
    const int c = cache[dev].load(std::memory_order_acquire);
    if (c > 0) {
      *out = c;
      return SWIGLU_B200_OK;
    }
  }
  if (cudaFuncSetAttribute(stag::swiglu_gemm_fwd_staggered_kernel<ACT_SILU>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, stag::SMEM_BYTES) != cudaSuccess ||
      cudaFuncSetAttribute(stag::swiglu_gemm_fwd_staggered_kernel<ACT_GELU_TANH>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, stag::SMEM_BYTES) != cudaSuccess ||
      cudaFuncSetAttribute(stag::swiglu_gemm_fwd_staggered_kernel<ACT_GELU_ERF>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, stag::SMEM_BYTES) != cudaSuccess)
    return SWIGLU_B200_ERR_DEVICE;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 148, 1, 1);
  cfg.blockDim = dim3(stag::S_THREADS, 1, 1);
  cfg.dynamicSmemBytes = stag::SMEM_BYTES;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, stag::swiglu_gemm_fwd_staggered_kernel<ACT_SILU>, &cfg) != cudaSuccess ||
      n < 1)
    return SWIGLU_B200_ERR_DEVICE;
  if (dev < 64) cache[dev].store(n, std::memory_order_release);
  *out = n;
  return SWIGLU_B200_OK;
}

// Which pair kernel runs.  Default: the staggered two-stream 256 x 256 tile where the problem has at least one tile
// per resident cluster and its rounds of tiles over the resident clusters, at 0.97 of the time of two 256 x 128
// tiles each (0.95 in long runs under the power cap, level in short bursts), take no longer than the rounds of
// 256 x 128 tiles; else the 256 x 128 tile (twice the tiles: a finer last round, which decides for problems of a
// few rounds: at N 14336, K 4096 the rule picks the staggered tile for 512, 1536 and from 6144 rows on, which is
// where it measured faster, by 2 to 7 %, and the 256 x 128 tile for 1024, 2048, 3072 and 4096 rows).  SWIGLU_B200_GEMM_TILE =
// narrow | wide | staggered forces one.  (When the pre-activations are written too, a half tile's epilogue, now
// with three outputs per element, outlasts the few K blocks between the two streams and they wait for it: the
// staggered tile then gains 1 % over the 256 x 128 one instead of 5 %, 2.97 against 3.00 ms; with 16-byte stores
// it lost, 3.28 against 3.04 ms.)  Measured on X [16384, 4096] x W [14336, 4096]^T x 2, the kernels taking
// turns in one loop so that all see the same power cap: staggered 2.83-2.87 ms, 256 x 128 2.92-2.99, 256 x 256 with
// one accumulator 3.02, cuBLAS on the stacked weights (no activation) 2.87.  Under ncu on a 4096-row case the
// 256 x 256 tile takes the L2 throughput from 47 % to 35 % and the SM clock from 1.47 to 1.53 GHz against the
// 256 x 128 tile, with the tensor pipe busy 86-87 % of the active cycles either way, but its exposed epilogue
// takes the elapsed figure from 83 % to 79 %; the staggered kernel keeps the saving and hides the epilogue.
int forced_tile() {  // read at every call, so that a test can switch it
  const char* v = getenv("SWIGLU_B200_GEMM_TILE");
  return !v ? 0 : v[0] == 'n' ? 1 : v[0] == 'w' ? 2 : v[0] == 's' ? 3 : 0;
}

// Shared by swiglu_b200_gemm_fwd (r = 0) and swiglu_b200_lora_gemm_fwd (adapters of rank r, pair kernels only).
int gemm_fwd_impl(void* h, void* gate_out, void* up_out, const void* x, const void* w_gate, const void* w_up,
                  const void* xa_scaled, const void* b_gate, const void* b_up, int64_t m, int64_t n, int64_t k, int r,
                  float gm, float dm, void* status, int device, void* stream, int act = ACT_SILU) {
  if (m < 0 || n < 0 || k < 0) return SWIGLU_B200_ERR_SHAPE;
  if (m == 0 || n == 0) return SWIGLU_B200_OK;
  // 16-byte global strides for the tiled copies and 32-byte output groups
  if (k == 0 || k % 8 != 0 || n % 16 != 0) return SWIGLU_B200_ERR_SHAPE;
  if (m > 0x7fffff00LL || n > 0x7fffff00LL || k > 0x7fffff00LL) return SWIGLU_B200_ERR_SHAPE;
  if (!h || !x || !w_gate || !w_up || !status) return SWIGLU_B200_ERR_NULL;
  if ((gate_out == nullptr) != (up_out == nullptr)) return SWIGLU_B200_ERR_NULL;
  if (((uintptr_t)h | (uintptr_t)x | (uintptr_t)w_gate | (uintptr_t)w_up | (uintptr_t)gate_out | (uintptr_t)up_out) % 16)
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

  CUtensorMap map_x, map_wg, map_wu, map_xa, map_bg, map_bu;
  if (!make_map(&map_x, x, m, k) || !make_map(&map_wg, w_gate, n, k) || !make_map(&map_wu, w_up, n, k))
    return SWIGLU_B200_ERR_DEVICE;
  if (r > 0) {
    // boxes as wide as a K block over matrices of only 2r / r columns: the loads fill the rest with zeros
    if (!make_map(&map_xa, xa_scaled, m, 2 * r) || !make_map(&map_bg, b_gate, n, r) || !make_map(&map_bu, b_up, n, r))
      return SWIGLU_B200_ERR_DEVICE;
  } else {
    map_xa = map_x;  // never read
    map_bg = map_wg;
    map_bu = map_wu;
  }

  static std::atomic<bool> attr_set[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
  if (dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(swiglu_gemm_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return SWIGLU_B200_ERR_DEVICE;
    if (dev < 64) attr_set[dev].store(true, std::memory_order_release);
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(status, 0, sizeof(int), st) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
  if (use_pair_kernel() || r > 0 || act != ACT_SILU) {
    GemmParams pp{static_cast<__nv_bfloat16*>(h), static_cast<__nv_bfloat16*>(gate_out),
                  static_cast<__nv_bfloat16*>(up_out), static_cast<int*>(status), m, n, k, gm, dm, r};
    {
      int wide_resident = 0;
      const int rcw = wide_clusters(dev, &wide_resident);
      if (rcw != SWIGLU_B200_OK) return rcw;
      const long long wide_tiles = ((m + 2 * BM - 1) / (2 * BM)) * ((n + wide::BNW - 1) / wide::BNW);
      const int forced = forced_tile();
      int resident = 0;
      const int rcs = staggered_clusters(dev, &resident);
      if (rcs != SWIGLU_B200_OK) return rcs;
      // rounds of tiles over the resident clusters: a 256 x 256 tile takes 0.97 of two 256 x 128 ones
      int narrow_resident = 0;
      const int rcn = pair_clusters(dev, &narrow_resident);
      if (rcn != SWIGLU_B200_OK) return rcn;
      const long long narrow_tiles = ((m + 2 * BM - 1) / (2 * BM)) * ((n + BN - 1) / BN);
      const long long rounds_s = (wide_tiles + resident - 1) / resident;
      const long long rounds_n = (narrow_tiles + narrow_resident - 1) / narrow_resident;
      if (forced == 3 || (forced == 0 && wide_tiles >= resident && 194 * rounds_s <= 100 * rounds_n)) {
        const long long use = wide_tiles < resident ? wide_tiles : resident;
        const unsigned grid = (unsigned)(2 * use);
        if (act == ACT_GELU_TANH)
          stag::swiglu_gemm_fwd_staggered_kernel<ACT_GELU_TANH><<<grid, stag::S_THREADS, stag::SMEM_BYTES, st>>>(
              map_x, map_wg, map_wu, map_xa, map_bg, map_bu, pp);
        else if (act == ACT_GELU_ERF)
          stag::swiglu_gemm_fwd_staggered_kernel<ACT_GELU_ERF><<<grid, stag::S_THREADS, stag::SMEM_BYTES, st>>>(
              map_x, map_wg, map_wu, map_xa, map_bg, map_bu, pp);
        else
          stag::swiglu_gemm_fwd_staggered_kernel<ACT_SILU><<<grid, stag::S_THREADS, stag::SMEM_BYTES, st>>>(
              map_x, map_wg, map_wu, map_xa, map_bg, map_bu, pp);
        if (cudaGetLastError() != cudaSuccess) return SWIGLU_B200_ERR_LAUNCH;
        g_gemm_launches.fetch_add(1, std::memory_order_relaxed);
        return SWIGLU_B200_OK;
      }
      if (forced == 2) {
        const long long use = wide_tiles < wide_resident ? wide_tiles : wide_resident;
        const unsigned grid = (unsigned)(2 * use);
        if (act == ACT_GELU_TANH)
          wide::swiglu_gemm_fwd_wide_kernel<ACT_GELU_TANH><<<grid, wide::W_THREADS, wide::SMEM_BYTES, st>>>(
              map_x, map_wg, map_wu, map_xa, map_bg, map_bu, pp);
        else if (act == ACT_GELU_ERF)
          wide::swiglu_gemm_fwd_wide_kernel<ACT_GELU_ERF><<<grid, wide::W_THREADS, wide::SMEM_BYTES, st>>>(
              map_x, map_wg, map_wu, map_xa, map_bg, map_bu, pp);
        else
          wide::swiglu_gemm_fwd_wide_kernel<ACT_SILU><<<grid, wide::W_THREADS, wide::SMEM_BYTES, st>>>(
              map_x, map_wg, map_wu, map_xa, map_bg, map_bu, pp);
        if (cudaGetLastError() != cudaSuccess) return SWIGLU_B200_ERR_LAUNCH;
        g_gemm_launches.fetch_add(1, std::memory_order_relaxed);
        return SWIGLU_B200_OK;
      }
    }
    int clusters = 0;
    const int rc = pair_clusters(dev, &clusters);
    if (rc != SWIGLU_B200_OK) return rc;
    const long long pair_tiles = ((m + 2 * BM - 1) / (2 * BM)) * ((n + BN - 1) / BN);
    const long long use = pair_tiles < clusters ? pair_tiles : clusters;
    const unsigned grid = (unsigned)(2 * use);
    if (act == ACT_GELU_TANH)
      pair::swiglu_gemm_fwd_pair_kernel<ACT_GELU_TANH><<<grid, THREADS, pair::SMEM_BYTES, st>>>(
          map_x, map_wg, map_wu, map_xa, map_bg, map_bu, pp);
    else if (act == ACT_GELU_ERF)
      pair::swiglu_gemm_fwd_pair_kernel<ACT_GELU_ERF><<<grid, THREADS, pair::SMEM_BYTES, st>>>(
          map_x, map_wg, map_wu, map_xa, map_bg, map_bu, pp);
    else
      pair::swiglu_gemm_fwd_pair_kernel<ACT_SILU><<<grid, THREADS, pair::SMEM_BYTES, st>>>(
          map_x, map_wg, map_wu, map_xa, map_bg, map_bu, pp);
    if (cudaGetLastError() != cudaSuccess) return SWIGLU_B200_ERR_LAUNCH;
    g_gemm_launches.fetch_add(1, std::memory_order_relaxed);
    return SWIGLU_B200_OK;
  }
  GemmParams p{static_cast<__nv_bfloat16*>(h), static_cast<__nv_bfloat16*>(gate_out), static_cast<__nv_bfloat16*>(up_out),
               static_cast<int*>(status), m, n, k, gm, dm, 0};
  const long long tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
  if (tiles > 0x7fffffffLL) return SWIGLU_B200_ERR_SHAPE;
  swiglu_gemm_fwd_kernel<<<(unsigned)tiles, THREADS, SMEM_BYTES, st>>>(map_x, map_wg, map_wu, p);
  if (cudaGetLastError() != cudaSuccess) return SWIGLU_B200_ERR_LAUNCH;
  g_gemm_launches.fetch_add(1, std::memory_order_relaxed);
  return SWIGLU_B200_OK;
}

}  // namespace

extern "C" {

uint64_t swiglu_b200_gemm_launch_count(void) { return g_gemm_launches.load(std::memory_order_relaxed); }

int swiglu_b200_gemm_fwd(void* h, void* gate_out, void* up_out, const void* x, const void* w_gate, const void* w_up,
                         int64_t m, int64_t n, int64_t k, float gm, float dm, void* status, int device, void* stream) {
  return gemm_fwd_impl(h, gate_out, up_out, x, w_gate, w_up, nullptr, nullptr, nullptr, m, n, k, 0, gm, dm, status,
                       device, stream);
}

int swiglu_b200_geglu_gemm_fwd(void* h, void* gate_out, void* up_out, const void* x, const void* w_gate,
                               const void* w_up, int64_t m, int64_t n, int64_t k, int approximate_tanh, void* status,
                               int device, void* stream) {
  return gemm_fwd_impl(h, gate_out, up_out, x, w_gate, w_up, nullptr, nullptr, nullptr, m, n, k, 0, 1.0f, 1.0f, status,
                       device, stream, approximate_tanh ? ACT_GELU_TANH : ACT_GELU_ERF);
}

namespace {

int lora_gemm_checked(void* h, void* e_out, void* g_out, const void* x, const void* w_gate, const void* w_up,
                      const void* xa_scaled, const void* b_gate, const void* b_up, int64_t m, int64_t n, int64_t k,
                      int64_t r, float gm, float dm, void* status, int device, void* stream, int act) {
  if (r < 0) return SWIGLU_B200_ERR_SHAPE;
  if (r == 0)
    return gemm_fwd_impl(h, e_out, g_out, x, w_gate, w_up, nullptr, nullptr, nullptr, m, n, k, 0, gm, dm, status,
                         device, stream, act);
  if (r > 64 || r % 8 != 0) return SWIGLU_B200_ERR_SHAPE;
  if (m > 0 && n > 0 && (!xa_scaled || !b_gate || !b_up)) return SWIGLU_B200_ERR_NULL;
  if (((uintptr_t)xa_scaled | (uintptr_t)b_gate | (uintptr_t)b_up) % 16) return SWIGLU_B200_ERR_ALIGN;
  return gemm_fwd_impl(h, e_out, g_out, x, w_gate, w_up, xa_scaled, b_gate, b_up, m, n, k, (int)r, gm, dm, status,
                       device, stream, act);
}

}  // namespace

int swiglu_b200_lora_gemm_fwd(void* h, void* e_out, void* g_out, const void* x, const void* w_gate, const void* w_up,
                              const void* xa_scaled, const void* b_gate, const void* b_up, int64_t m, int64_t n,
                              int64_t k, int64_t r, float gm, float dm, void* status, int device, void* stream) {
  return lora_gemm_checked(h, e_out, g_out, x, w_gate, w_up, xa_scaled, b_gate, b_up, m, n, k, r, gm, dm, status, device,
                           stream, ACT_SILU);
}

int swiglu_b200_lora_geglu_gemm_fwd(void* h, void* e_out, void* g_out, const void* x, const void* w_gate,
                                    const void* w_up, const void* xa_scaled, const void* b_gate, const void* b_up,
                                    int64_t m, int64_t n, int64_t k, int64_t r, int approximate_tanh, void* status,
                                    int device, void* stream) {
  return lora_gemm_checked(h, e_out, g_out, x, w_gate, w_up, xa_scaled, b_gate, b_up, m, n, k, r, 1.0f, 1.0f, status,
                           device, stream, approximate_tanh ? ACT_GELU_TANH : ACT_GELU_ERF);
}


// ------------------------------------------------------------------------------------------
// Entry point for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need the fused GEMM: a
// serving process whose memory planner (or another framework's caching allocator) already owns
// all of the device memory, so that a raw allocation fails; a latency-critical loop in which
// cudaMalloc/cudaFree are banned because they synchronise the whole device; a plug-in that is
// handed its tensors and nothing else.  swiglu_b200_gemm_fwd asks such a caller for one device
// word (the kernel's status word); this variant keeps that word in a small array that lives in
// the library image itself, so the caller passes inputs and outputs only.
//
// The array below is the device-side object; in host code its NAME is only a handle, not a
// device address, so it is translated once per device with cudaGetSymbolAddress while that
// device is current, and the translated pointer is what the kernel receives.
constexpr size_t kNoAllocScratchBytes = 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

namespace {

// Device address of g_noalloc_scratch on the CURRENT device (looked up once per device).
int noalloc_scratch(void** out) {
  static std::mutex mu;
  static void* cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(mu);
  if (dev < 64 && cache[dev]) {
    *out = cache[dev];
    return SWIGLU_B200_OK;
  }
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || ptr == nullptr) return SWIGLU_B200_ERR_DEVICE;
  if (dev < 64) cache[dev] = ptr;
  *out = ptr;
  return SWIGLU_B200_OK;
}

}  // namespace

int swiglu_b200_gemm_fwd_noalloc(void* h, const void* x, const void* w_gate, const void* w_up, int64_t m, int64_t n,
                                 int64_t k, float gm, float dm, int* status_host, int device, void* stream) {
  // Scratch the kernel needs for this problem: one status word, whatever m, n and k are.  The
  // check is written against the array size so that it keeps guarding if either ever changes.
  const size_t scratch_needed = sizeof(int);
  if (scratch_needed > kNoAllocScratchBytes) return SWIGLU_B200_ERR_WORKSPACE;

  int prev = -1;
  bool switched = false;
  if (device >= 0) {
    if (cudaGetDevice(&prev) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
    if (prev != device) {
      if (cudaSetDevice(device) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
      switched = true;
    }
  }
  void* status_dev = nullptr;
  int rc = noalloc_scratch(&status_dev);  // with the target device current
  if (rc == SWIGLU_B200_OK) {
    // The existing entry point zeroes the status word on the stream before the kernel starts
    // (the array still holds whatever the previous call left) and allocates nothing itself.
    rc = swiglu_b200_gemm_fwd(h, nullptr, nullptr, x, w_gate, w_up, m, n, k, gm, dm, status_dev, -1, stream);
    if (rc == SWIGLU_B200_OK && status_host != nullptr) {
      if (m > 0 && n > 0) {
        if (cudaMemcpyAsync(status_host, status_dev, sizeof(int), cudaMemcpyDeviceToHost,
                            static_cast<cudaStream_t>(stream)) != cudaSuccess)
          rc = SWIGLU_B200_ERR_COPY;
      } else {
        *status_host = 0;  // empty problem: nothing was launched, so nothing can have failed
      }
    }
  }
  if (switched) cudaSetDevice(prev);
  return rc;
}

}  // extern "C"
