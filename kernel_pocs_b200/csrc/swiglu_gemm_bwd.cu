// Backward GEMMs of the fused gate/up projection, on the tcgen05 tensor cores:
//
//     dX  [M, K] = dgate [M, N] . Wg [N, K]  +  dup [M, N] . Wu [N, K]
//     dWg [N, K] = dgate^T . X [M, K]            dWu [N, K] = dup^T . X [M, K]
//
// dgate/dup come from the SwiGLU backward kernel (swiglu_b200_bwd) applied to the pre-activations the
// forward kernel saved.  The reference computes these with cuBLAS through autograd of
// down_proj(swiglu(gate_proj(x), up_proj(x))) (forge/forge/patching/kernels/basic.py:97-102).
//
// Both products run on the CTA-pair scheme of the forward kernel (cluster of 2, cta_group::2 MMA with
// M = 256, N = 256, K = 16, persistent over tiles, a ring of operand stages, accumulators in TMEM; pair
// tiles of 256 or 512 output columns, see Tile below), with one new ingredient: operands whose contiguous dimension is NOT the contraction dimension.  Wg/Wu in dX
// (contraction over n, contiguous along k) and all three operands of dW (contraction over m) are such
// "MN-major" operands; they are loaded as 64-element x 64-row boxes and described to the MMA with the
// MN-major shared-memory descriptor, so no transposed copy of any matrix is ever made.
//
//   dX : pair tile 256 (m) x 256 or 512 (k).  A = dgate rows then dup rows (K-major, 128 rows per CTA),
//        B = Wg then Wu (MN-major, each CTA loads 128 of the 256 output columns); the contraction runs
//        over n for the gate pair and then over n again for the up pair into the same accumulator.
//   dW : pair tile {dWg, dWu} x 128 (n) x 256 or 512 (k).  CTA 0 of the pair accumulates dWg, CTA 1 dWu: the
//        "M = 256" of the MMA is 128 columns of dgate stacked on the same 128 columns of dup (both
//        MN-major), B = X (MN-major, each CTA loads 128 of the 256 output columns); contraction over m.
// Every mbarrier wait is bounded; a wait that gives up records its code in the status word.
#include "swiglu_b200.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "tcgen05_common.cuh"

#ifndef SWIGLU_GEMM_BWD_WIDE_COST
#define SWIGLU_GEMM_BWD_WIDE_COST 0.91
#endif

namespace {

using namespace swiglu_b200::tc;

constexpr int BK = 64;                        // contraction elements per stage
constexpr int UMMA_K = 16;
constexpr int A_BYTES = 128 * BK * 2;         // 16 KiB: 128 rows (or columns) x 64 contraction elements
constexpr int B_BYTES = 128 * BK * 2;         // 16 KiB: 64 contraction rows x 128 output columns
constexpr int CHUNK_BYTES = 64 * BK * 2;      // 8 KiB: one 64-column chunk of an MN-major tile
constexpr int TMEM_COLS = 512;                // all of it: two accumulators of 256 fp32 columns, or one of 512
constexpr int EPI_PARTS = 2;                  // epilogue warps per TMEM lane quarter; they split a tile's columns
constexpr int THREADS = 64 + 128 * EPI_PARTS;

// NT = output columns of a pair tile.  256: one MMA of N = 256 per 16 contraction elements, two accumulator
// buffers, so a tile's epilogue overlaps the next tile's MMAs.  512: two such MMAs share the A operand, which
// cuts the operand bytes per flop by a quarter (A 16 KiB + B 32 KiB per CTA and K block instead of 2 x
// (16 + 16)); the single 512-column accumulator leaves the epilogue exposed, a percent or two of a tile.
template <int NT>
struct Tile {
  static_assert(NT == 256 || NT == 512, "one or two N = 256 MMAs per step");
  static constexpr int HALVES = NT / 256;
  static constexpr int STAGE_BYTES = A_BYTES + HALVES * B_BYTES;
  static constexpr int STAGES = NT == 256 ? 6 : 4;
  static constexpr int ACC_BUFS = 512 / NT;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
  static_assert(SMEM_BYTES <= 227 * 1024, "exceeds the shared memory of an SM");
};
constexpr int MAX_STAGES = 6;

enum Mode : int { MODE_DX = 0, MODE_DW = 1 };

// kind::f16, D fp32, A and B bf16, M = 256, N = 256; bit 15 / 16 select an MN-major A / B.
__host__ __device__ constexpr uint32_t idesc(bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((256u >> 3) << 17) | ((256u >> 4) << 24);
}

struct BwdParams {
  __nv_bfloat16* out0;   // dX, or dWg
  __nv_bfloat16* out1;   // unused, or dWu
  int* status;
  long long m, n, k;     // problem sizes of the FORWARD: x [m, k], w [n, k], dgate/dup [m, n]
};

// Tiles in bands of 8 row-tiles so that the operands in flight stay in L2.
//
// Tail split (512-column tiles only): when the tiles left over after the last full wave of the resident pairs
// number at most half the pairs, each of them is handed out as two 256-column halves, so that the last wave
// costs one narrow tile instead of one wide tile on a few pairs while the others idle.  `split_from` is the
// index of the first such tile (= the number of wide tiles), `total` counts work items.
struct Walk {
  long long tiles_r, tiles_c, total, split_from;
  int col_tile;
  __device__ __forceinline__ Walk(long long rows, long long row_tile, long long cols, int col_tile_, long long pairs)
      : tiles_r((rows + row_tile - 1) / row_tile), tiles_c((cols + col_tile_ - 1) / col_tile_), col_tile(col_tile_) {
    const long long tiles = tiles_r * tiles_c;
    const long long rest = tiles % pairs;
    const bool split = col_tile_ == 512 && rest > 0 && 2 * rest <= pairs && tiles > pairs;
    split_from = split ? tiles - rest : tiles;
    total = split ? tiles + rest : tiles;
  }
  // item t -> row tile, first output column, number of 256-column MMAs
  __device__ __forceinline__ void at(long long t, long long& tr, int& col, int& halves) const {
    long long tile = t;
    int half = 0;
    halves = col_tile / 256;
    if (t >= split_from) {
      tile = split_from + ((t - split_from) >> 1);
      half = (int)((t - split_from) & 1);
      halves = 1;
    }
    const long long per_band = 8 * tiles_c;
    const long long band = tile / per_band;
    const long long r = tile - band * per_band;
    const long long in_band = (tiles_r - band * 8) < 8 ? (tiles_r - band * 8) : 8;
    const long long tc = r / in_band;
    tr = band * 8 + (r - tc * in_band);
    col = (int)(tc * col_tile) + half * 256;
  }
};

// MODE_DX: maps = {dgate (K-major boxes of 128 rows), dup (same), Wg (MN boxes), Wu (MN boxes)}
// MODE_DW: maps = {dgate (MN boxes), dup (MN boxes), X (MN boxes), unused}
template <int MODE, int NT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
swiglu_gemm_bwd_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                       const __grid_constant__ CUtensorMap map2, const __grid_constant__ CUtensorMap map3,
                       const BwdParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int STAGES = Tile<NT>::STAGES, STAGE_BYTES = Tile<NT>::STAGE_BYTES, ACC_BUFS = Tile<NT>::ACC_BUFS,
                HALVES = Tile<NT>::HALVES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);  // used in the leader only
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* acc_full = empty + MAX_STAGES;
  uint64_t* acc_empty = acc_full + 2;                                         // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cta_rank();
  const long long pair_id = blockIdx.x >> 1;
  const long long n_pairs = gridDim.x >> 1;

  // output rows per pair tile: 256 rows of dX, or 128 rows of each of dWg and dWu
  const long long out_rows = MODE == MODE_DX ? p.m : p.n;
  const Walk walk(out_rows, MODE == MODE_DX ? 256 : 128, p.k, NT, n_pairs);
  // K blocks of one tile: dX contracts over n twice (gate pair, then up pair), dW over m once
  const int blocks_per_pass = (int)(((MODE == MODE_DX ? p.n : p.m) + BK - 1) / BK);
  const int k_blocks = MODE == MODE_DX ? 2 * blocks_per_pass : blocks_per_pass;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 2);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < ACC_BUFS; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8 * EPI_PARTS);  // every epilogue warp of both CTAs
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
  cluster_sync();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      long long it = 0;
      bool ok = true;
      for (long long t = pair_id; t < walk.total && ok; t += n_pairs) {
        long long tr;
        int col, halves;
        walk.at(t, tr, col, halves);
        const int col0 = col + (int)rank * 128;  // this CTA's 128 output columns of B (first MMA)
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          if (it >= STAGES) {
            ok = wait<false>(&empty[s], (uint32_t)((it / STAGES - 1) & 1), p.status, 100 + s);
            if (!ok) break;
          }
          const uint32_t leader_full = map_to_rank(smem_u32(&full[s]), 0);
          remote_expect_tx(leader_full, (uint32_t)(A_BYTES + halves * B_BYTES));
          unsigned char* a_dst = smem + s * STAGE_BYTES;
          unsigned char* b_dst = a_dst + A_BYTES;
          if (MODE == MODE_DX) {
            const bool up_pass = kb >= blocks_per_pass;
            const int c0 = (up_pass ? kb - blocks_per_pass : kb) * BK;  // contraction offset (n)
            // A: 128 rows of dgate / dup, 64 n; one K-major box
            tma_load_2d_pair(a_dst, up_pass ? &map1 : &map0, c0, (int)(tr * 256) + (int)rank * 128, leader_full);
            // B: 64 n-rows x 128 k-columns of Wg / Wu per MMA; two MN-major boxes each
            const CUtensorMap* w = up_pass ? &map3 : &map2;
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
              if (h < halves) {
                tma_load_2d_pair(b_dst + h * B_BYTES, w, col0 + h * 256, c0, leader_full);
                tma_load_2d_pair(b_dst + h * B_BYTES + CHUNK_BYTES, w, col0 + h * 256 + 64, c0, leader_full);
              }
            }
          } else {
            const int c0 = kb * BK;  // contraction offset (m)
            // A: 64 m-rows x 128 n-columns of dgate (CTA 0) or dup (CTA 1); two MN-major boxes
            const CUtensorMap* g = rank == 0 ? &map0 : &map1;
            const int n0 = (int)(tr * 128);
            tma_load_2d_pair(a_dst, g, n0, c0, leader_full);
            tma_load_2d_pair(a_dst + CHUNK_BYTES, g, n0 + 64, c0, leader_full);
            // B: 64 m-rows x 128 k-columns of X per MMA; two MN-major boxes each
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
              if (h < halves) {
                tma_load_2d_pair(b_dst + h * B_BYTES, &map2, col0 + h * 256, c0, leader_full);
                tma_load_2d_pair(b_dst + h * B_BYTES + CHUNK_BYTES, &map2, col0 + h * 256 + 64, c0, leader_full);
              }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t kIdesc = idesc(MODE == MODE_DW, true);
      long long it = 0, i = 0;
      bool ok = true;
      for (long long t = pair_id; t < walk.total && ok; t += n_pairs, ++i) {
        long long tr_unused;
        int col_unused, halves;
        walk.at(t, tr_unused, col_unused, halves);
        const int b = (int)(i % ACC_BUFS);
        if (i >= ACC_BUFS) {
          ok = wait<true>(&acc_empty[b], (uint32_t)((i / ACC_BUFS - 1) & 1), p.status, 400 + b);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t tmem_d = tmem_base + (uint32_t)b * 256u;  // NT = 512: b is 0, the halves at +0 and +256
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = (int)(it % STAGES);
          ok = wait<false>(&full[s], (uint32_t)((it / STAGES) & 1), p.status, 200 + s);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t a_desc = MODE == MODE_DX ? umma_desc(a_addr) : umma_desc_mn(a_addr, CHUNK_BYTES);
          constexpr int A_STEP = MODE == MODE_DX ? 2 : 128;  // descriptor advance per 16 contraction elements
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
              if (h < halves) {
                const uint64_t b_desc = umma_desc_mn(a_addr + A_BYTES + h * B_BYTES, CHUNK_BYTES);
                umma_pair(tmem_d + (uint32_t)h * 256u, a_desc + A_STEP * kk, b_desc + 128 * kk, kIdesc,
                          (kb | kk) != 0);
              }
            }
          }
          commit_both(&empty[s]);
        }
        if (ok) commit_both(&acc_full[b]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;
    long long i = 0;
    bool ok = true;
    for (long long t = pair_id; t < walk.total && ok; t += n_pairs, ++i) {
      long long tr;
      int col_base, halves;
      walk.at(t, tr, col_base, halves);
      const int b = (int)(i % ACC_BUFS);
      ok = wait<false, 200>(&acc_full[b], (uint32_t)((i / ACC_BUFS) & 1), p.status, 300 + b);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // dX: CTA r owns rows tr*256 + r*128 ..; dW: CTA 0 writes dWg rows tr*128 .., CTA 1 the same rows of dWu
      const long long row = MODE == MODE_DX ? tr * 256 + (long long)rank * 128 + quarter * 32 + lane
                                            : tr * 128 + quarter * 32 + lane;
      __nv_bfloat16* out = (MODE == MODE_DW && rank == 1) ? p.out1 : p.out0;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)b * 256u;
      // 64 columns per wait: the loads' latency, not their count, is what an epilogue thread spends its time on,
      // and with a single 512-column accumulator that time is not hidden behind the next tile's MMAs
#pragma unroll 1
      for (int c = part * 64; c < halves * 256; c += 64 * EPI_PARTS) {
        uint32_t v[64];
        tmem_ld32(t_row + c, v);
        tmem_ld32(t_row + c + 32, v + 32);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < out_rows) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (col_base + c + 16 * q < p.k) {  // k is a multiple of 16: groups of 16 columns are all in or all out
              uint32_t o[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                __nv_bfloat162 x = __floats2bfloat162_rn(__uint_as_float(v[16 * q + 2 * j]),
                                                         __uint_as_float(v[16 * q + 2 * j + 1]));
                o[j] = *reinterpret_cast<uint32_t*>(&x);
              }
              uint4* dst = reinterpret_cast<uint4*>(out + row * p.k + col_base + c + 16 * q);
              dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
              dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) remote_arrive(map_to_rank(smem_u32(&acc_empty[b]), 0));
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  settle_before_teardown(p.status);
  cluster_sync();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

std::atomic<uint64_t> g_bwd_launches{0};

template <int MODE, int NT>
int resident_clusters(int dev, int* out) {
  constexpr int SMEM_BYTES = Tile<NT>::SMEM_BYTES;
  static std::atomic<int> cache[64];
  if (dev < 64) {
    const int c = cache[dev].load(std::memory_order_acquire);
    if (c > 0) {
      *out = c;
      return SWIGLU_B200_OK;
    }
  }
  auto kernel = swiglu_gemm_bwd_kernel<MODE, NT>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
    return SWIGLU_B200_ERR_DEVICE;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 148, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n < 1) return SWIGLU_B200_ERR_DEVICE;
  if (dev < 64) cache[dev].store(n, std::memory_order_release);
  *out = n;
  return SWIGLU_B200_OK;
}


template <int MODE, int NT>
int launch_tile(int dev, long long row_tiles, long long k, const CUtensorMap& m0, const CUtensorMap& m1,
                const CUtensorMap& m2, const CUtensorMap& m3, const BwdParams& p, cudaStream_t st) {
  int clusters = 0;
  int rc = resident_clusters<MODE, NT>(dev, &clusters);
  if (rc != SWIGLU_B200_OK) return rc;
  const long long tiles = row_tiles * ((k + NT - 1) / NT);
  const long long use = tiles < clusters ? tiles : clusters;
  swiglu_gemm_bwd_kernel<MODE, NT><<<(unsigned)(2 * use), THREADS, Tile<NT>::SMEM_BYTES, st>>>(m0, m1, m2, m3, p);
  if (cudaGetLastError() != cudaSuccess) return SWIGLU_B200_ERR_LAUNCH;
  g_bwd_launches.fetch_add(1, std::memory_order_relaxed);
  return SWIGLU_B200_OK;
}

// Tile width: 512 columns where its waves over the resident pairs cost less than those of 256 columns.  A
// 512-column tile does the work of two 256-column tiles in kWide512Cost of their time (measured: fewer
// operand bytes per flop).  SWIGLU_B200_GEMM_BWD_TILE=256|512 in the environment forces one, for experiments.
constexpr double kWide512Cost = SWIGLU_GEMM_BWD_WIDE_COST;

template <int MODE>
int launch_mode(int dev, long long row_tiles, long long k, const CUtensorMap& m0, const CUtensorMap& m1,
                const CUtensorMap& m2, const CUtensorMap& m3, const BwdParams& p, cudaStream_t st) {
  int clusters = 0;
  int rc = resident_clusters<MODE, 256>(dev, &clusters);
  if (rc != SWIGLU_B200_OK) return rc;
  const long long t256 = row_tiles * ((k + 255) / 256), t512 = row_tiles * ((k + 511) / 512);
  const double cost256 = (double)((t256 + clusters - 1) / clusters);
  // the kernel hands a short last wave out as 256-column halves (see Walk)
  const long long rest = t512 % clusters;
  const double tail = rest == 0 ? 0.0 : (2 * rest <= clusters && t512 > clusters) ? 1.0 : 2.0 * kWide512Cost;
  const double cost512 = (double)(t512 / clusters) * 2.0 * kWide512Cost + tail;
  bool wide = cost512 < cost256;
  if (const char* force = std::getenv("SWIGLU_B200_GEMM_BWD_TILE")) {
    if (std::strcmp(force, "256") == 0) wide = false;
    if (std::strcmp(force, "512") == 0) wide = true;
  }
  return wide ? launch_tile<MODE, 512>(dev, row_tiles, k, m0, m1, m2, m3, p, st)
              : launch_tile<MODE, 256>(dev, row_tiles, k, m0, m1, m2, m3, p, st);
}

}  // namespace

extern "C" {

uint64_t swiglu_b200_gemm_bwd_launch_count(void) { return g_bwd_launches.load(std::memory_order_relaxed); }

int swiglu_b200_gemm_bwd(void* dx, void* dw_gate, void* dw_up, const void* dgate, const void* dup, const void* x,
                         const void* w_gate, const void* w_up, int64_t m, int64_t n, int64_t k, void* status,
                         int device, void* stream) {
  if (m < 0 || n < 0 || k < 0) return SWIGLU_B200_ERR_SHAPE;
  if (m == 0 || n == 0 || k == 0) return SWIGLU_B200_OK;
  // 16-byte global strides for every tiled copy and 32-byte output groups
  if (k % 16 != 0 || n % 8 != 0) return SWIGLU_B200_ERR_SHAPE;
  if (m > 0x7fffff00LL || n > 0x7fffff00LL || k > 0x7fffff00LL) return SWIGLU_B200_ERR_SHAPE;
  if ((dw_gate == nullptr) != (dw_up == nullptr)) return SWIGLU_B200_ERR_NULL;
  if (!dgate || !dup || !status) return SWIGLU_B200_ERR_NULL;
  if (dx && (!w_gate || !w_up)) return SWIGLU_B200_ERR_NULL;
  if (dw_gate && !x) return SWIGLU_B200_ERR_NULL;
  if (((uintptr_t)dx | (uintptr_t)dw_gate | (uintptr_t)dw_up | (uintptr_t)dgate | (uintptr_t)dup | (uintptr_t)x |
       (uintptr_t)w_gate | (uintptr_t)w_up) % 16)
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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(status, 0, sizeof(int), st) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;

  if (dx) {
    CUtensorMap mg, mu, mwg, mwu;
    // dgate/dup [m, n]: K-major boxes of 128 rows x 64 n.  Wg/Wu [n, k]: boxes of 64 n-rows x 64 k.
    if (!make_map(&mg, dgate, m, n, 128) || !make_map(&mu, dup, m, n, 128) || !make_map(&mwg, w_gate, n, k, 64) ||
        !make_map(&mwu, w_up, n, k, 64))
      return SWIGLU_B200_ERR_DEVICE;
    BwdParams p{static_cast<__nv_bfloat16*>(dx), nullptr, static_cast<int*>(status), m, n, k};
    int rc = launch_mode<MODE_DX>(dev, (m + 255) / 256, k, mg, mu, mwg, mwu, p, st);
    if (rc != SWIGLU_B200_OK) return rc;
  }
  if (dw_gate) {
    CUtensorMap mg, mu, mx;
    // all three as boxes of 64 m-rows x 64 contiguous elements
    if (!make_map(&mg, dgate, m, n, 64) || !make_map(&mu, dup, m, n, 64) || !make_map(&mx, x, m, k, 64))
      return SWIGLU_B200_ERR_DEVICE;
    BwdParams p{static_cast<__nv_bfloat16*>(dw_gate), static_cast<__nv_bfloat16*>(dw_up), static_cast<int*>(status),
                m, n, k};
    int rc = launch_mode<MODE_DW>(dev, (n + 127) / 128, k, mg, mu, mx, mx, p, st);
    if (rc != SWIGLU_B200_OK) return rc;
  }
  return SWIGLU_B200_OK;
}

}  // extern "C"
