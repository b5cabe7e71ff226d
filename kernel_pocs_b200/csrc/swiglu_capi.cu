// C ABI of the SwiGLU library: argument checking, access-width selection and launch.
// Declarations and the contract of every entry point are in include/swiglu_b200.h.
#include "swiglu_b200.h"

#include <atomic>

#include "swiglu_kernels.cuh"

namespace {

using namespace swiglu_b200;

// Launch shape of the streaming kernels, chosen from a sweep on B200 over threads {128,256,512},
// unroll {1,2,4,8}, 16- and 32-byte accesses, cache hints and grid sizes (bf16 [32768,14336]):
//  * one CTA per tile beats a persistent grid of (SMs x resident CTAs) walking tiles with a fixed
//    stride by about 20 % (7.07 vs 5.6 TB/s forward): with a fixed stride every CTA gets the same
//    share and the slowest SM sets the finish time, while the hardware block scheduler hands the
//    next tile to whichever SM frees up first.  The grid-stride loop stays in the kernel and takes
//    over only when the tile count exceeds the grid limit.
//  * 512 threads x 4 vectors (forward) / x 2 vectors (backward) of 16 bytes were the fastest
//    shapes; 32-byte accesses and the cache-hint variants were within +-0.5 % of them.
#ifndef SWIGLU_THREADS
#define SWIGLU_THREADS 512
#endif
#ifndef SWIGLU_FWD_UNROLL
#define SWIGLU_FWD_UNROLL 4
#endif
#ifndef SWIGLU_BWD_UNROLL
#define SWIGLU_BWD_UNROLL 2
#endif
#ifndef SWIGLU_SKEW_UNROLL
#define SWIGLU_SKEW_UNROLL 3  // skewed-load kernels keep words of a second granule per vector in registers
#endif
#ifndef SWIGLU_SKEW1_BWD_UNROLL
#define SWIGLU_SKEW1_BWD_UNROLL 3
#endif
#ifndef SWIGLU_LD_RO
#define SWIGLU_LD_RO LD_NC_NOALLOC  // backward: inputs that this launch never writes
#endif
#ifndef SWIGLU_LD_RO_FWD
#define SWIGLU_LD_RO_FWD LD_PLAIN   // forward: plain loads measured 1.6 % faster than the no-allocate hint
#endif                              // (bf16 [32768, 14336]: 7.15 against 7.04 TB/s; fp32 alike)
// Ragged-row kernels: most warps of one CTA, and the resident CTAs per SM the register budget is set for.  Measured
// on B200 (bf16, packed gate|up, half-widths 5503 and 11009): the forward is latency-bound and gains from 1536
// resident threads at 40 registers (6.68 TB/s against 5.6 with 1024 threads at 64 registers); the backward, three
// windows wide, does best with nine CTAs at 56 registers (6.38 / 5.81 TB/s; 6.20 / 5.63 with eight at 64, 6.01 / 5.34
// with seven, 5.3 / 5.2 at 40 registers) -- small CTAs in both.
#ifndef SWIGLU_RAGGED_FWD_WARPS
#define SWIGLU_RAGGED_FWD_WARPS 4
#endif
#ifndef SWIGLU_RAGGED_FWD_CTAS
#define SWIGLU_RAGGED_FWD_CTAS 12
#endif
#ifndef SWIGLU_RAGGED_BWD_WARPS
#define SWIGLU_RAGGED_BWD_WARPS 4
#endif
#ifndef SWIGLU_RAGGED_BWD_CTAS
#define SWIGLU_RAGGED_BWD_CTAS 9
#endif
#ifndef SWIGLU_LD_RAGGED
#define SWIGLU_LD_RAGGED LD_PLAIN  // ragged-row kernels: neighbouring lanes read overlapping lines, so let L1 keep them
#endif
#ifndef SWIGLU_LD_ALIASED
#define SWIGLU_LD_ALIASED LD_PLAIN  // gate/up when dgate/dup overwrite them
#endif
#ifndef SWIGLU_ST
#define SWIGLU_ST ST_CS
#endif

std::atomic<uint64_t> g_launches{0};
thread_local int t_last_cuda_error = 0;

int fail_cuda(int code, cudaError_t e) {
  t_last_cuda_error = (int)e;
  return code;
}

struct DeviceScope {
  // Makes `device` current for the duration of a call (no-op for -1 or when it already is).
  int prev = -1;
  bool switched = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceScope(int device) {
    if (device < 0) return;
    err = cudaGetDevice(&prev);
    if (err != cudaSuccess) return;
    if (prev != device) {
      err = cudaSetDevice(device);
      switched = (err == cudaSuccess);
    }
  }
  ~DeviceScope() {
    if (switched) cudaSetDevice(prev);
  }
};

constexpr long long kMaxGrid = 0x7fffffffLL;  // gridDim.x limit

unsigned grid_for(long long n_vec, int threads, int unroll) {
  const long long tile = (long long)threads * unroll;
  long long tiles = (n_vec + tile - 1) / tile;
  if (tiles < 1) tiles = 1;  // an edge-only launch still needs one CTA
  return (unsigned)(tiles < kMaxGrid ? tiles : kMaxGrid);
}

inline int elem_size(int dtype) { return dtype == SWIGLU_B200_F32 ? 4 : 2; }

// Largest power of two <= limit that divides v (v == 0 divides everything).
inline int pow2_divisor(unsigned long long v, int limit) {
  int b = limit;
  while (b > 1 && (v % (unsigned long long)b) != 0) b >>= 1;
  return b;
}

struct Plan {
  bool ragged;  // per-row alignment: 16-byte accesses with skewed loads and a skewed second store (see
                // swiglu_*_ragged_kernel); chosen when neither the flat nor the pitched 16-byte path applies
  RaggedShape rshape;
  bool rows;   // 2-D addressing
  bool shift;  // flat, 16-byte body, some input skewed against the outputs (see ld_skewed)
  bool one_word;  // ... and every skew is within 4 bytes of a boundary: one word of a neighbouring granule
                  // completes a vector
  int bytes;   // access width of the body
  Shape shape;
  long long skip;  // bytes by which every base pointer is advanced (flat head)
  int skew[3];     // per input, in the order the caller listed them
};

// Chooses addressing and access width.  `out` are the addresses written, `in` the addresses only
// read (an in-place backward lists gate/up under `out`, since dgate/dup are the same addresses);
// pitch[k] (elements) are the row strides in play.
Plan make_plan(const unsigned long long* out, int n_out, const unsigned long long* in, int n_in,
               const long long* pitch, int n_pitch, long long rows, long long cols, int es) {
  constexpr int kWide = 16;
  Plan p{};
  bool flat = true;
  if (rows != 1)
    for (int k = 0; k < n_pitch; ++k) flat = flat && (pitch[k] == cols);
  p.rows = !flat;
  const long long n = rows * cols;
  int common = kWide;  // widest power of two dividing every address
  for (int k = 0; k < n_out; ++k) common = pow2_divisor(out[k], common);
  for (int k = 0; k < n_in; ++k) common = pow2_divisor(in[k], common);
  if (flat) {
    bool out_congruent = true;
    for (int k = 1; k < n_out; ++k) out_congruent = out_congruent && ((out[k] % kWide) == (out[0] % kWide));
    if (out_congruent) {
      // Peel a scalar head so that the outputs' body starts on a 16-byte boundary; inputs that do
      // not land on one as well are read through the skewed-load path.
      long long head = (long long)((kWide - out[0] % kWide) % kWide) / es;
      if (head > n) head = n;
      const int epv = kWide / es;
      p.bytes = kWide;
      p.shape.n_vec = (n - head) / epv;
      p.shape.head = (int)head;
      p.shape.edge = (int)(n - p.shape.n_vec * epv);
      p.skip = head * es;
      p.one_word = true;
      for (int k = 0; k < n_in; ++k) {
        p.skew[k] = (int)((in[k] + (unsigned long long)p.skip) % kWide);
        p.shift = p.shift || p.skew[k] != 0;
        p.one_word = p.one_word && (p.skew[k] <= 4 || p.skew[k] >= 12);
      }
      if (p.shift && n_out == 1) {
        // Forward with inputs skewed against the output: one long ragged row.  Its window loads beat the shuffled
        // loads of the flat kernel (width 11009, inputs 2 / 8 / 14 bytes off: 7.04 / 7.01 / 6.84 TB/s against
        // 6.71 / 6.41 / 6.26); the backward, three inputs wide, is faster with the shuffled loads (6.70 / 6.26 /
        // 6.13 against 6.16 / 6.06 / 5.93) and keeps them.
        p = Plan{};
        p.ragged = true;
        p.bytes = kWide;
        p.rshape.rows = 1;
        p.rshape.cols = n;
      }
    } else {
      // two outputs skewed against each other: one long ragged row
      p.ragged = true;
      p.bytes = kWide;
      p.rshape.rows = 1;
      p.rshape.cols = n;
    }
  } else {
    int b = common;
    b = pow2_divisor((unsigned long long)cols * es, b);
    for (int k = 0; k < n_pitch; ++k) b = pow2_divisor((unsigned long long)pitch[k] * es, b);
    if (b == kWide) {
      // every row of every tensor starts on a 16-byte boundary and is a whole number of vectors
      p.bytes = b;
      p.shape.vecs_per_row = cols * es / b;
      p.shape.n_vec = rows * p.shape.vecs_per_row;
      swiglu_b200::set_row_divisor(p.shape);
    } else {
      p.ragged = true;
      p.bytes = kWide;
      p.rshape.rows = rows;
      p.rshape.cols = cols;
    }
    p.skip = 0;
  }
  if (p.ragged) p.rshape.tasks_per_row = 0;  // set by the launcher
  return p;
}

// Ragged-row launches: a warp task is 32 frames of 32 bytes of one row; a CTA is up to `max_warps` consecutive
// tasks of one row, the row's tasks spread evenly over its CTAs so that no warp idles; grid.x walks the row,
// grid.y and grid.z the rows.
struct RaggedLaunch {
  dim3 grid;
  unsigned block;
};
template <class T>
RaggedLaunch ragged_launch(RaggedShape& s, long long max_warps) {
  const long long epv = 32 / (long long)sizeof(T);
  long long tasks = (s.cols / epv + 31) / 32;
  if (tasks < 1) tasks = 1;  // the row's scalar elements still need a task
  s.tasks_per_row = (int)tasks;
  const long long ctas = (tasks + max_warps - 1) / max_warps;
  const long long warps = (tasks + ctas - 1) / ctas;
  RaggedLaunch l;
  l.block = (unsigned)(32 * warps);
  // rows = y * z as evenly as the 65535 limit of grid.y allows: surplus CTAs (row >= rows) return at once but
  // still cost a launch slot each
  const long long z = (s.rows + 65534) / 65535;
  const long long y = (s.rows + z - 1) / z;
  l.grid = dim3((unsigned)ctas, (unsigned)y, (unsigned)z);
  return l;
}

// ------------------------------------------------------------------ forward dispatch

template <class T, int ACT, int BYTES, bool ROWS>
int launch_fwd(void* out, const void* gate, const void* up, const Shape& s, float gm, float dm, cudaStream_t st) {
  constexpr bool FAST = (sizeof(T) == 2);
  constexpr int UNROLL = SWIGLU_FWD_UNROLL;
  auto kernel =
      swiglu_fwd_kernel<T, BYTES, FAST, ROWS, SWIGLU_THREADS, UNROLL, SWIGLU_LD_RO_FWD, SWIGLU_ST, ACT>;
  const unsigned grid = grid_for(s.n_vec, SWIGLU_THREADS, UNROLL);
  kernel<<<grid, SWIGLU_THREADS, 0, st>>>(out, gate, up, s, gm, dm);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda(SWIGLU_B200_ERR_LAUNCH, err);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return SWIGLU_B200_OK;
}

template <class T, int ACT, bool ROWS>
int fwd_by_width(int bytes, void* out, const void* gate, const void* up, const Shape& s, float gm, float dm,
                 cudaStream_t st) {
  switch (bytes) {
    case 16: return launch_fwd<T, ACT, 16, ROWS>(out, gate, up, s, gm, dm, st);
    case 8: return launch_fwd<T, ACT, 8, ROWS>(out, gate, up, s, gm, dm, st);
    case 4: return launch_fwd<T, ACT, 4, ROWS>(out, gate, up, s, gm, dm, st);
    case 2:
      if constexpr (sizeof(T) == 2) return launch_fwd<T, ACT, 2, ROWS>(out, gate, up, s, gm, dm, st);
  }
  return SWIGLU_B200_ERR_ALIGN;
}

template <class T, int ACT>
int launch_fwd_ragged(void* out, const void* gate, const void* up, const RaggedShape& s, float gm, float dm,
                      cudaStream_t st) {
  constexpr bool FAST = (sizeof(T) == 2);
  auto kernel = swiglu_fwd_ragged_kernel<T, FAST, 32 * SWIGLU_RAGGED_FWD_WARPS, SWIGLU_RAGGED_FWD_CTAS, SWIGLU_LD_RAGGED,
                                         SWIGLU_ST, ACT>;
  RaggedShape rs = s;
  const RaggedLaunch l = ragged_launch<T>(rs, SWIGLU_RAGGED_FWD_WARPS);
  kernel<<<l.grid, l.block, 0, st>>>(out, gate, up, rs, gm, dm);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda(SWIGLU_B200_ERR_LAUNCH, err);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return SWIGLU_B200_OK;
}

template <class T, int ACT>
int fwd_typed(const Plan& p, void* out, const void* gate, const void* up, float gm, float dm, cudaStream_t st) {
  if (p.ragged) return launch_fwd_ragged<T, ACT>(out, gate, up, p.rshape, gm, dm, st);
  if (p.shift) return SWIGLU_B200_ERR_ALIGN;  // not planned for the forward: skewed inputs take the ragged-row kernel
  return p.rows ? fwd_by_width<T, ACT, true>(p.bytes, out, gate, up, p.shape, gm, dm, st)
                : fwd_by_width<T, ACT, false>(p.bytes, out, gate, up, p.shape, gm, dm, st);
}

// ------------------------------------------------------------------ backward dispatch

template <class T, int ACT, int BYTES, bool ROWS, bool INPLACE, int SHIFT = 0>
int launch_bwd(void* dgate, void* dup, const void* dout, const void* gate, const void* up, const Shape& s, float gm,
               float dm, cudaStream_t st) {
  constexpr bool FAST = (sizeof(T) == 2);
  constexpr int LD_IO = INPLACE ? SWIGLU_LD_ALIASED : SWIGLU_LD_RO;
  constexpr int UNROLL = SHIFT == 2 ? SWIGLU_SKEW_UNROLL : SHIFT == 1 ? SWIGLU_SKEW1_BWD_UNROLL : SWIGLU_BWD_UNROLL;
  auto kernel =
      swiglu_bwd_kernel<T, BYTES, FAST, ROWS, SWIGLU_THREADS, UNROLL, SWIGLU_LD_RO, LD_IO, SWIGLU_ST, SHIFT, ACT>;
  const unsigned grid = grid_for(s.n_vec, SWIGLU_THREADS, UNROLL);
  kernel<<<grid, SWIGLU_THREADS, 0, st>>>(dgate, dup, dout, gate, up, s, gm, dm);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda(SWIGLU_B200_ERR_LAUNCH, err);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return SWIGLU_B200_OK;
}

template <class T, int ACT, bool ROWS, bool INPLACE>
int bwd_by_width(int bytes, void* dgate, void* dup, const void* dout, const void* gate, const void* up,
                 const Shape& s, float gm, float dm, cudaStream_t st) {
  switch (bytes) {
    case 16: return launch_bwd<T, ACT, 16, ROWS, INPLACE>(dgate, dup, dout, gate, up, s, gm, dm, st);
    case 8: return launch_bwd<T, ACT, 8, ROWS, INPLACE>(dgate, dup, dout, gate, up, s, gm, dm, st);
    case 4: return launch_bwd<T, ACT, 4, ROWS, INPLACE>(dgate, dup, dout, gate, up, s, gm, dm, st);
    case 2:
      if constexpr (sizeof(T) == 2) return launch_bwd<T, ACT, 2, ROWS, INPLACE>(dgate, dup, dout, gate, up, s, gm, dm, st);
  }
  return SWIGLU_B200_ERR_ALIGN;
}

template <class T, int ACT, bool INPLACE>
int launch_bwd_ragged(void* dgate, void* dup, const void* dout, const void* gate, const void* up,
                      const RaggedShape& s, float gm, float dm, cudaStream_t st) {
  constexpr bool FAST = (sizeof(T) == 2);
  constexpr int LD_IO = INPLACE ? SWIGLU_LD_ALIASED : SWIGLU_LD_RAGGED;
  auto kernel = swiglu_bwd_ragged_kernel<T, FAST, 32 * SWIGLU_RAGGED_BWD_WARPS, SWIGLU_RAGGED_BWD_CTAS, SWIGLU_LD_RAGGED,
                                         LD_IO, SWIGLU_ST, ACT>;
  RaggedShape rs = s;
  const RaggedLaunch l = ragged_launch<T>(rs, SWIGLU_RAGGED_BWD_WARPS);
  kernel<<<l.grid, l.block, 0, st>>>(dgate, dup, dout, gate, up, rs, gm, dm);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda(SWIGLU_B200_ERR_LAUNCH, err);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return SWIGLU_B200_OK;
}

template <class T, int ACT>
int bwd_typed(const Plan& p, bool inplace, void* dgate, void* dup, const void* dout, const void* gate,
              const void* up, float gm, float dm, cudaStream_t st) {
  if (p.ragged)
    return inplace ? launch_bwd_ragged<T, ACT, true>(dgate, dup, dout, gate, up, p.rshape, gm, dm, st)
                   : launch_bwd_ragged<T, ACT, false>(dgate, dup, dout, gate, up, p.rshape, gm, dm, st);
  if (p.shift) {
    if (p.one_word)
      return inplace ? launch_bwd<T, ACT, 16, false, true, 1>(dgate, dup, dout, gate, up, p.shape, gm, dm, st)
                     : launch_bwd<T, ACT, 16, false, false, 1>(dgate, dup, dout, gate, up, p.shape, gm, dm, st);
    return inplace ? launch_bwd<T, ACT, 16, false, true, 2>(dgate, dup, dout, gate, up, p.shape, gm, dm, st)
                   : launch_bwd<T, ACT, 16, false, false, 2>(dgate, dup, dout, gate, up, p.shape, gm, dm, st);
  }
  if (p.rows) {
    return inplace ? bwd_by_width<T, ACT, true, true>(p.bytes, dgate, dup, dout, gate, up, p.shape, gm, dm, st)
                   : bwd_by_width<T, ACT, true, false>(p.bytes, dgate, dup, dout, gate, up, p.shape, gm, dm, st);
  }
  return inplace ? bwd_by_width<T, ACT, false, true>(p.bytes, dgate, dup, dout, gate, up, p.shape, gm, dm, st)
                 : bwd_by_width<T, ACT, false, false>(p.bytes, dgate, dup, dout, gate, up, p.shape, gm, dm, st);
}

// ------------------------------------------------------------------ backward with h recomputed

template <class T, int ACT, int BYTES, bool ALIASED>
int launch_recompute(void* h, void* dgate, void* dup, const void* dout, const void* gate, const void* up, long long n,
                     float gm, float dm, cudaStream_t st) {
  constexpr bool FAST = (sizeof(T) == 2);
  constexpr int LDM = ALIASED ? SWIGLU_LD_ALIASED : SWIGLU_LD_RO;
  constexpr int EPV = BYTES / (int)sizeof(T);
  const long long n_vec = n / EPV;
  auto kernel = swiglu_bwd_recompute_kernel<T, BYTES, FAST, SWIGLU_THREADS, SWIGLU_BWD_UNROLL, LDM, SWIGLU_ST, ACT>;
  const unsigned grid = grid_for(n_vec, SWIGLU_THREADS, SWIGLU_BWD_UNROLL);
  kernel<<<grid, SWIGLU_THREADS, 0, st>>>(h, dgate, dup, dout, gate, up, n_vec, (int)(n - n_vec * EPV), gm, dm);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail_cuda(SWIGLU_B200_ERR_LAUNCH, err);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return SWIGLU_B200_OK;
}

template <class T, int ACT>
int recompute_by_width(int bytes, bool aliased, void* h, void* dgate, void* dup, const void* dout, const void* gate,
                       const void* up, long long n, float gm, float dm, cudaStream_t st) {
#define SWIGLU_RECOMPUTE_CASE(B)                                                                          \
  return aliased ? launch_recompute<T, ACT, B, true>(h, dgate, dup, dout, gate, up, n, gm, dm, st)        \
                 : launch_recompute<T, ACT, B, false>(h, dgate, dup, dout, gate, up, n, gm, dm, st)
  switch (bytes) {
    case 16: SWIGLU_RECOMPUTE_CASE(16);
    case 8: SWIGLU_RECOMPUTE_CASE(8);
    case 4: SWIGLU_RECOMPUTE_CASE(4);
    case 2:
      if constexpr (sizeof(T) == 2) { SWIGLU_RECOMPUTE_CASE(2); }
  }
#undef SWIGLU_RECOMPUTE_CASE
  return SWIGLU_B200_ERR_ALIGN;
}

inline int plan_code(const Plan& p) {
  return p.bytes | (p.rows ? 1 << 8 : 0) | (p.shift ? 1 << 9 : 0) | (p.shift && p.one_word ? 1 << 10 : 0) |
         (p.ragged ? 1 << 11 : 0) | (p.shape.head << 16) | (p.shape.edge << 24);
}

inline unsigned long long addr_of(const void* p) { return (unsigned long long)(uintptr_t)p; }
inline const void* advance(const void* p, long long bytes) { return static_cast<const char*>(p) + bytes; }
inline void* advance(void* p, long long bytes) { return static_cast<char*>(p) + bytes; }

// Byte extent [lo, hi) touched by a rows x cols tensor with the given row stride.
struct Extent {
  unsigned long long lo, hi;
};
inline Extent extent(const void* p, long long rows, long long cols, long long stride, int es) {
  const unsigned long long lo = addr_of(p);
  return Extent{lo, lo + (unsigned long long)(((rows - 1) * stride + cols) * es)};
}
inline bool overlaps(const Extent& a, const Extent& b) { return a.lo < b.hi && b.lo < a.hi; }

}  // namespace

extern "C" {

int swiglu_b200_version(void) { return 1000; }

const char* swiglu_b200_strerror(int code) {
  switch (code) {
    case SWIGLU_B200_OK: return "success";
    case SWIGLU_B200_ERR_DTYPE: return "unsupported dtype code (expected 0=fp32, 1=fp16, 2=bf16)";
    case SWIGLU_B200_ERR_NULL: return "null pointer for a non-empty tensor";
    case SWIGLU_B200_ERR_SHAPE: return "negative size or row stride smaller than cols";
    case SWIGLU_B200_ERR_ALIGN: return "pointer not aligned to the element size";
    case SWIGLU_B200_ERR_ALIAS: return "output overlaps an input without aliasing it exactly";
    case SWIGLU_B200_ERR_DEVICE: return "CUDA device selection or attribute query failed";
    case SWIGLU_B200_ERR_LAUNCH: return "CUDA kernel launch failed";
    case SWIGLU_B200_ERR_COPY: return "CUDA host<->device copy failed";
    case SWIGLU_B200_ERR_WORKSPACE: return "device workspace too small for one chunk of token rows";
    default: return "unknown swiglu_b200 error code";
  }
}

int swiglu_b200_last_cuda_error(void) { return t_last_cuda_error; }

uint64_t swiglu_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"

namespace {

template <int ACT>
int fwd_entry(void* out, const void* gate, const void* up, int64_t rows, int64_t cols, int64_t in_row_stride,
              int64_t out_row_stride, int dtype, float gm, float dm, int device, void* stream) {
  if (dtype != SWIGLU_B200_F32 && dtype != SWIGLU_B200_F16 && dtype != SWIGLU_B200_BF16) return SWIGLU_B200_ERR_DTYPE;
  if (rows < 0 || cols < 0) return SWIGLU_B200_ERR_SHAPE;
  if (rows == 0 || cols == 0) return SWIGLU_B200_OK;
  if (in_row_stride < cols || out_row_stride < cols) return SWIGLU_B200_ERR_SHAPE;
  if (!out || !gate || !up) return SWIGLU_B200_ERR_NULL;
  const int es = elem_size(dtype);
  if (addr_of(out) % es || addr_of(gate) % es || addr_of(up) % es) return SWIGLU_B200_ERR_ALIGN;
  {
    const Extent eo = extent(out, rows, cols, out_row_stride, es);
    if (overlaps(eo, extent(gate, rows, cols, in_row_stride, es)) ||
        overlaps(eo, extent(up, rows, cols, in_row_stride, es)))
      return SWIGLU_B200_ERR_ALIAS;
  }

  DeviceScope scope(device);
  if (scope.err != cudaSuccess) return fail_cuda(SWIGLU_B200_ERR_DEVICE, scope.err);

  const unsigned long long outs[1] = {addr_of(out)};
  const unsigned long long ins[2] = {addr_of(gate), addr_of(up)};
  const long long pitch[2] = {in_row_stride, out_row_stride};
  Plan p = make_plan(outs, 1, ins, 2, pitch, 2, rows, cols, es);
  p.shape.skew_gate = p.skew[0];
  p.shape.skew_up = p.skew[1];
  p.shape.skew_dout = 0;
  p.shape.pitch_in = in_row_stride * es;
  p.shape.pitch_out = out_row_stride * es;
  p.shape.pitch_grad = 0;
  p.rshape.pitch_in = p.shape.pitch_in;
  p.rshape.pitch_out = p.shape.pitch_out;
  p.rshape.pitch_grad = 0;
  out = advance(out, p.skip);
  gate = advance(gate, p.skip);
  up = advance(up, p.skip);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SWIGLU_B200_F32: return fwd_typed<float, ACT>(p, out, gate, up, gm, dm, st);
    case SWIGLU_B200_F16: return fwd_typed<__half, ACT>(p, out, gate, up, gm, dm, st);
    default: return fwd_typed<__nv_bfloat16, ACT>(p, out, gate, up, gm, dm, st);
  }
}

template <int ACT>
int bwd_entry(void* dgate, void* dup, const void* dout, const void* gate, const void* up, int64_t rows, int64_t cols,
              int64_t in_row_stride, int64_t grad_row_stride, int64_t dout_row_stride, int dtype, float gm, float dm,
              int device, void* stream) {
  if (dtype != SWIGLU_B200_F32 && dtype != SWIGLU_B200_F16 && dtype != SWIGLU_B200_BF16) return SWIGLU_B200_ERR_DTYPE;
  if (rows < 0 || cols < 0) return SWIGLU_B200_ERR_SHAPE;
  if (rows == 0 || cols == 0) return SWIGLU_B200_OK;
  if (in_row_stride < cols || grad_row_stride < cols || dout_row_stride < cols) return SWIGLU_B200_ERR_SHAPE;
  if (!dgate || !dup || !dout || !gate || !up) return SWIGLU_B200_ERR_NULL;
  const int es = elem_size(dtype);
  if (addr_of(dgate) % es || addr_of(dup) % es || addr_of(dout) % es || addr_of(gate) % es || addr_of(up) % es)
    return SWIGLU_B200_ERR_ALIGN;

  // Either both gradients overwrite their inputs exactly, or no output touches any input.
  const bool same_g = (dgate == gate), same_u = (dup == up);
  bool inplace = false;
  if (same_g || same_u) {
    if (!(same_g && same_u) || grad_row_stride != in_row_stride) return SWIGLU_B200_ERR_ALIAS;
    inplace = true;
  }
  {
    const Extent edg = extent(dgate, rows, cols, grad_row_stride, es);
    const Extent edu = extent(dup, rows, cols, grad_row_stride, es);
    const Extent ed = extent(dout, rows, cols, dout_row_stride, es);
    if (overlaps(edg, ed) || overlaps(edu, ed)) return SWIGLU_B200_ERR_ALIAS;
    if (!inplace) {
      const Extent eg = extent(gate, rows, cols, in_row_stride, es);
      const Extent eu = extent(up, rows, cols, in_row_stride, es);
      // Interleaved rows of a packed buffer make the bounding extents of dgate and dup
      // overlap each other legitimately; only input/output overlap is an error.
      if (overlaps(edg, eg) || overlaps(edg, eu) || overlaps(edu, eg) || overlaps(edu, eu))
        return SWIGLU_B200_ERR_ALIAS;
    }
  }

  DeviceScope scope(device);
  if (scope.err != cudaSuccess) return fail_cuda(SWIGLU_B200_ERR_DEVICE, scope.err);

  const unsigned long long outs[2] = {addr_of(dgate), addr_of(dup)};
  const unsigned long long ins[3] = {addr_of(dout), addr_of(gate), addr_of(up)};  // in place: gate/up == outs
  const long long pitch[3] = {in_row_stride, grad_row_stride, dout_row_stride};
  Plan p = make_plan(outs, 2, ins, 3, pitch, 3, rows, cols, es);
  p.shape.skew_dout = p.skew[0];
  p.shape.skew_gate = p.skew[1];
  p.shape.skew_up = p.skew[2];
  p.shape.pitch_in = in_row_stride * es;
  p.shape.pitch_out = dout_row_stride * es;
  p.shape.pitch_grad = grad_row_stride * es;
  p.rshape.pitch_in = p.shape.pitch_in;
  p.rshape.pitch_out = p.shape.pitch_out;
  p.rshape.pitch_grad = p.shape.pitch_grad;
  dgate = advance(dgate, p.skip);
  dup = advance(dup, p.skip);
  dout = advance(dout, p.skip);
  gate = advance(gate, p.skip);
  up = advance(up, p.skip);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SWIGLU_B200_F32: return bwd_typed<float, ACT>(p, inplace, dgate, dup, dout, gate, up, gm, dm, st);
    case SWIGLU_B200_F16: return bwd_typed<__half, ACT>(p, inplace, dgate, dup, dout, gate, up, gm, dm, st);
    default: return bwd_typed<__nv_bfloat16, ACT>(p, inplace, dgate, dup, dout, gate, up, gm, dm, st);
  }
}

// Backward that also returns h (see swiglu_bwd_recompute_kernel): six flat tensors of n elements.
template <int ACT>
int recompute_entry(void* h, void* dgate, void* dup, const void* dout, const void* gate, const void* up, int64_t n,
                    int dtype, float gm, float dm, int device, void* stream) {
  if (dtype != SWIGLU_B200_F32 && dtype != SWIGLU_B200_F16 && dtype != SWIGLU_B200_BF16) return SWIGLU_B200_ERR_DTYPE;
  if (n < 0) return SWIGLU_B200_ERR_SHAPE;
  if (n == 0) return SWIGLU_B200_OK;
  if (!h || !dgate || !dup || !dout || !gate || !up) return SWIGLU_B200_ERR_NULL;
  const int es = elem_size(dtype);
  void* outs[3] = {h, dgate, dup};
  const void* ins[3] = {dout, gate, up};
  int width = 16;
  for (int k = 0; k < 3; ++k) {
    if (addr_of(outs[k]) % es || addr_of(ins[k]) % es) return SWIGLU_B200_ERR_ALIGN;
    width = pow2_divisor(addr_of(outs[k]), width);
    width = pow2_divisor(addr_of(ins[k]), width);
  }
  // An output may overwrite one input exactly; any other overlap (outputs with each other included) is an error.
  bool aliased = false;
  for (int a = 0; a < 3; ++a) {
    const Extent ea = extent(outs[a], 1, n, n, es);
    for (int b = a + 1; b < 3; ++b)
      if (overlaps(ea, extent(outs[b], 1, n, n, es))) return SWIGLU_B200_ERR_ALIAS;
    for (int b = 0; b < 3; ++b) {
      if (outs[a] == ins[b]) aliased = true;
      else if (overlaps(ea, extent(ins[b], 1, n, n, es))) return SWIGLU_B200_ERR_ALIAS;
    }
  }
  DeviceScope scope(device);
  if (scope.err != cudaSuccess) return fail_cuda(SWIGLU_B200_ERR_DEVICE, scope.err);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SWIGLU_B200_F32: return recompute_by_width<float, ACT>(width, aliased, h, dgate, dup, dout, gate, up, n, gm, dm, st);
    case SWIGLU_B200_F16: return recompute_by_width<__half, ACT>(width, aliased, h, dgate, dup, dout, gate, up, n, gm, dm, st);
    default: return recompute_by_width<__nv_bfloat16, ACT>(width, aliased, h, dgate, dup, dout, gate, up, n, gm, dm, st);
  }
}

}  // namespace

extern "C" {

int swiglu_b200_fwd(void* out, const void* gate, const void* up, int64_t rows, int64_t cols, int64_t in_row_stride,
                    int64_t out_row_stride, int dtype, float gm, float dm, int device, void* stream) {
  return fwd_entry<ACT_SILU>(out, gate, up, rows, cols, in_row_stride, out_row_stride, dtype, gm, dm, device, stream);
}

int swiglu_b200_bwd(void* dgate, void* dup, const void* dout, const void* gate, const void* up, int64_t rows,
                    int64_t cols, int64_t in_row_stride, int64_t grad_row_stride, int64_t dout_row_stride, int dtype,
                    float gm, float dm, int device, void* stream) {
  return bwd_entry<ACT_SILU>(dgate, dup, dout, gate, up, rows, cols, in_row_stride, grad_row_stride, dout_row_stride,
                             dtype, gm, dm, device, stream);
}

int swiglu_b200_geglu_fwd(void* out, const void* gate, const void* up, int64_t rows, int64_t cols,
                          int64_t in_row_stride, int64_t out_row_stride, int dtype, int approximate_tanh, int device,
                          void* stream) {
  return approximate_tanh
             ? fwd_entry<ACT_GELU_TANH>(out, gate, up, rows, cols, in_row_stride, out_row_stride, dtype, 1.0f, 1.0f,
                                        device, stream)
             : fwd_entry<ACT_GELU_ERF>(out, gate, up, rows, cols, in_row_stride, out_row_stride, dtype, 1.0f, 1.0f,
                                       device, stream);
}

int swiglu_b200_geglu_bwd(void* dgate, void* dup, const void* dout, const void* gate, const void* up, int64_t rows,
                          int64_t cols, int64_t in_row_stride, int64_t grad_row_stride, int64_t dout_row_stride,
                          int dtype, int approximate_tanh, int device, void* stream) {
  return approximate_tanh
             ? bwd_entry<ACT_GELU_TANH>(dgate, dup, dout, gate, up, rows, cols, in_row_stride, grad_row_stride,
                                        dout_row_stride, dtype, 1.0f, 1.0f, device, stream)
             : bwd_entry<ACT_GELU_ERF>(dgate, dup, dout, gate, up, rows, cols, in_row_stride, grad_row_stride,
                                       dout_row_stride, dtype, 1.0f, 1.0f, device, stream);
}

int swiglu_b200_bwd_recompute(void* h, void* dgate, void* dup, const void* dout, const void* gate, const void* up,
                              int64_t n, int dtype, float gm, float dm, int device, void* stream) {
  return recompute_entry<ACT_SILU>(h, dgate, dup, dout, gate, up, n, dtype, gm, dm, device, stream);
}

int swiglu_b200_geglu_bwd_recompute(void* h, void* dgate, void* dup, const void* dout, const void* gate,
                                    const void* up, int64_t n, int dtype, int approximate_tanh, int device,
                                    void* stream) {
  return approximate_tanh
             ? recompute_entry<ACT_GELU_TANH>(h, dgate, dup, dout, gate, up, n, dtype, 1.0f, 1.0f, device, stream)
             : recompute_entry<ACT_GELU_ERF>(h, dgate, dup, dout, gate, up, n, dtype, 1.0f, 1.0f, device, stream);
}

// Reports, without launching anything, how a forward / backward call with these addresses and strides
// would be executed: bits 0-7 the access width in bytes, bit 8 pitched-row addressing, bit 9 the
// skewed-load kernel, bit 10 its one-word variant, bit 11 the ragged-row kernel (16-byte accesses with the
// alignment taken row by row and the second output realigned on the way out), bits 16-23 the scalar head
// elements, bits 24-31 head + tail scalar elements (both zero for the ragged-row kernel, which peels per row).
// Negative: the argument error the real call would return, negated.
int swiglu_b200_plan_fwd(const void* out, const void* gate, const void* up, int64_t rows, int64_t cols,
                         int64_t in_row_stride, int64_t out_row_stride, int dtype) {
  if (dtype != SWIGLU_B200_F32 && dtype != SWIGLU_B200_F16 && dtype != SWIGLU_B200_BF16) return -SWIGLU_B200_ERR_DTYPE;
  if (rows <= 0 || cols <= 0 || in_row_stride < cols || out_row_stride < cols) return -SWIGLU_B200_ERR_SHAPE;
  const int es = elem_size(dtype);
  if (addr_of(out) % es || addr_of(gate) % es || addr_of(up) % es) return -SWIGLU_B200_ERR_ALIGN;
  const unsigned long long outs[1] = {addr_of(out)};
  const unsigned long long ins[2] = {addr_of(gate), addr_of(up)};
  const long long pitch[2] = {in_row_stride, out_row_stride};
  const Plan p = make_plan(outs, 1, ins, 2, pitch, 2, rows, cols, es);
  return plan_code(p);
}

int swiglu_b200_plan_bwd(const void* dgate, const void* dup, const void* dout, const void* gate, const void* up,
                         int64_t rows, int64_t cols, int64_t in_row_stride, int64_t grad_row_stride,
                         int64_t dout_row_stride, int dtype) {
  if (dtype != SWIGLU_B200_F32 && dtype != SWIGLU_B200_F16 && dtype != SWIGLU_B200_BF16) return -SWIGLU_B200_ERR_DTYPE;
  if (rows <= 0 || cols <= 0 || in_row_stride < cols || grad_row_stride < cols || dout_row_stride < cols)
    return -SWIGLU_B200_ERR_SHAPE;
  const int es = elem_size(dtype);
  if (addr_of(dgate) % es || addr_of(dup) % es || addr_of(dout) % es || addr_of(gate) % es || addr_of(up) % es)
    return -SWIGLU_B200_ERR_ALIGN;
  const unsigned long long outs[2] = {addr_of(dgate), addr_of(dup)};
  const unsigned long long ins[3] = {addr_of(dout), addr_of(gate), addr_of(up)};
  const long long pitch[3] = {in_row_stride, grad_row_stride, dout_row_stride};
  const Plan p = make_plan(outs, 2, ins, 3, pitch, 3, rows, cols, es);
  return plan_code(p);
}

}  // extern "C"
