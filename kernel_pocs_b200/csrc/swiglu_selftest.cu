// Test-only kernel for the failure path of the tensor-core kernels: a bounded wait that runs out.
//
// The tcgen05 kernels of this library bound every mbarrier wait; a wait that gives up stores a code
// in the launch's status word and the kernel returns instead of hanging.  Making a real kernel's wait
// run out would take a deliberately broken pipeline, so this file has ONE small kernel that uses
// the very same wait functions (tcgen05_common.cuh) on a barrier that nothing ever arrives at, with
// a limit of about a millisecond: one CTA, one warp, no bulk copy, no tensor memory, no MMA.  It
// always terminates: by the limit, or at once if the status word is already non-zero.
// Contract: include/swiglu_b200.h (swiglu_b200_selftest_wait_timeout).
#include "swiglu_b200.h"
#include "tcgen05_common.cuh"

namespace {

using namespace swiglu_b200::tc;

constexpr long long kMaxLimitCycles = 40000000LL;  // ~20 ms of SM clock: the most a caller may ask for

__global__ void __launch_bounds__(32) selftest_wait_timeout_kernel(int* status, int mode, long long limit, int code) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  bool flipped;
  switch (mode) {
    case 1: flipped = wait<false>(&bar, 0, status, code, limit); break;
    case 2: flipped = wait<false, 200>(&bar, 0, status, code, limit); break;
    case 3: flipped = wait<true>(&bar, 0, status, code, limit); break;
    default: flipped = mbar_wait(&bar, 0, status, code, limit); break;
  }
  // nobody arrives, so a wait that reports success is itself the failure
  if (flipped) atomicCAS(status, 0, -code);
  // the same barrier the real kernels run before they free their resources
  settle_before_teardown(status);
}

}  // namespace

extern "C" int swiglu_b200_selftest_wait_timeout(void* status, int mode, int64_t limit_cycles, int code, int device,
                                                 void* stream) {
  if (!status) return SWIGLU_B200_ERR_NULL;
  if ((uintptr_t)status % 4) return SWIGLU_B200_ERR_ALIGN;
  if (mode < 0 || mode > 3 || code == 0 || limit_cycles < 0 || limit_cycles > kMaxLimitCycles)
    return SWIGLU_B200_ERR_SHAPE;
  int prev = -1;
  bool switched = false;
  if (device >= 0) {
    if (cudaGetDevice(&prev) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
    if (prev != device) {
      if (cudaSetDevice(device) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
      switched = true;
    }
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = SWIGLU_B200_OK;
  if (cudaMemsetAsync(status, 0, sizeof(int), st) != cudaSuccess) {
    rc = SWIGLU_B200_ERR_DEVICE;
  } else {
    selftest_wait_timeout_kernel<<<1, 32, 0, st>>>(static_cast<int*>(status), mode, (long long)limit_cycles, code);
    if (cudaGetLastError() != cudaSuccess) rc = SWIGLU_B200_ERR_LAUNCH;
  }
  if (switched) cudaSetDevice(prev);
  return rc;
}
