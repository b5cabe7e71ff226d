// Host-buffer entry point: forward + backward of SwiGLU for tensors that live in HOST memory,
// streamed through a caller-provided device workspace in row chunks so that the host-to-device
// copies, the two kernels and the device-to-host copies of different chunks overlap.
// Contract: include/swiglu_b200.h (swiglu_b200_host_fwd_bwd).
#include "swiglu_b200.h"

#include <cuda_runtime.h>

#include <mutex>

namespace {

constexpr int kSlots = 3;            // chunks in flight: one copying in, one computing, one copying out
constexpr uint64_t kAlign = 256;     // alignment of every staging buffer inside the workspace

inline uint64_t round_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

constexpr int kEvents = 3 * kSlots + 1;
constexpr int kMaxDevices = 64;

// The two copy streams and the events of the pipeline are made once per device, on the first call
// for that device, and kept until the process exits: creating and destroying them on every call
// cost more host time than enqueueing the pipeline itself.  One call at a time per device holds
// the lock while it enqueues; a later call may reuse the events at once, because a stream wait
// refers to the record that was current when the wait was issued.
struct DevicePipeline {
  std::mutex lock;
  bool ready = false;
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t ev[kEvents] = {};
};

DevicePipeline g_pipeline[kMaxDevices];

// Must be called with p.lock held and the device current.
bool ensure_pipeline(DevicePipeline& p) {
  if (p.ready) return true;
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t ev[kEvents] = {};
  int made = 0;
  bool ok = cudaStreamCreateWithFlags(&in, cudaStreamNonBlocking) == cudaSuccess &&
            cudaStreamCreateWithFlags(&out, cudaStreamNonBlocking) == cudaSuccess;
  for (; ok && made < kEvents; ++made) ok = cudaEventCreateWithFlags(&ev[made], cudaEventDisableTiming) == cudaSuccess;
  if (!ok) {
    for (int i = 0; i < made; ++i) if (ev[i]) cudaEventDestroy(ev[i]);
    if (in) cudaStreamDestroy(in);
    if (out) cudaStreamDestroy(out);
    return false;
  }
  p.in = in;
  p.out = out;
  for (int i = 0; i < kEvents; ++i) p.ev[i] = ev[i];
  p.ready = true;
  return true;
}

struct DeviceScope {
  int prev_device = -1;
  bool switched = false;
  ~DeviceScope() {
    if (switched) cudaSetDevice(prev_device);
  }
};

}  // namespace

extern "C" {

uint64_t swiglu_b200_host_workspace_bytes(int64_t rows, int64_t cols, int dtype) {
  if (rows <= 0 || cols <= 0) return 0;
  const uint64_t es = dtype == SWIGLU_B200_F32 ? 4 : 2;
  const uint64_t row_bytes = (uint64_t)cols * es;
  // about 32 MiB per staged tensor chunk, at least one row, at most the whole problem
  uint64_t chunk_rows = (32ull << 20) / row_bytes;
  if (chunk_rows < 1) chunk_rows = 1;
  if (chunk_rows > (uint64_t)rows) chunk_rows = (uint64_t)rows;
  return (uint64_t)kSlots * 4 * round_up(chunk_rows * row_bytes, kAlign);
}

int swiglu_b200_host_fwd_bwd(void* h, void* dgate, void* dup, const void* gate, const void* up, const void* dout,
                             int64_t rows, int64_t cols, int dtype, float gm, float dm, void* workspace,
                             uint64_t workspace_bytes, int device, void* stream) {
  if (dtype != SWIGLU_B200_F32 && dtype != SWIGLU_B200_F16 && dtype != SWIGLU_B200_BF16) return SWIGLU_B200_ERR_DTYPE;
  if (rows < 0 || cols < 0) return SWIGLU_B200_ERR_SHAPE;
  if (rows == 0 || cols == 0) return SWIGLU_B200_OK;
  if (!h || !dgate || !dup || !gate || !up || !dout || !workspace) return SWIGLU_B200_ERR_NULL;
  const uint64_t es = dtype == SWIGLU_B200_F32 ? 4 : 2;
  const uint64_t row_bytes = (uint64_t)cols * es;
  if (((uintptr_t)workspace) % kAlign) return SWIGLU_B200_ERR_ALIGN;

  // Largest chunk (in rows) for which kSlots x 4 aligned buffers fit the workspace.
  uint64_t per_buffer = workspace_bytes / (kSlots * 4) / kAlign * kAlign;
  int64_t chunk_rows = (int64_t)(per_buffer / row_bytes);
  if (chunk_rows < 1) return SWIGLU_B200_ERR_WORKSPACE;
  if (chunk_rows > rows) chunk_rows = rows;
  per_buffer = round_up((uint64_t)chunk_rows * row_bytes, kAlign);

  DeviceScope scope;
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
  if (device >= 0 && current != device) {
    scope.prev_device = current;
    if (cudaSetDevice(device) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
    scope.switched = true;
    current = device;
  }
  if (current < 0 || current >= kMaxDevices) return SWIGLU_B200_ERR_DEVICE;
  DevicePipeline& pipe = g_pipeline[current];
  std::lock_guard<std::mutex> guard(pipe.lock);
  if (!ensure_pipeline(pipe)) return SWIGLU_B200_ERR_DEVICE;
  struct { cudaStream_t in, out; cudaEvent_t* ev; } c = {pipe.in, pipe.out, pipe.ev};
  cudaStream_t compute = static_cast<cudaStream_t>(stream);
  cudaEvent_t* loaded = &c.ev[0];            // [slot] inputs of the slot are on the device
  cudaEvent_t* computed = &c.ev[kSlots];     // [slot] both kernels of the slot are done
  cudaEvent_t* drained = &c.ev[2 * kSlots];  // [slot] outputs of the slot are back on the host
  cudaEvent_t start = c.ev[3 * kSlots];

  // Work queued earlier on the caller's stream (it may still use the workspace) goes first.
  if (cudaEventRecord(start, compute) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
  if (cudaStreamWaitEvent(c.in, start, 0) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;

  char* ws = static_cast<char*>(workspace);
  const int64_t n_chunks = (rows + chunk_rows - 1) / chunk_rows;
  for (int64_t k = 0; k < n_chunks; ++k) {
    const int slot = (int)(k % kSlots);
    const int64_t r0 = k * chunk_rows;
    const int64_t nr = (rows - r0) < chunk_rows ? (rows - r0) : chunk_rows;
    const uint64_t bytes = (uint64_t)nr * row_bytes;
    const uint64_t off = (uint64_t)r0 * row_bytes;
    char* d_gate = ws + ((uint64_t)slot * 4 + 0) * per_buffer;
    char* d_up = ws + ((uint64_t)slot * 4 + 1) * per_buffer;
    char* d_dout = ws + ((uint64_t)slot * 4 + 2) * per_buffer;
    char* d_h = ws + ((uint64_t)slot * 4 + 3) * per_buffer;

    // copy in (after the slot's previous occupant has been drained)
    if (k >= kSlots && cudaStreamWaitEvent(c.in, drained[slot], 0) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
    if (cudaMemcpyAsync(d_gate, static_cast<const char*>(gate) + off, bytes, cudaMemcpyHostToDevice, c.in) != cudaSuccess ||
        cudaMemcpyAsync(d_up, static_cast<const char*>(up) + off, bytes, cudaMemcpyHostToDevice, c.in) != cudaSuccess ||
        cudaMemcpyAsync(d_dout, static_cast<const char*>(dout) + off, bytes, cudaMemcpyHostToDevice, c.in) != cudaSuccess)
      return SWIGLU_B200_ERR_COPY;
    if (cudaEventRecord(loaded[slot], c.in) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;

    // compute: forward, then the in-place backward over the staged gate/up
    if (cudaStreamWaitEvent(compute, loaded[slot], 0) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
    int rc = swiglu_b200_fwd(d_h, d_gate, d_up, nr, cols, cols, cols, dtype, gm, dm, -1, compute);
    if (rc != SWIGLU_B200_OK) return rc;
    rc = swiglu_b200_bwd(d_gate, d_up, d_dout, d_gate, d_up, nr, cols, cols, cols, cols, dtype, gm, dm, -1, compute);
    if (rc != SWIGLU_B200_OK) return rc;
    if (cudaEventRecord(computed[slot], compute) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;

    // copy out
    if (cudaStreamWaitEvent(c.out, computed[slot], 0) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
    if (cudaMemcpyAsync(static_cast<char*>(h) + off, d_h, bytes, cudaMemcpyDeviceToHost, c.out) != cudaSuccess ||
        cudaMemcpyAsync(static_cast<char*>(dgate) + off, d_gate, bytes, cudaMemcpyDeviceToHost, c.out) != cudaSuccess ||
        cudaMemcpyAsync(static_cast<char*>(dup) + off, d_up, bytes, cudaMemcpyDeviceToHost, c.out) != cudaSuccess)
      return SWIGLU_B200_ERR_COPY;
    if (cudaEventRecord(drained[slot], c.out) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
  }
  // The caller's stream completes only when every output has landed on the host.
  const int64_t tail = n_chunks < kSlots ? n_chunks : kSlots;
  for (int64_t s = 0; s < tail; ++s)
    if (cudaStreamWaitEvent(compute, drained[s], 0) != cudaSuccess) return SWIGLU_B200_ERR_DEVICE;
  return SWIGLU_B200_OK;
}

}  // extern "C"
