/* swiglu_b200 -- C ABI of the B200 (sm_100a) SwiGLU activation library.
 *
 * The reference (Forge-researchlab/kernel-POCs) has no native boundary for this path: its
 * Python launch wrappers start Triton kernels directly.  Each entry point below replaces one
 * such wrapper-to-kernel hand-off and is what a binding of the reference would call instead:
 *
 *   swiglu_b200_fwd   <- kernels/swiglu/swiglu.py:219-228 (_swiglu_forward_kernel launch in
 *                        swiglu_forward) and :282-291 (_swiglu_packed_forward_kernel launch)
 *   swiglu_b200_bwd   <- kernels/swiglu/swiglu.py:250-261 (_swiglu_backward_kernel launch in
 *                        swiglu_backward) and :312-322 (_swiglu_packed_backward_kernel launch)
 *
 * All pointers are device pointers owned by the caller.  The library allocates no device memory,
 * never synchronises the stream and never aborts: every failure is a non-zero return code.  Calls
 * are asynchronous on `stream` and may be made concurrently from several host threads (for example
 * one per device).  State the library keeps between calls, all of it per process: the launch
 * counters; per device, the SM count and the shared-memory opt-in of the tensor-core kernels,
 * queried or set on their first launch there; per device, once swiglu_b200_host_fwd_bwd has been
 * called for it, two copy streams and ten events that every later call of that entry point on the
 * device reuses (never destroyed; calls for one device are serialised on the host while they
 * enqueue); and the status array of swiglu_b200_gemm_fwd_noalloc described at its declaration.
 *
 * Layouts.  A tensor is `rows` x `cols` elements with a row stride given in ELEMENTS.
 *   separate gate/up  : in_row_stride == out_row_stride == cols
 *   packed gate|up    : gate = base, up = base + cols, in_row_stride = 2*cols,
 *                       out_row_stride = cols (and dup = dgate + cols in the backward)
 * Every combination of base addresses, strides and `cols` is served with wide (16- or 32-byte) accesses:
 * contiguous tensors as one flat stream whatever their alignment (inputs skewed against the outputs are
 * realigned in registers); pitched rows whose pitch, width and bases are multiples of 16 bytes as 16-byte
 * vectors; anything else (the packed layout with an odd half-width, outputs skewed against each other) by
 * kernels that work out the alignment row by row and realign the second output on the way out.  Only the
 * up to 15 elements at each ragged end of a row (or of the flat stream) are handled one at a time.
 *
 * Aliasing.  In the backward, dgate may equal gate and dup may equal up exactly (same address,
 * same stride): the in-place mode of the reference (swiglu.py:247-248, 310).  No other
 * overlap between an output and any input is allowed.
 */
#ifndef SWIGLU_B200_H_
#define SWIGLU_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define SWIGLU_B200_API __attribute__((visibility("default")))
#else
#define SWIGLU_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Element types (the three the reference accepts, swiglu.py:48-50). */
#define SWIGLU_B200_F32 0
#define SWIGLU_B200_F16 1
#define SWIGLU_B200_BF16 2

/* Return codes. */
#define SWIGLU_B200_OK 0
#define SWIGLU_B200_ERR_DTYPE 1       /* dtype is not one of the three codes above            */
#define SWIGLU_B200_ERR_NULL 2        /* a required pointer is NULL while rows*cols > 0        */
#define SWIGLU_B200_ERR_SHAPE 3       /* negative size, or a row stride smaller than cols      */
#define SWIGLU_B200_ERR_ALIGN 4       /* a pointer is not aligned to its element size          */
#define SWIGLU_B200_ERR_ALIAS 5       /* outputs overlap inputs in a way other than exact alias */
#define SWIGLU_B200_ERR_DEVICE 6      /* cudaSetDevice / attribute query failed                */
#define SWIGLU_B200_ERR_LAUNCH 7      /* the kernel launch was rejected by the runtime          */
#define SWIGLU_B200_ERR_COPY 8        /* a host<->device copy of the host-buffer entry failed  */
#define SWIGLU_B200_ERR_WORKSPACE 9   /* the device workspace cannot hold even one token row   */

/* ABI version of this header: major*1000 + minor. */
SWIGLU_B200_API int swiglu_b200_version(void);

/* Static, human-readable text for a return code. */
SWIGLU_B200_API const char* swiglu_b200_strerror(int code);

/* The CUDA runtime error (cudaError_t as int) behind the calling thread's most recent
 * ERR_DEVICE / ERR_LAUNCH / ERR_COPY, 0 if none. */
SWIGLU_B200_API int swiglu_b200_last_cuda_error(void);

/* Number of kernels this library has launched in this process (all threads, all devices).
 * Monotonic; used by benchmarks to report how many launches a timed region contained. */
SWIGLU_B200_API uint64_t swiglu_b200_launch_count(void);

/* Forward: out[r][c] = silu(gate[r][c] * gm) * up[r][c] * dm, computed in fp32 and rounded
 * once to `dtype`.
 *   out            rows x cols, row stride out_row_stride
 *   gate, up       rows x cols, row stride in_row_stride (both)
 *   device         CUDA device ordinal owning the buffers, or -1 for the current device
 *   stream         cudaStream_t (0 = legacy default stream)
 * rows*cols == 0 succeeds without a launch. */
SWIGLU_B200_API int swiglu_b200_fwd(void* out, const void* gate, const void* up, int64_t rows, int64_t cols, int64_t in_row_stride,
                    int64_t out_row_stride, int dtype, float gm, float dm, int device, void* stream);

/* Backward: with z = gate*gm, s = sigmoid(z), d = dout*dm
 *   dup   = d * z * s
 *   dgate = d * up * s * (1 + z*(1 - s)) * gm
 *   dgate, dup     rows x cols, row stride grad_row_stride; may alias gate, up exactly
 *   dout           rows x cols, row stride dout_row_stride
 *   gate, up       rows x cols, row stride in_row_stride */
SWIGLU_B200_API int swiglu_b200_bwd(void* dgate, void* dup, const void* dout, const void* gate, const void* up, int64_t rows,
                    int64_t cols, int64_t in_row_stride, int64_t grad_row_stride, int64_t dout_row_stride, int dtype,
                    float gm, float dm, int device, void* stream);

/* Backward that also recomputes the forward output, in one pass over six flat tensors of n elements:
 *   h = silu(gate*gm) * up * dm,  (dgate, dup) as swiglu_b200_bwd  -- each bit-identical to what
 * swiglu_b200_fwd / swiglu_b200_bwd return for the same inputs.  Replaces the elementwise step of the
 * reference's LoRA-MLP backward (swiglu_DWf_DW_dfg_kernel, called at
 * kernels/lora_mlp/experiments/v3/lora_mlp_kernel_v3.py:324, which overwrites DW with h, e with the
 * gradient of g and g with the gradient of e).  Each output may overwrite ONE input exactly (same address,
 * any pairing); any other overlap returns SWIGLU_B200_ERR_ALIAS.  Pointers that are not all 16-byte aligned
 * run at the widest access every one of them allows. */
SWIGLU_B200_API int swiglu_b200_bwd_recompute(void* h, void* dgate, void* dup, const void* dout, const void* gate,
                              const void* up, int64_t n, int dtype, float gm, float dm, int device, void* stream);

/* swiglu_b200_bwd_recompute for the GeGLU sibling: h = gelu(gate) * up with its backward, no multipliers; results
 * bit-identical to swiglu_b200_geglu_fwd / swiglu_b200_geglu_bwd.  No counterpart in the reference (its LoRA MLP is
 * SiLU only, kernels/lora_mlp/experiments/v3/lora_mlp_kernel_v3.py:133); this is what a LoRA MLP with a GELU gate
 * needs in its backward. */
SWIGLU_B200_API int swiglu_b200_geglu_bwd_recompute(void* h, void* dgate, void* dup, const void* dout, const void* gate,
                                    const void* up, int64_t n, int dtype, int approximate_tanh, int device,
                                    void* stream);

/* Dry run of the access planning of swiglu_b200_fwd / swiglu_b200_bwd (and their GeGLU twins): which
 * access width and addressing a call with these pointers and strides would use.  No CUDA call is made and
 * no memory is touched, so the host-side planning can be tested without a device.  No counterpart in the
 * reference (Triton picks its own vector widths).  Returns, when >= 0:
 *   bits 0-7   access width of the body in bytes (16, 8, 4 or 2)
 *   bit  8     pitched-row addressing (a row stride differs from cols)
 *   bit  9     inputs skewed against the outputs: aligned loads + shuffle + funnel shift
 *   bit  10    ... and every input is within 4 bytes of a boundary: one word from a neighbour completes a vector
 *   bits 16-23 scalar elements peeled in front of the body, bits 24-31 scalar elements in front and behind
 * and when < 0 the negated SWIGLU_B200_ERR_* code the real call would return for these arguments. */
SWIGLU_B200_API int swiglu_b200_plan_fwd(const void* out, const void* gate, const void* up, int64_t rows, int64_t cols,
                         int64_t in_row_stride, int64_t out_row_stride, int dtype);
SWIGLU_B200_API int swiglu_b200_plan_bwd(const void* dgate, const void* dup, const void* dout, const void* gate, const void* up,
                         int64_t rows, int64_t cols, int64_t in_row_stride, int64_t grad_row_stride,
                         int64_t dout_row_stride, int dtype);

/* GeGLU, the sibling operator: h = gelu(gate) * up and its backward, with the tanh approximation
 * (approximate_tanh != 0) or the exact erf form.  Same layouts, strides, aliasing rule and
 * return codes as swiglu_b200_fwd / swiglu_b200_bwd; there are no multipliers.  They replace the
 * Triton launches of the reference's kernels/geglu/geglu.py (forward :396, packed forward :456,
 * backward :425, packed backward :486). */
SWIGLU_B200_API int swiglu_b200_geglu_fwd(void* out, const void* gate, const void* up, int64_t rows, int64_t cols,
                          int64_t in_row_stride, int64_t out_row_stride, int dtype, int approximate_tanh, int device,
                          void* stream);
SWIGLU_B200_API int swiglu_b200_geglu_bwd(void* dgate, void* dup, const void* dout, const void* gate, const void* up, int64_t rows,
                          int64_t cols, int64_t in_row_stride, int64_t grad_row_stride, int64_t dout_row_stride,
                          int dtype, int approximate_tanh, int device, void* stream);

/* Forward + backward for tensors held in HOST memory (pinned memory recommended; pageable
 * memory works but its copies do not overlap).  No counterpart in the reference, whose path
 * only takes device tensors; it serves callers that keep activations off the device and is
 * the call the end-to-end benchmark times.
 *
 * All six tensors are contiguous rows x cols in host memory: gate, up, dout are read; h,
 * dgate, dup are written.  The rows are cut into chunks that fit the caller's device
 * `workspace` (256-byte aligned, any size that holds at least 12 token rows; see
 * swiglu_b200_host_workspace_bytes for a size that makes the chunks about 32 MiB) and three
 * chunks are kept in flight: while one is copied in, the kernels run on the previous one and
 * the one before is copied out, on two internal copy streams (created on the first call for the
 * device and kept) and the caller's `stream`.
 * The call only enqueues work; when `stream` is synchronised every output is on the host.
 * The workspace must not be used by other work until then. */
SWIGLU_B200_API int swiglu_b200_host_fwd_bwd(void* h, void* dgate, void* dup, const void* gate, const void* up, const void* dout,
                             int64_t rows, int64_t cols, int dtype, float gm, float dm, void* workspace,
                             uint64_t workspace_bytes, int device, void* stream);

/* Recommended workspace size in bytes for swiglu_b200_host_fwd_bwd (0 for an empty problem). */
SWIGLU_B200_API uint64_t swiglu_b200_host_workspace_bytes(int64_t rows, int64_t cols, int dtype);

/* Fused gate/up projection with SwiGLU epilogue (bf16, fp32 accumulation on the tcgen05 tensor
 * cores):   h[m][n] = silu((x . w_gate[n]) * gm) * (x . w_up[n]) * dm
 * Replaces, in one launch, the reference's two projection GEMMs followed by the activation
 * kernel (forge/forge/patching/kernels/basic.py:97-102: swiglu(gate_proj(x), up_proj(x))); the
 * reference's own fused attempts are kernels/lora_mlp/experiments/v2/lora_mlp_kernel_v2.py:32-138
 * (Triton dual GEMM) and kernels/lora_mlp/experiments/v4/cublaslt_silu.cu:9-92 (cuBLASLt SWISH).
 *   x              m x k bf16, row-major (k contiguous)
 *   w_gate, w_up   n x k bf16, row-major (the layout of torch.nn.Linear.weight)
 *   h              m x n bf16, row-major
 *   gate_out,up_out  both NULL, or both m x n bf16: the pre-activations rounded to bf16, for a
 *                  backward pass through swiglu_b200_bwd
 *   status         device int, 4-byte aligned, owned by the caller.  The launch zeroes it; after
 *                  the stream has been synchronised it is 0, or the code of the first internal
 *                  wait that gave up (every wait in the kernel is bounded; on such a failure the
 *                  kernel returns early and h is incomplete).
 * Requires k % 8 == 0, n % 16 == 0 and 16-byte aligned pointers. */
SWIGLU_B200_API int swiglu_b200_gemm_fwd(void* h, void* gate_out, void* up_out, const void* x, const void* w_gate, const void* w_up,
                         int64_t m, int64_t n, int64_t k, float gm, float dm, void* status, int device, void* stream);

/* swiglu_b200_gemm_fwd for callers that cannot allocate device memory.  It has no counterpart in
 * the reference; it exists for hosts that are not allowed to (or cannot successfully) call
 * cudaMalloc when they need the kernel: processes in which a memory planner or another
 * framework's caching allocator already holds all device memory, latency-critical loops where
 * cudaMalloc/cudaFree are banned because they synchronise the device, plug-ins that receive their
 * tensors and nothing else.  Same computation and the same requirements on m, n, k and the
 * pointers as swiglu_b200_gemm_fwd (without the optional pre-activation outputs), but the
 * kernel's status word lives in a 256-byte array inside the library image, so the caller passes
 * inputs and outputs only.  The call performs no cudaMalloc/cudaFree and uses no allocating
 * library routine.
 *   status_host    NULL, or where to copy the status word after the kernel, asynchronously on
 *                  `stream`: 0 once the stream is synchronised means success.  It must be pinned
 *                  (page-locked) host memory: a copy to pageable memory blocks the host until it
 *                  is done and cannot be issued while a stream is being captured.  For an empty
 *                  problem (m or n zero) nothing is launched and 0 is stored there directly.
 * Limit: the scratch array is 256 bytes per device and is held by every GPU that loads the
 * library until the process exits; a call needs 4 of them for any problem size, and a call whose
 * need exceeded the array would be refused with SWIGLU_B200_ERR_WORKSPACE.
 * Set-up: the first call on each device looks up the array's device address (and, like the first
 * swiglu_b200_gemm_fwd call, configures the kernel); make that first call before any stream
 * capture is begun.
 * Sharing: every call on a device uses the same array, which keeps the previous call's contents;
 * each call zeroes the status word on `stream` before its kernel runs.  Calls whose kernels
 * overlap on the GPU (different streams, or several host threads) race on that word: serialise
 * them on one stream, or use swiglu_b200_gemm_fwd with a status word per stream. */
SWIGLU_B200_API int swiglu_b200_gemm_fwd_noalloc(void* h, const void* x, const void* w_gate, const void* w_up, int64_t m, int64_t n,
                                 int64_t k, float gm, float dm, int* status_host, int device, void* stream);

/* swiglu_b200_gemm_fwd with the GELU of the GeGLU sibling in the epilogue: h = gelu(x.w_gate^T) * (x.w_up^T),
 * tanh approximation when approximate_tanh != 0, else the erf form; no multipliers.  One launch for the
 * gate/up stage of the reference's geglu_mlp (kernels/geglu/geglu.py:322-377: one or two library GEMMs followed
 * by its GeGLU kernel).  A packed [2n, k] weight (pack_geglu_gate_up_weight, :275-286) is passed as
 * w_gate = packed, w_up = packed + n*k.  Other arguments and requirements as swiglu_b200_gemm_fwd. */
SWIGLU_B200_API int swiglu_b200_geglu_gemm_fwd(void* h, void* gate_out, void* up_out, const void* x, const void* w_gate,
                               const void* w_up, int64_t m, int64_t n, int64_t k, int approximate_tanh, void* status,
                               int device, void* stream);

/* Fused gate/up projection WITH LoRA adapters + SwiGLU, one launch:
 *   e = x.w_gate^T + s_g (x.A_g^T).B_g^T,  g = x.w_up^T + s_u (x.A_u^T).B_u^T,  h = silu(e*gm) * g * dm.
 * Replaces the reference's Triton dual GEMM with fused LoRA, _fused_gate_up_swiglu_kernel / fused_gate_up_swiglu
 * (kernels/lora_mlp/experiments/v2/lora_mlp_kernel_v2.py:32-209), and, against its v3 path, the two base GEMMs
 * plus fused_lora_swiglu (v3:141-200) without e and g ever leaving the chip unless asked for.
 *   xa_scaled [m, 2r]  = [s_g * x.A_g^T | s_u * x.A_u^T], bf16, prepared by the caller (a skinny library GEMM)
 *   b_gate, b_up [n, r] the adapters' second factors; r a multiple of 8, at most 64 (r = 0: no adapters)
 *   e_out, g_out       NULL, or where to store e and g (bf16) for a backward pass
 * The adapter terms are extra steps of the same contraction (see csrc/swiglu_gemm.cu); other arguments and
 * requirements as swiglu_b200_gemm_fwd. */
SWIGLU_B200_API int swiglu_b200_lora_gemm_fwd(void* h, void* e_out, void* g_out, const void* x, const void* w_gate,
                              const void* w_up, const void* xa_scaled, const void* b_gate, const void* b_up, int64_t m,
                              int64_t n, int64_t k, int64_t r, float gm, float dm, void* status, int device,
                              void* stream);

/* swiglu_b200_lora_gemm_fwd with the GELU of the GeGLU sibling in the epilogue (tanh approximation when
 * approximate_tanh != 0, else the erf form): the gate/up stage of a LoRA MLP of the Gemma family in one launch.
 * The reference has no fused kernel for this case and routes it through its projection modules and geglu
 * (forge/forge/patching/kernels/lora.py:166-188). */
SWIGLU_B200_API int swiglu_b200_lora_geglu_gemm_fwd(void* h, void* e_out, void* g_out, const void* x, const void* w_gate,
                                    const void* w_up, const void* xa_scaled, const void* b_gate, const void* b_up,
                                    int64_t m, int64_t n, int64_t k, int64_t r, int approximate_tanh, void* status,
                                    int device, void* stream);

/* Backward GEMMs of the fused projection, from dgate/dup (the outputs of swiglu_b200_bwd on the
 * saved pre-activations):
 *     dx      [m, k] = dgate . w_gate + dup . w_up        (skipped when dx is NULL)
 *     dw_gate [n, k] = dgate^T . x,  dw_up [n, k] = dup^T . x   (both NULL to skip, or both given)
 * bf16 in and out, fp32 accumulation on the tcgen05 tensor cores, no transposed copies.  In the
 * reference these are the cuBLAS GEMMs autograd derives for down_proj(swiglu(gate_proj(x), up_proj(x)))
 * (forge/forge/patching/kernels/basic.py:97-102).  dgate, dup: m x n; x: m x k; w_gate, w_up: n x k;
 * all row-major and 16-byte aligned; requires k % 16 == 0 and n % 8 == 0.  `status` as in
 * swiglu_b200_gemm_fwd (one word serves both launches). */
SWIGLU_B200_API int swiglu_b200_gemm_bwd(void* dx, void* dw_gate, void* dw_up, const void* dgate, const void* dup, const void* x,
                         const void* w_gate, const void* w_up, int64_t m, int64_t n, int64_t k, void* status,
                         int device, void* stream);

/* Number of backward-GEMM kernels launched by this process. */
SWIGLU_B200_API uint64_t swiglu_b200_gemm_bwd_launch_count(void);

/* TEST-ONLY: makes a bounded wait run out.  No counterpart in the reference.  Every mbarrier wait of
 * the tensor-core kernels above gives up after a limit, stores a code in the launch's status word
 * and lets the kernel return; this entry launches one CTA of one warp that initialises a barrier
 * nothing ever arrives at and waits on it with the same wait function and a limit of
 * `limit_cycles` SM clock cycles (at most 40 000 000, about 20 ms).  No bulk copy, tensor memory or
 * MMA is involved, and the real kernels are not altered for it.  After the stream is synchronised
 * `status` (device int, zeroed by the launch, as for swiglu_b200_gemm_fwd) holds `code` (non-zero).
 *   mode   0: the CTA-scope wait of the one-CTA kernels; 1: the CTA-scope wait of the CTA-pair
 *          kernels; 2: the same with its 200 ns pause between polls; 3: their cluster-scope wait. */
SWIGLU_B200_API int swiglu_b200_selftest_wait_timeout(void* status, int mode, int64_t limit_cycles, int code, int device,
                                      void* stream);

/* LoRA + SwiGLU epilogue (bf16):
 *     e = e_base + s_gate * (xa_gate . b_gate^T),  g = g_base + s_up * (xa_up . b_up^T),  h = silu(e) * g
 * Replaces the launch of _fused_lora_swiglu_kernel in the reference's fused_lora_swiglu
 * (kernels/lora_mlp/experiments/v3/lora_mlp_kernel_v3.py:141-200).
 *   e_base, g_base   m x n   outputs of the frozen gate / up projections
 *   xa_gate, xa_up   m x r   x . A^T of the two adapters        b_gate, b_up   n x r
 *   h                m x n   result;   e_out, g_out: both NULL, or m x n to receive e and g (the
 *                            reference's save_eg=True, for the backward)
 * All row-major, contiguous, 16-byte aligned; requires r % 8 == 0, 8 <= r <= 64, n % 8 == 0.
 * `status` as in swiglu_b200_gemm_fwd. */
SWIGLU_B200_API int swiglu_b200_lora_swiglu_fwd(void* h, void* e_out, void* g_out, const void* e_base, const void* g_base,
                                const void* xa_gate, const void* xa_up, const void* b_gate, const void* b_up,
                                int64_t m, int64_t n, int64_t r, float s_gate, float s_up, void* status, int device,
                                void* stream);

/* Number of LoRA + SwiGLU epilogue kernels launched by this process. */
SWIGLU_B200_API uint64_t swiglu_b200_lora_launch_count(void);

/* Number of fused-GEMM kernels launched by this process. */
SWIGLU_B200_API uint64_t swiglu_b200_gemm_launch_count(void);

#ifdef __cplusplus
}
#endif

#endif /* SWIGLU_B200_H_ */
