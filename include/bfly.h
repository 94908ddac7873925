/* bfly.h -- C ABI of the B200 butterfly-multiply library (libbfly_b200.so).
 *
 * The library replaces the device side of HazyResearch/butterfly's `torch_butterfly`
 * operators for CUDA tensors: the forward and backward of the product of
 * nblocks*log2(n) sparse factors made of 2x2 "twiddle" blocks, and the radix-4
 * ("base-4") variant.  Every entry point
 *   - takes plain device pointers and sizes (no torch types),
 *   - enqueues its kernels on `stream` (a cudaStream_t, NULL = default stream) and
 *     returns without synchronising,
 *   - never allocates device memory (scratch is passed in by the caller),
 *   - returns 0 or a negative BFLY_E_* code (see bfly_strerror); it never throws.
 * There is no CPU implementation behind these symbols.
 *
 * Layouts (all row-major, element type float or interleaved complex64):
 *   twiddle   (nstacks, nblocks, log_n, n/2, 2, 2)   contiguous, 16-byte aligned
 *   twiddle4  (nstacks, nblocks, log_n/2, n/4, 4, 4) contiguous, 16-byte aligned
 *   twiddle2  (nstacks, nblocks, log_n%2, n/2, 2, 2) contiguous, 16-byte aligned
 *   x         (batch, nstacks, input_size)  last dim contiguous; x_sB / x_sS are the
 *             element strides of the batch and stack dims (x_sS may be 0: one row
 *             broadcast to every stack, as Butterfly.pre_process's expand() produces)
 *   out       (batch, nstacks, n) contiguous; only columns < output_size are written (products
 *             with rows wider than one launch covers -- n > 8192 float32 (4096 without the forward's
 *             workspace), > 2048 complex64 -- or of more than about 120 stages run as several
 *             launches and use the columns beyond output_size as working space)
 *   grad      (batch, nstacks, output_size), strides g_sB / g_sS, last dim contiguous
 *   d_twiddle (d_twiddle4, d_twiddle2): like the twiddle they belong to, 16-byte aligned
 *   d_x       (batch, nstacks, max(input_size, n)) contiguous; columns < input_size
 *             hold the input gradient (columns >= n of them are zero)
 * Input columns >= n are ignored, missing ones (input_size < n) read as zero, exactly as
 * the reference pads (csrc/cpu/butterfly_cpu.cpp:47-49, csrc/cuda/butterfly_cuda.cu:148-149).
 */
#ifndef BFLY_H_
#define BFLY_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BFLY_OK 0
#define BFLY_E_ARG (-1)          /* inconsistent sizes or a null pointer */
#define BFLY_E_UNSUPPORTED (-2)  /* shape outside what the kernels cover */
#define BFLY_E_ALIGN (-3)        /* twiddle or d_twiddle pointer not 16-byte aligned */
#define BFLY_E_WORKSPACE (-4)    /* workspace missing, misaligned or too small */
#define BFLY_E_CUDA (-5)         /* a CUDA runtime call or launch failed */
#define BFLY_E_NODEVICE (-6)     /* no usable CUDA device */
#define BFLY_E_TOOLARGE (-7)     /* needs more scratch than the built-in buffer of the no-allocation entry point */

#define BFLY_F32 0
#define BFLY_C64 1

/* Human-readable text for a status code. */
const char* bfly_strerror(int status);

/* Library version (major*10000 + minor*100 + patch) and the CUDA toolkit version it was
 * compiled with (CUDA_VERSION, e.g. 12090).  The latter backs the reference's
 * `torch_butterfly::cuda_version` operator (csrc/version.cpp:14-23). */
int bfly_version(void);
int bfly_cuda_version(void);

/* Scratch bytes the forward can use for this shape (0 = none; dtype is BFLY_F32 or BFLY_C64):
 * room for a copy of the twiddles re-ordered for the fastest forward kernel (float32 rows of
 * 512 .. 8192 columns in one launch; wider single-stack rows pass by pass).  Returns a negative
 * status on error. */
int64_t bfly_fw_workspace_bytes(int dtype, int batch, int nstacks, int log_n, int nblocks);

/* Forward: out = B_{nblocks-1} ... B_0 x.
 * Replaces butterfly_multiply_fw_cuda (csrc/cuda/butterfly_cuda.h:6-9,
 * csrc/cuda/butterfly_cuda.cu:349-416), reached from the operator
 * torch_butterfly::butterfly_multiply_fw (csrc/butterfly.cpp:20-53).
 * `workspace` (16-byte aligned, bfly_fw_workspace_bytes long) is optional: with NULL / too few
 * bytes the call still computes the same result, on the generic (slower) kernel. */
int bfly_fw_f32(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS, float* out,
                int batch, int nstacks, int log_n, int nblocks, int input_size, int output_size,
                int increasing_stride, void* workspace, size_t workspace_bytes, void* stream);
int bfly_fw_c64(const void* twiddle, const void* x, int64_t x_sB, int64_t x_sS, void* out,
                int batch, int nstacks, int log_n, int nblocks, int input_size, int output_size,
                int increasing_stride, void* workspace, size_t workspace_bytes, void* stream);

/* Scratch bytes bfly_bw_* needs for this shape (0 when the whole product is one
 * backward phase; it includes the scratch of the forward pass the backward runs).  dtype is BFLY_F32 or BFLY_C64.  Returns a negative status on error. */
int64_t bfly_bw_workspace_bytes(int dtype, int batch, int nstacks, int log_n, int nblocks);

/* Backward: d_twiddle (same layout as twiddle, overwritten) and d_x from grad.
 * Replaces butterfly_multiply_bw_cuda (csrc/cuda/butterfly_cuda.h:11-15,
 * csrc/cuda/butterfly_cuda.cu:534-646), reached from torch_butterfly::butterfly_multiply_bw
 * (csrc/butterfly.cpp:56-93).  `workspace` (256-byte aligned, workspace_bytes long) takes
 * the place of the reference's `intermediate_storage` tensor (butterfly_cuda.cu:554-555). */
int bfly_bw_f32(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS, const float* grad,
                int64_t g_sB, int64_t g_sS, float* d_twiddle, float* d_x, int batch, int nstacks,
                int log_n, int nblocks, int input_size, int output_size, int increasing_stride,
                void* workspace, size_t workspace_bytes, void* stream);
int bfly_bw_c64(const void* twiddle, const void* x, int64_t x_sB, int64_t x_sS, const void* grad,
                int64_t g_sB, int64_t g_sS, void* d_twiddle, void* d_x, int batch, int nstacks,
                int log_n, int nblocks, int input_size, int output_size, int increasing_stride,
                void* workspace, size_t workspace_bytes, void* stream);

/* Backward for callers that cannot give the library scratch memory.  (No counterpart in the
 * reference: its backward always allocates its `intermediate_storage` through torch.)
 *
 * Same arguments and results as bfly_bw_f32, minus the workspace: the snapshots of the
 * activation that the backward writes between its phases go into a buffer that is part of
 * the library image itself, a fixed BFLY_NOALLOC_SCRATCH_BYTES per GPU that stays resident
 * from the moment the library is loaded on that GPU until the process exits.  It exists for
 * hosts where a device allocation is not an option at the call site: code running inside a
 * CUDA-graph capture or a real-time loop where cudaMalloc would synchronise the device, a
 * plugin whose host framework owns all device memory and hands out none, a process whose
 * memory budget was fixed at start-up.  The call makes no cudaMalloc / cudaFree and uses no
 * allocating library routine.
 *
 * Limits and rules:
 *  - the shape must need at most BFLY_NOALLOC_SCRATCH_BYTES of scratch (what
 *    bfly_bw_workspace_bytes reports); larger problems return BFLY_E_TOOLARGE and do nothing.
 *    Shapes whose backward is a single phase (nblocks * log_n <= 8 with n <= 1024) need none.
 *  - the first call on each GPU looks up the buffer's device address (one
 *    cudaGetSymbolAddress with that GPU current); make that first call outside any stream
 *    capture.
 *  - every call on a GPU shares the one buffer, and the buffer keeps the previous call's
 *    contents.  Nothing in it needs clearing (each snapshot is written in full before it is
 *    read), but two calls whose kernels overlap on the GPU -- different streams, different
 *    host threads -- race on it: serialise them.
 */
#define BFLY_NOALLOC_SCRATCH_BYTES (32u << 20)
int bfly_bw_f32_noalloc(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS,
                        const float* grad, int64_t g_sB, int64_t g_sS, float* d_twiddle, float* d_x,
                        int batch, int nstacks, int log_n, int nblocks, int input_size,
                        int output_size, int increasing_stride, void* stream);

/* Base-4 forward / backward (float32).  The reference computes this product with
 * PyTorch view/permute/sum ops only (torch_butterfly/multiply_base4.py:7-41,
 * butterfly_multiply_base4_torch); these entry points are its native counterpart.
 * twiddle2 may be NULL when log_n is even, twiddle4 may be NULL when log_n == 1. */
int bfly4_fw_f32(const float* twiddle4, const float* twiddle2, const float* x, int64_t x_sB,
                 int64_t x_sS, float* out, int batch, int nstacks, int log_n, int nblocks,
                 int input_size, int output_size, int increasing_stride, void* stream);
int bfly4_fw_c64(const void* twiddle4, const void* twiddle2, const void* x, int64_t x_sB, int64_t x_sS,
                 void* out, int batch, int nstacks, int log_n, int nblocks, int input_size,
                 int output_size, int increasing_stride, void* stream);
int bfly4_bw_c64(const void* twiddle4, const void* twiddle2, const void* x, int64_t x_sB,
                 int64_t x_sS, const void* grad, int64_t g_sB, int64_t g_sS, void* d_twiddle4,
                 void* d_twiddle2, void* d_x, int batch, int nstacks, int log_n, int nblocks,
                 int input_size, int output_size, int increasing_stride, void* workspace,
                 size_t workspace_bytes, void* stream);
int64_t bfly4_bw_workspace_bytes(int dtype, int batch, int nstacks, int log_n, int nblocks);
int bfly4_bw_f32(const float* twiddle4, const float* twiddle2, const float* x, int64_t x_sB,
                 int64_t x_sS, const float* grad, int64_t g_sB, int64_t g_sS, float* d_twiddle4,
                 float* d_twiddle2, float* d_x, int batch, int nstacks, int log_n, int nblocks,
                 int input_size, int output_size, int increasing_stride, void* workspace,
                 size_t workspace_bytes, void* stream);

/* Forward / backward pair that trades memory for time.  No counterpart in the reference, whose
 * autograd node saves only {twiddle, input} and recomputes everything in the backward
 * (csrc/butterfly.cpp:99-118).
 *
 * bfly_fw_*_saving is the forward that also leaves in `snapshots` the activations at the
 * backward's phase boundaries (bfly_bw_workspace_bytes bytes for the same problem; 0 bytes when
 * the backward has a single phase).  bfly_bw_*_saved is the backward that starts from them
 * instead of recomputing them: same arguments and results as bfly_bw_*, with `snapshots` as
 * written by the matching forward (same twiddle, x, sizes and direction) and left untouched. */
int bfly_fw_f32_saving(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS, float* out,
                       int batch, int nstacks, int log_n, int nblocks, int input_size,
                       int output_size, int increasing_stride, void* snapshots,
                       size_t snapshot_bytes, void* stream);
int bfly_fw_c64_saving(const void* twiddle, const void* x, int64_t x_sB, int64_t x_sS, void* out,
                       int batch, int nstacks, int log_n, int nblocks, int input_size,
                       int output_size, int increasing_stride, void* snapshots,
                       size_t snapshot_bytes, void* stream);
int bfly_bw_f32_saved(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS,
                      const float* grad, int64_t g_sB, int64_t g_sS, float* d_twiddle, float* d_x,
                      int batch, int nstacks, int log_n, int nblocks, int input_size,
                      int output_size, int increasing_stride, void* snapshots,
                      size_t snapshot_bytes, void* stream);
int bfly_bw_c64_saved(const void* twiddle, const void* x, int64_t x_sB, int64_t x_sS,
                      const void* grad, int64_t g_sB, int64_t g_sS, void* d_twiddle, void* d_x,
                      int batch, int nstacks, int log_n, int nblocks, int input_size,
                      int output_size, int increasing_stride, void* snapshots,
                      size_t snapshot_bytes, void* stream);

/* Development and test switches (no counterpart in the reference).  They are read from the
 * environment once, when the library first needs them, and can be changed at run time here; the
 * launch path never reads the environment.  Names (environment variable): "tma" (BFLY_TMA: 0 =
 * per-thread tile copies instead of the TMA unit), "fw2" (BFLY_FW2: 0 = generic forward kernel
 * only), "bw_v2" (BFLY_BW_V2), "fw_kmax", "fw_rows", "fw_logcmax", "bw_rows", "bw_maxsg" (planner
 * overrides; -1 = default), "autograd_save" (BFLY_AUTOGRAD_SAVE: the torch autograd operator keeps
 * the forward's snapshots: 0 never, 1 always, -1 by size).  Returns BFLY_E_ARG for an unknown name. */
int bfly_set_option(const char* name, int value);
int bfly_get_option(const char* name, int* value);

/* Butterfly as a linear layer, fused (float32).  Replaces the PyTorch glue around the operator in
 * the reference's Butterfly module (torch_butterfly/butterfly.py:152-169: pre_process expands the
 * input over the stacks, post_process flattens the stacks, slices and adds the bias) and what
 * autograd makes of it in the backward (sum of the input gradient over the stacks, column sum of
 * grad for the bias).
 *   x       (batch, input_size) rows with pitch x_sB, shared by all stacks
 *   out     (batch, nstacks * n) contiguous; the layer's output is its first output_size columns
 *           (output_size <= nstacks * n; columns beyond it are working space)
 *   bias    (output_size) or NULL: added in the forward kernel's store epilogue
 * bfly_linear_bw_f32 returns d_twiddle, d_input (batch, input_size; pitch d_input_sB) already summed
 * over the stacks (the last phase adds its tiles into it: float32 additions in no fixed order, so
 * the last bits can differ between runs) and d_bias (output_size, or NULL).  It needs grad
 * (batch, output_size; pitch g_sB) with output_size == nstacks * n, input_size a multiple of 32 and
 * <= n, 16-byte aligned rows and batch >= 5; otherwise, or when a phase does not fit its kernel, it
 * returns BFLY_E_UNSUPPORTED before writing anything and the caller composes bfly_bw_f32 with its
 * own reductions.  Workspace: bfly_linear_bw_workspace_bytes (forward: bfly_fw_workspace_bytes). */
int bfly_linear_fw_f32(const float* twiddle, const float* x, int64_t x_sB, float* out, const float* bias,
                       int batch, int nstacks, int log_n, int nblocks, int input_size, int output_size,
                       int increasing_stride, void* workspace, size_t workspace_bytes, void* stream);
int64_t bfly_linear_bw_workspace_bytes(int batch, int nstacks, int log_n, int nblocks);
int bfly_linear_bw_f32(const float* twiddle, const float* x, int64_t x_sB, const float* grad, int64_t g_sB,
                       float* d_twiddle, float* d_input, int64_t d_input_sB, float* d_bias, int batch,
                       int nstacks, int log_n, int nblocks, int input_size, int output_size,
                       int increasing_stride, void* workspace, size_t workspace_bytes, void* stream);

/* Forward with glue operators folded into the launch.  Replaces the element-wise and gather
 * modules that surround a Butterfly in the reference's exact-transform pipelines, each of which is
 * a pass of its own over the rows there: FixedPermutation (torch_butterfly/permutation.py:65-75),
 * Real2Complex / Complex2Real and index_last_dim (torch_butterfly/complex_utils.py:100-142),
 * Diagonal (torch_butterfly/diagonal.py:11-38), as composed in torch_butterfly/special.py
 * (fft / ifft with their bit-reversal, circulant = fft, diagonal, ifft).  In order:
 *   x_is_real   x holds float32 rows that enter the complex product with zero imaginary part
 *   in_perm     (n int32, or NULL) row[c] <- row[in_perm[c]] before the first factor
 *   out_diag    (n elements, or NULL) y[c] <- y[c] * out_diag[c] after the last factor
 *   out_perm    (n int32, or NULL) y[c] <- y[out_perm[c]] after the diagonal
 *   out_is_real out receives float32 rows: the real parts of the result
 * Same arguments and result as bfly_fw_* otherwise; x_sB / x_sS count elements of x as given
 * (floats when x_is_real), out is (batch, nstacks, n) contiguous in its own element type.
 * Gathers and the diagonal need input_size == n / output_size == n.  Rows must fit one CTA's
 * shared memory (n <= 4096 float32, n <= 2048 complex64); otherwise BFLY_E_UNSUPPORTED and the
 * caller runs the operators one by one. */
int bfly_fw_glue_f32(const float* twiddle, const float* x, int64_t x_sB, int64_t x_sS, float* out,
                     const int32_t* in_perm, const float* out_diag, const int32_t* out_perm, int batch,
                     int nstacks, int log_n, int nblocks, int input_size, int output_size,
                     int increasing_stride, void* stream);
int bfly_fw_glue_c64(const void* twiddle, const void* x, int x_is_real, int64_t x_sB, int64_t x_sS,
                     void* out, int out_is_real, const int32_t* in_perm, const void* out_diag,
                     const int32_t* out_perm, int batch, int nstacks, int log_n, int nblocks,
                     int input_size, int output_size, int increasing_stride, void* stream);

/* Twiddles of a unitary butterfly from their angles, and the gradient of the angles.  Replaces the
 * chain of cos / sin / stack operators (and autograd's backward of it) that the reference's
 * ButterflyUnitary.forward runs on every call (torch_butterfly/butterfly.py:271-280).
 *   angles     (blocks, 4) float32: phi, alpha, psi, chi of each 2x2 block
 *   twiddle    (blocks, 2, 2) complex64 = [[cos(phi) e^{i(alpha+psi)},  sin(phi) e^{i(alpha+chi)}],
 *                                          [-sin(phi) e^{i(alpha-chi)}, cos(phi) e^{i(alpha-psi)}]]
 *   d_twiddle  gradient of the entries (dL/dRe + i dL/dIm), d_angles (blocks, 4) float32
 * `blocks` = nstacks * nblocks * log_n * n/2.  All pointers 16-byte aligned, tensors contiguous. */
int bfly_unitary_twiddle_fw(const float* angles, void* twiddle, int64_t blocks, void* stream);
int bfly_unitary_twiddle_bw(const float* angles, const void* d_twiddle, float* d_angles, int64_t blocks,
                            void* stream);

/* Number of kernels the library has launched in this process so far (all entry points). */
int64_t bfly_launch_count(void);

/* Every wait inside the kernels (on a bulk tensor copy) is bounded; a kernel whose wait ran out
 * stops early, leaves invalid output and raises a flag in device memory.  This call waits for
 * the current device to go idle, returns the flag (0 = no kernel has given up since the last
 * call, 1 = a wait ran out, 2 = a kernel found its shared-memory window misaligned) and clears it; a negative status on a CUDA error.  No counterpart in the
 * reference; meant for tests and for hosts that want to double-check a run. */
int bfly_device_error(void);
/* The same flag without waiting for the device: enqueues, on `stream`, a copy of the flag into
 * *host_flag (host memory, pinned for a truly asynchronous copy).  The caller reads it after its own
 * next synchronisation with that stream; the flag is not cleared (bfly_device_error clears it).  A
 * training loop calls this once per step behind its kernels and looks at the value where it
 * synchronises anyway (butterfly_b200/host.py does, in HostPipeline.wait). */
int bfly_device_error_async(int* host_flag, void* stream);

/* Self-test of that protocol, for tests: launches one warp that waits, for at most `polls` polls
 * (1 .. 2^20), on a barrier whose data never arrives, gives up, raises the flag and returns.  After
 * it bfly_device_error() returns 1 once and the device is as usable as before.  No counterpart in
 * the reference. */
int bfly_selftest_bounded_wait(int polls, void* stream);

/* Per-kernel timing for benchmarks.  While enabled, every launch is bracketed by a pair of
 * CUDA events on its stream.  bfly_profile_collect waits for the recorded launches, adds
 * their count and device time into launches[id] / total_ms[id] (ids below; n_ids entries each)
 * and forgets them.  Leave it disabled in production: the events serialise nothing but do cost
 * host time. */
#define BFLY_KERNEL_FW 0   /* generic forward kernel (bfly_fw_kernel) */
#define BFLY_KERNEL_BW 1   /* first-generation backward phase kernel (bfly_bw_kernel) */
#define BFLY_KERNEL_FW2 2  /* packed-pair forward kernel with its twiddle re-ordering kernel (bfly_fw2_kernel) */
#define BFLY_KERNEL_BW2 3  /* backward phase kernel with accumulators in tensor memory (bfly_bw2_kernel) */
#define BFLY_KERNEL_BW3 4  /* packed-pair backward phase kernel (bfly_bw3_kernel) */
#define BFLY_KERNEL_IDS 5
void bfly_profile_enable(int on);
int bfly_profile_collect(int64_t* launches, double* total_ms, int n_ids);

#ifdef __cplusplus
}
#endif
#endif /* BFLY_H_ */
