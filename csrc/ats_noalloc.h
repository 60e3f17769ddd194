/* Entry points of libats_b200.so that never allocate memory.
 *
 * This header has no counterpart in the reference project: its kernels always receive their scratch buffers from
 * Python wrappers that allocate them with cudaMalloc / cudaMallocAsync.
 *
 * Who needs this: callers that cannot call cudaMalloc (or any routine that might) at the point where they run the
 * backward pass -- code inside a region where allocation is not permitted, latency-critical loops that must stay out
 * of the driver's allocator, and embedders that give the library a fixed memory budget up front.
 *
 * ats_rmsnorm_bwd_noalloc computes exactly what ats_rmsnorm_bwd computes (input gradient dx and weight gradient dw
 * of y = x * rsqrt(mean(x^2) + eps) * w, bf16 tensors, fp32 math); only the scratch for the per-block weight-gradient
 * partials differs: it is a 4 MiB array built into the library image instead of a caller-supplied buffer.
 *
 *   x, w, dy      bf16 inputs [rows, cols], [cols], [rows, cols]
 *   rstd          fp32 [rows], as written by ats_rmsnorm_fwd
 *   dres_in       optional bf16 [rows, cols] added to dx (may be NULL)
 *   dx            bf16 output [rows, cols]
 *   dw_bf16       optional bf16 output [cols];  dw_f32: optional fp32 output [cols]; accumulate != 0 adds into them
 *   stream        cudaStream_t
 *
 * Limits and rules
 *   - cols must be a multiple of 8 and at most the max_cols reported by ats_rmsnorm_bwd_noalloc_limits (8192);
 *     larger problems are refused with ATS_ERR_NOALLOC_TOO_LARGE and nothing is launched.  rows may be anything up to
 *     2^31 - 1 (more is refused with ATS_ERR_BAD_SHAPE: the kernels index rows with 32-bit integers).
 *   - Every GPU that loads the library holds the 4 MiB array until the process exits.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, no allocation).  Make
 *     that first call before starting any stream capture on that device.
 *   - All calls on one GPU share the one array.  Two calls that can overlap on the GPU (different streams without
 *     an ordering between them) race on it; issue them on one stream or order them with events.
 *   - The array keeps the previous call's contents; the function itself overwrites every element it later reads,
 *     so callers need not clear anything.
 *   - The function calls no cudaMalloc, cudaFree or other allocating routine.
 *
 * Return value: 0 on success, one of the ATS_ERR_* codes below, or a cudaError_t from the launch.
 * ats_noalloc_error_string turns a code into text.
 */
#ifndef ATS_NOALLOC_H
#define ATS_NOALLOC_H

#ifdef __cplusplus
extern "C" {
#endif

#define ATS_ERR_BAD_SHAPE 1003
#define ATS_ERR_NOALLOC_TOO_LARGE 2001
#define ATS_ERR_NOALLOC_DEVICE 2002

int ats_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, const void* dres_in,
                            void* dx, void* dw_bf16, float* dw_f32, int accumulate, long long rows, int cols,
                            void* stream);
void ats_rmsnorm_bwd_noalloc_limits(int* max_cols, long long* scratch_bytes);
const char* ats_noalloc_error_string(int code);

#ifdef __cplusplus
}
#endif
#endif
