// Allocation-free entry point of the native library.
//
// This entry point has no counterpart in the reference (awslabs/state-space-models-neuron): it exists for
// hosts that embed these kernels but are not allowed to obtain device memory while they run.  Typical cases
// are a serving process that handed the whole HBM budget to its own arena at start-up, a latency-critical
// loop where an allocator call is forbidden because cudaMalloc/cudaFree may take driver locks and
// synchronise the device, and plug-in hosts whose policy gives the plug-in no allocator at all.  Such a
// caller still owns its inputs and outputs; what it cannot provide is the temporary storage some kernels need.
//
// ssm_add_rmsnorm_bwd_noalloc is the backward pass of "residual add + RMSNorm" (same math as
// ssm_add_rmsnorm_bwd) that keeps its per-slice partial sums of the weight gradient in a fixed array inside
// the library instead of a caller-provided buffer, and finishes the reduction itself:
//
//   dsum[row, :] = dres_out[row, :] + rmsnorm_backward(dout[row, :])        (bf16 or fp32, like `res`)
//   dw[:]        = sum over rows of dout * normalised(res)                  (fp32 [D], overwritten)
//
// Limits and rules
//   * D must be a multiple of 8 and at most SSM_NOALLOC_MAX_D (8192); larger sizes are rejected with
//     -SSM_NOALLOC_ERR_TOO_LARGE and nothing is launched.  rows >= 1.
//   * res, w, dout, dres_out and dsum must be 16-byte aligned (the kernels use 16-byte vector accesses; rows are
//     then aligned too because D is a multiple of 8) and dw 4-byte aligned; a sub-tensor that starts at an odd
//     offset is rejected with -SSM_NOALLOC_ERR_BAD_ARG before anything is launched.
//   * The library holds SSM_NOALLOC_SLICES * SSM_NOALLOC_MAX_D floats (2 MiB) of device memory per GPU that
//     loads it, from load until the process exits.
//   * The first call on each device looks up the device address of that array (cudaGetSymbolAddress, with
//     that device current).  Make this first call during start-up, before any stream capture begins.
//   * No cudaMalloc, cudaFree or allocating library routine is called, ever.
//   * All calls on a device share the array, and it keeps whatever the previous call left there; the kernels
//     overwrite every entry they later read, so nothing needs clearing between calls.  Two calls that may
//     overlap on the GPU (different streams without an ordering between them) race on it: serialise them.
//   * Returns 0 on success, a negative SSM_NOALLOC_ERR_* code for rejected arguments, a positive cudaError_t
//     otherwise (the value of cudaGetLastError() after the launches, so an error left pending by earlier work on
//     the same thread is reported here too).
#pragma once
#include <cuda_runtime.h>

#define SSM_NOALLOC_MAX_D 8192
#define SSM_NOALLOC_SLICES 64
#define SSM_NOALLOC_ERR_BAD_ARG 3
#define SSM_NOALLOC_ERR_TOO_LARGE 4

#ifdef __cplusplus
extern "C" {
#endif

// res   : the summed residual r' = r + x saved by the forward pass, [rows, D], bf16 (res_fp32 = 0) or fp32
// w     : bf16 [D]
// dout  : bf16 [rows, D], gradient of the normalised output
// dres_out : gradient arriving on the residual stream, same dtype as res, [rows, D], or NULL
// dsum  : output, same dtype as res, [rows, D]
// dw    : output, fp32 [D]
int ssm_add_rmsnorm_bwd_noalloc(const void* res, const void* w, const void* dout, const void* dres_out, void* dsum,
                                void* dw, long long rows, int D, float eps, int res_fp32, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
