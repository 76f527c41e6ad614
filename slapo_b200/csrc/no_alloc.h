// A C entry point for the backward of the fused bias + activation that
// allocates nothing.  It has no counterpart in the reference framework, whose
// kernels always run under torch's allocator.
//
// Why it exists: the regular entry point (the torch op `bias_act_bwd`) asks
// torch's caching allocator for its outputs and for the fp32 scratch that
// holds the per-chunk column sums of the bias gradient.  Some callers cannot
// do that: a plain C or C++ host program that links this library without
// torch has no such allocator at all, and a runtime that has handed every
// byte of device memory to its own flat parameter / activation arena must not
// let a kernel wrapper grow the footprint behind its back.  For them the
// scratch lives in a file-scope `static __device__` array inside the library
// image, and every other buffer is the caller's.
//
// Limits: cols <= SLAPO_NOALLOC_MAX_COLS, cols a multiple of 8, and the scratch
// this shape needs (chunks x cols floats, at most SLAPO_NOALLOC_SCRATCH_FLOATS
// = 1.25 MiB) must fit; anything larger is refused with
// SLAPO_NOALLOC_E_TOO_LARGE and nothing is launched.
//
// How much scratch a shape needs depends on the GPU: the column sums are split into
// about 8 chunks of rows per SM (never more than rows / 8), so the need is
// min(ceil(8 * SMs / ceil(cols / 256)), ceil(rows / 8)) * cols floats.  On a 148-SM B200
// that is at most 1184 * 256 + cols floats, which fits for every cols up to the
// maximum; a part with 160 SMs or more would refuse some tall shapes that fit here.
// slapo_bias_act_bwd_noalloc_scratch_floats(rows, cols) returns the figure for the
// current device, so a caller can check a shape without launching anything.
//
// Set-up: the first call on each device looks up the device address of the
// scratch array (once per device, with that device current) and caches it.
// That look-up is not a stream operation, so make the first call on a device
// before any stream capture is begun on it.
//
// Concurrency: there is ONE scratch array per device.  Two calls whose kernels
// may overlap on the same device (different streams, or different host
// threads) race on it and give wrong bias gradients; serialise them on one
// stream or with events.  Calls on one stream are ordered and safe.
//
// Nothing in the scratch has to start at zero: every element that the second
// kernel of a call reads was written by the first kernel of the same call.
#pragma once
#include <cuda_runtime.h>

#define SLAPO_NOALLOC_MAX_COLS 16384
#define SLAPO_NOALLOC_SCRATCH_FLOATS 327680  /* 1.25 MiB of fp32 */

#define SLAPO_NOALLOC_OK 0
#define SLAPO_NOALLOC_E_ARGUMENT 1   /* null pointer, bad dtype/act code, cols % 8 != 0 */
#define SLAPO_NOALLOC_E_TOO_LARGE 2  /* shape needs more scratch than the static array has */
#define SLAPO_NOALLOC_E_CUDA 3       /* a CUDA runtime call failed; see the message */

#ifdef __cplusplus
extern "C" {
#endif

// dx = dy * act'(x + bias) and, when dbias != NULL, dbias = column sums of dx.
//   dy, x, dx : [rows, cols] contiguous, element type `dtype`
//               (0 = bf16, 1 = fp16, 2 = fp32); bias, dbias : [cols] or NULL
//   act       : 0 GeLU (erf), 1 GeLU (tanh), 2 ReLU - the codes of the torch op
//   err       : optional buffer of err_len bytes that receives a message when
//               the return value is not SLAPO_NOALLOC_OK
// The kernels are enqueued on `stream` of the current device; the call does not
// synchronise.
int slapo_bias_act_bwd_noalloc(const void* dy, const void* x, const void* bias, void* dx,
                               void* dbias, int rows, int cols, int act, int dtype,
                               cudaStream_t stream, char* err, int err_len);

// Scratch floats that (rows, cols) needs on the current device (148 SMs are assumed when no
// device can be queried); the call above refuses shapes for which this exceeds
// SLAPO_NOALLOC_SCRATCH_FLOATS.
long slapo_bias_act_bwd_noalloc_scratch_floats(int rows, int cols);

#ifdef __cplusplus
}
#endif
