// Entry points of the kernel library that never allocate device memory.
//
// This header has no counterpart in the reference project: it exists for hosts that embed
// the library but are not allowed to obtain device memory themselves.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Column sums of a row-major bf16 matrix (the bias-gradient reduction):
//     out[c] (+)= sum over r of x[r][c]        x: [rows][cols] bf16, cols % 8 == 0
//
// Same arithmetic as mb_colsum, but the partial sums between its two stages live in a
// fixed array inside the library (4 MiB per GPU, resident from the moment the library is
// loaded on that GPU until the process exits) instead of a buffer supplied by the caller.
// It is meant for callers that cannot call cudaMalloc or any allocating wrapper: a plugin
// running inside an application whose memory manager owns the whole device, or a service
// that freezes its memory layout after start-up and treats later allocations as errors.
// The caller passes only the input and the output.
//
//   out_fp32 != 0: out is float[cols], else bf16[cols];  accumulate != 0: add to out.
//
// Limit: ceil(rows / 256) * cols <= mb_colsum_static_capacity() (1,048,576 floats).
// Larger problems are refused with return code -22 and a message on stderr; nothing is
// launched.  Other return codes: 0 ok, -1 bad shape, -3 set-up failed, -4 launch failed.
//
// The first call on each GPU looks up the device address of the array (one
// cudaGetSymbolAddress with that GPU current) and remembers it; make that first call
// before starting any stream capture.
// All calls on a GPU use the same array and it keeps whatever the previous call left there.
// That is harmless here because the first stage overwrites every element the second stage
// reads, so nothing has to be cleared; but two calls that overlap on the GPU (different
// streams, or the same stream from two threads without ordering) would race on it.
int mb_colsum_static(const void* x, void* out, int rows, int cols, int out_fp32, int accumulate,
                     cudaStream_t stream);

// Number of floats in the built-in scratch array.
long mb_colsum_static_capacity(void);

#ifdef __cplusplus
}
#endif
