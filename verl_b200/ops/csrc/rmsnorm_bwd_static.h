// RMSNorm backward that never allocates.
//
// This entry point has no counterpart in the reference project; it exists for callers of this library that
// are not allowed to allocate device memory at the point where they call us: code running inside a
// fixed-footprint serving process, a plug-in that is handed raw device pointers by a host it does not
// control, or C / ctypes users that link the shared object without the tensor library and therefore have no
// caching allocator to ask.  The regular launcher (vb_rmsnorm_bwd) leaves the partial-sum buffer to the
// caller; this one owns a fixed buffer that is part of the loaded module instead.
#pragma once
#include <cuda_runtime.h>

extern "C" {
// Largest problem the built-in buffer covers: rows are unlimited, the row length is not.
#define VB_RMSNORM_BWD_STATIC_MAX_H 8192     // elements per row (multiple of 8)
#define VB_RMSNORM_BWD_STATIC_MAX_BLOCKS 148 // partial rows kept (one per SM)

// dx[T,H] (bf16) and dw[H] (fp32; overwritten, or added to when accumulate_dw != 0) from dy, x, w (bf16),
// rstd[T] (fp32) and an optional incoming residual gradient dres_in (bf16, may be null).  Rows are contiguous
// (row stride H).  dy, x, w, dx and dres_in are read and written 16 bytes at a time and must be 16-byte
// aligned; rstd and dw need the natural 4-byte alignment.  With T == 0 there is nothing to sum: dw is set to
// zero (left as it is when accumulate_dw != 0) and dx is not touched.
//
// Returns 0, a positive cudaError_t, or a negative code that vb_rmsnorm_bwd_static_strerror() explains:
//   -1  H is not a multiple of 8            -2  H exceeds VB_RMSNORM_BWD_STATIC_MAX_H
//   -3  T is negative                       -4  more devices than the per-device table holds
//   -5  a required pointer is null          -6  a pointer is not aligned as stated above
// The argument checks (-1 .. -6) run on the host before anything is launched.
//
// * No cudaMalloc / cudaFree / allocating library call is made, on the first call or later.
// * The first call on each device looks up the address of the built-in buffer (cudaGetSymbolAddress) and
//   remembers it.  That lookup is set-up work: make one call on every device you use before you begin any
//   stream capture on it.
// * Nothing in the buffer has to start at zero: each call first overwrites every element it later reads.
// * The buffer is one per device and shared by all callers.  Two calls that can overlap in time on the same
//   device (different streams, or different host threads on different streams) race on it and give wrong
//   dw; order them on one stream or with events.
int vb_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in,
                          void* dx, float* dw, int T, int H, int accumulate_dw, cudaStream_t stream);
const char* vb_rmsnorm_bwd_static_strerror(int code);
}
