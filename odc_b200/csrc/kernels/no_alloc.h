// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for users of this library
// whose code runs where cudaMalloc is off limits: inside a framework that hands out one fixed
// arena up front, inside a latency-critical loop where an allocation would synchronise the
// device, or in a process whose memory budget is fully pre-planned.  The regular path
// (launch_rmsnorm_bwd in api.h) needs a [CTAs, cols] fp32 workspace that its caller allocates;
// this variant keeps that workspace in a fixed array that is part of the library image.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest row width accepted, and the size of the built-in workspace that follows from it.
#define ODC_NOALLOC_MAX_COLS 8192
#define ODC_NOALLOC_MAX_CTAS 148
#define ODC_NOALLOC_SCRATCH_BYTES (ODC_NOALLOC_MAX_CTAS * ODC_NOALLOC_MAX_COLS * 4) /* 4.6 MiB per GPU */

// dx[rows, cols] (bf16) and dw[cols] (fp32) from dy, x (bf16 [rows, cols]), w (bf16 [cols]) and
// rstd (fp32 [rows], as produced by the forward pass).  All pointers are device memory owned by
// the caller; `stream` is a cudaStream_t.  Returns 0 on success; otherwise a non-zero code and a
// message in `err` (if err_len > 0).  Requirements: cols a multiple of 8 and at most
// ODC_NOALLOC_MAX_COLS (larger widths are refused, nothing is launched); rows >= 0; dy, x, w and dx
// 16-byte aligned, rstd and dw 4-byte aligned (a misaligned pointer is refused with an error code,
// nothing is launched).
//
// * No device memory is allocated or freed, by this function or by anything it calls.  (The CUDA
//   runtime may still load this library's GPU code on the first launch in a process; that is the
//   runtime's own one-time work, not a per-call allocation.)
// * The workspace is one array shared by every call on a GPU; each GPU that loads the library
//   holds ODC_NOALLOC_SCRATCH_BYTES of it until the process exits.  Every call overwrites the
//   part it reads, so nothing needs clearing between calls, but two calls that overlap on the
//   same GPU (different streams, or different threads) race on it: serialise them.
// * The first call on each GPU looks up the workspace's device address (with that GPU current)
//   and remembers it; make that first call before starting any stream capture.
int odc_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                            int rows, int cols, void* stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
