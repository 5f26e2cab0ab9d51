// Allocation-free entry point.  It has no counterpart in the reference (which is pure Python on top of
// PyTorch's allocator); it exists for embedders of this library that are not allowed to allocate device memory.
//
// Who that is: a host program whose device memory is handed out once at start-up by its own pool (a serving
// runtime, a plugin loaded into another framework, a process running under a fixed memory budget).  Such a caller
// can pass in the buffers it already owns, but it cannot let a library call cudaMalloc / cudaFree on its behalf:
// those calls take memory the pool does not know about and they synchronise the whole device.
//
// rtp_linear_bwd_noalloc computes the backward pass of one (single-rank) linear layer y = x W^T + b exactly like
// rtp_linear_bwd, but the scratch memory that path gets from its callers' allocators (the kernel's flag/status
// block and the fp32 column sums of dy that feed the bias gradient) lives in a fixed array inside the library.
//
// Limits and rules:
//   * out_features <= RTP_NOALLOC_MAX_OUT_FEATURES, else the call fails with a clear error and launches nothing.
//     The array costs RTP_NOALLOC_SCRATCH_BYTES (320 KB) of device memory on every GPU that loads the
//     library, from load until the process exits.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, cached per device) and
//     raises the kernel's shared-memory limit on that device (also kept per device).  Make that first call before
//     starting any stream capture.
//   * Every call reuses the same array and the array keeps the previous call's contents; the entry point clears
//     the parts that must start at zero.  Two calls that overlap on the GPU (different streams, no ordering) race
//     on it: order them on one stream or with events.
//   * The kernel's waits are bounded; one that runs out leaves a non-zero code in a status word that also lives in
//     the array.  The entry point returns before the kernel has run, so poll rtp_noalloc_status after the work (it
//     copies the word to the host and synchronises the stream; it allocates nothing either).  The next call clears
//     the word.
//   * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.  Inputs and outputs are the
//     caller's buffers: x [M, in], dy [M, out], w = flat shard (weight [out, in], bias at element bias_off or -1),
//     dx [M, in] (may be null), grad_flat (same layout as w).  All bf16, 16-byte aligned, row pitches in elements.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#define RTP_NOALLOC_MAX_OUT_FEATURES 65536
#define RTP_NOALLOC_SCRATCH_BYTES (65536 + 4 * RTP_NOALLOC_MAX_OUT_FEATURES)   /* flag block (RTP_FLAG_BYTES) + column sums */

int rtp_linear_bwd_noalloc(const void* x, long long ldx, const void* dy, long long ldy, const void* w,
                           long long bias_off, int M, int in_features, int out_features, void* dx, long long lddx,
                           void* grad_flat, void* stream);
// Copies the status word of the last rtp_linear_bwd_noalloc call on the current device into *host_out (0 = ok, else
// the code of the first bounded wait that ran out) and synchronises `stream`.
int rtp_noalloc_status(void* stream, unsigned long long* host_out);
const char* rtp_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
