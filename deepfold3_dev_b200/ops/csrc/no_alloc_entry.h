// C entry point that allocates nothing. It has no counterpart in the reference implementation; it
// exists so that a host runtime which must not touch any allocator (torch's caching allocator
// included) can still run the LayerNorm backward kernel.
//
// df3_layer_norm_bwd_noalloc computes, for x, dy of shape [rows, channels] (contiguous, bf16 or fp32):
//     dx[rows, channels]  gradient of the input (same element type as x)
//     dw[channels]        sum over rows of dy * xhat            (fp32; may be null together with db)
//     db[channels]        sum over rows of dy                   (fp32)
// from the saved fp32 statistics mean[rows], rstd[rows] and the optional fp32 weight w[channels].
//
// Scratch: the per-block partial sums of dw/db live in ONE file-scope __device__ array of fixed size
// (kNoAllocMaxBlocks x 2 x kNoAllocMaxChannels floats = 2.3 MiB per device). Consequences:
//   * channels above kNoAllocMaxChannels (1024) are rejected with kNoAllocBadSize; rows are unlimited.
//   * the first call on a device looks the array's address up (cudaGetSymbolAddress). Make that first
//     call before any stream capture begins on that device.
//   * every call on a device uses the same array: two calls that overlap in time (different streams
//     or threads) race on it. Serialise them on one stream.
//   * the caller must have made the buffers' device current (cudaSetDevice) before the call: the scratch array, the
//     launch and the stream all belong to the current device, and the function does not switch devices.
//   * nothing in the array has to start at zero: each launched block overwrites its own slice before
//     the reduction reads it.
// The function calls no cudaMalloc/cudaFree and no allocating library routine; all outputs are
// written into buffers the caller owns.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

enum {
  kNoAllocOk = 0,
  kNoAllocBadSize = -1,     // channels outside [1, kNoAllocMaxChannels] or rows < 0
  kNoAllocBadPointer = -2,  // a required pointer is null
  kNoAllocBadDevice = -3,   // device ordinal beyond the table of cached scratch addresses
  // positive values are cudaError_t codes from set-up or launch
};

#define DF3_NO_ALLOC_MAX_CHANNELS 1024
#define DF3_NO_ALLOC_MAX_BLOCKS 296

// is_bf16: 1 when dy/x/dx hold bf16, 0 for fp32. stream: a cudaStream_t (null = default stream).
// Returns kNoAllocOk, a negative code above, or a positive cudaError_t.
int df3_layer_norm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* mean, const float* rstd,
                               void* dx, float* dw, float* db, long long rows, int channels, int is_bf16,
                               void* stream);

// Text of the last error returned on the calling thread ("" when none).
const char* df3_no_alloc_last_error(void);

#ifdef __cplusplus
}
#endif
