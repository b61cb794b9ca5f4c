// mynah_attn_decode_no_alloc: the decode attention for callers that must not
// allocate device memory. It has no counterpart in the reference, which keeps
// all of its working memory in host arrays made once at start-up.
//
// Who needs it: a process that has given all free device memory to a pool of
// its own (a serving process that sizes its cache to whatever the device has
// left has nothing for cudaMalloc to hand out), and a caller inside a loop
// with a latency bound, where an allocation would stall the whole device
// while the driver maps memory.
//
// Same arguments and same result as mynah_attn_decode, without the scratch
// pointer: the partial results of the page splits live in a fixed array
// inside the library instead (MYNAH_NO_ALLOC_SCRATCH_FLOATS floats, 16 MiB,
// held by every device that loads the library until the process exits).
//
//   * B * H * n_splits * (head_dim + 2) must not exceed
//     MYNAH_NO_ALLOC_SCRATCH_FLOATS; a larger problem is refused with an
//     error message, nothing is launched.
//   * The first call on each device looks the array's device address up
//     (one cudaGetSymbolAddress, no allocation). Make that first call before
//     any stream capture begins, and before the process hands the device's
//     free memory to a pool of its own: with CUDA's lazy module loading the
//     driver reserves the 16 MiB of the array when this file's code is first
//     used on a device, which is that first call, and a device with nothing
//     left makes it fail.
//   * The address is remembered per device ordinal for the life of the
//     process. It does not survive a cudaDeviceReset: do not call this entry
//     point again on a device that has been reset.
//   * All calls share the one array, and it keeps what the last call left in
//     it. The kernels write every partial result they later read, so nothing
//     has to be cleared between calls; but two calls that overlap on the
//     device (different streams, no ordering between them) race on it. Order
//     them on one stream or with events.
//   * It calls no cudaMalloc, cudaFree or any routine that allocates.
#pragma once

#include <cuda_runtime.h>

#define MYNAH_NO_ALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, or a negative code with the reason in mynah_last_error().
int mynah_attn_decode_no_alloc(
    const void* q, void* out, int dtype, int B, int H, int KV, int HD, int ldq, int ldo,
    const void* k_cache, const void* v_cache, const int* kv_len,
    const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
    int window, int n_splits, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
