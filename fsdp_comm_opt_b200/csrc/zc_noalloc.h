// Allocation-free entry point of the v1 split-layout encoder.
//
// This declaration has no counterpart in the reference: there every compress call is surrounded by
// fresh torch allocations for its scratch and outputs.
//
// Who needs it.  zc_v1_encode_split() asks its caller for a scratch buffer of one byte per padded
// element.  Some callers of this library cannot get one at call time:
//   * comm hooks that run on FSDP's side streams while the framework's caching allocator already
//     owns almost all of HBM -- a raw cudaMalloc there either fails or makes the allocator flush
//     its cache, which synchronises the device and serialises the streams the hook is meant to
//     overlap;
//   * latency-critical loops that must not call cudaMalloc / cudaFree at all because those calls
//     synchronise the device.
// For them the scratch lives inside the library: a file-scope `static __device__` array of
// ZC_NOALLOC_MAX_ELEMS bytes (16 MiB).  Every GPU whose context loads the library holds that array
// until the process exits.
//
// Contract.
//   * Same inputs and outputs as zc_v1_encode_split(), minus the scratch pointer; the bytes written
//     to `det`, `esc_final` and `counts` are identical to that entry point's.
//   * Every n_8[i] (device memory) must be a multiple of 4096 and total_blocks must equal
//     sum(n_8) / 4096: block b stages its outliers at scratch offset 4096 * b, so with whole blocks
//     per work the staging never leaves the first total_blocks * 4096 bytes of the array.
//   * total_blocks * 4096 must not exceed ZC_NOALLOC_MAX_ELEMS; larger requests are refused with
//     ZC_ERR_TOO_LARGE and a message on stderr, nothing is launched.
//   * Return value: 0 on success (also for total_blocks <= 0: nothing to do); -1 for n_works <= 0;
//     ZC_ERR_TOO_LARGE (-3); ZC_ERR_SYMBOL (-4) when the array's device address cannot be resolved;
//     a positive cudaError_t when a launch was refused.
//   * The call allocates nothing: no cudaMalloc, cudaFree or any allocating library routine.
//   * First call on a device: it resolves the device address of the scratch array once (with that
//     device current) and caches it.  Make that first call before any stream capture begins.
//   * All calls on a device share the one array, and it keeps whatever the previous call left in
//     it.  Nothing in it has to start at zero: the compaction pass reads only the bytes that the
//     encode pass of the same call wrote.  Two calls that overlap on the GPU (different streams
//     without an ordering between them) race on the array; order them.
#pragma once
#include <cuda_runtime.h>

#define ZC_NOALLOC_MAX_ELEMS (16ll * 1024 * 1024)
#define ZC_ERR_TOO_LARGE (-3)
#define ZC_ERR_SYMBOL (-4)

#ifdef __cplusplus
extern "C" {
#endif

int zc_v1_encode_split_noalloc(const void* in, long long total_n, const int* n_8, const int* orig_n, int n_works,
                               const int* bases, void* det, void* esc_final, int* counts, long long total_blocks,
                               cudaStream_t stream);

#ifdef __cplusplus
}
#endif
