// An entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference project: it exists for hosts that embed the kernel
// library directly through its C interface and cannot call cudaMalloc where they run it:
// for example a serving loop that has handed the whole device to a fixed memory plan, a
// plug-in that lives inside someone else's process and allocator, or code running at a point
// where an allocation would synchronise the device.  Such a caller still owns its inputs and
// outputs, but it has nowhere to take the split-KV decode kernel's scratch memory from.
//
// fe_paged_decode_mma_static is fe_paged_decode_mma with that scratch memory (the partial
// outputs and log-sum-exps of the key splits) taken from a fixed array inside the library
// instead of from the caller.
//
//   * The array is FE_STATIC_SCRATCH_BYTES (8 MiB) of device memory; every GPU on which the
//     library is loaded holds it until the process exits.  A call that would need more
//     (requests * nq * splits * (d + 1) * 4 bytes) is refused with an error, nothing is launched.
//   * The function calls no cudaMalloc, cudaFree or other allocating routine.
//   * The first call on a device looks up the array's device address (once per device, with
//     that device current).  Make that first call outside any stream capture.
//   * Every call on a device uses the same array.  Nothing in it has to start at zero (each
//     split writes its slot before the merge reads it) and nothing is kept for the next call, but
//     two calls that overlap on the GPU (different streams) would overwrite each other's
//     partial results: keep calls on one stream, or order them yourself.
//
// Arguments and return value are those of fe_paged_decode_mma, without ``scratch``:
// 0 on success; otherwise fe_last_error() holds the reason.
#pragma once

#include <cuda_runtime.h>

#define FE_STATIC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int fe_paged_decode_mma_static(const void* q, long long q_stride, void* out, long long out_stride, const void* kc,
                               const void* vc, const int* block_table, int bt_stride, const int* cu_q,
                               const int* q_start, int requests, int nq, int nkv, int d, int ps, int num_pages,
                               float scale, int window, int splits, int* status, cudaStream_t stream);

// The size of the built-in scratch array, for callers that want to size their batches to it.
long long fe_static_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
