// b200_plan_noalloc -- dispatch plan for callers that must not allocate.
//
// This entry point has no counterpart in the reference project.
//
// Who needs it: code that runs where device allocation is off limits -- inside
// a serving loop that pre-sized all of its memory, under a framework whose
// allocator must not be re-entered (a custom-op callback, a memory-pool hook),
// or in a process that hands this library raw buffers and has no allocator to
// offer for temporaries.  The regular entry point, b200_plan, needs a
// caller-provided temporary (one int per routed copy, `rank_in_bucket`); here
// that temporary lives in a fixed array inside the library instead.
//
// What it does: the same two kernels as b200_plan.  From topk_idx (n_flat
// global expert ids, token-major then slot) it writes
//   counts       [num_experts]      routed copies per expert
//   bucket_start [num_experts + 1]  exclusive scan of counts
//   send_order   [n_flat]           flat (token*k+slot) ids sorted by expert, stable
//   dst_slot     [n_flat]           inverse of send_order (may be null)
// The caller passes inputs and outputs only.
//
// Limit: n_flat <= B200_PLAN_NOALLOC_MAX (1 048 576 routed copies, a 4 MiB
// array).  Every GPU that loads the library holds those 4 MiB until the
// process exits.  Larger inputs are rejected with B200_PLAN_NOALLOC_TOO_LARGE
// before anything is launched.
//
// Rules of use:
//  * The call allocates nothing: no cudaMalloc / cudaFree, no allocating
//    library routine, no PyTorch allocator.
//  * The first call on each device looks up the array's device address (once
//    per device, with that device current) and caches it.  Make that first call
//    outside any stream capture.  Host threads may make it concurrently.  The
//    cached address belongs to the device's primary context: after a
//    cudaDeviceReset() the library must be reloaded before this entry point is
//    used again on that device.
//  * All calls on one device share the one array.  Its contents after a call
//    are whatever that call left; nothing in it has to be zero on entry,
//    because each call writes every element before reading it.  Two calls
//    whose kernels overlap on the GPU (different streams, no dependency
//    between them) race on the array: order them.
#pragma once

#define B200_PLAN_NOALLOC_MAX (1 << 20)
#define B200_PLAN_NOALLOC_TOO_LARGE (-20)
#define B200_PLAN_NOALLOC_BAD_ARG (-21)
#define B200_PLAN_NOALLOC_NO_DEVICE (-22)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, one of the negative codes above, or a positive cudaError_t.
// All pointers are device pointers on the current device; `stream` is a
// cudaStream_t (null = default stream).
int b200_plan_noalloc(const int* topk_idx, int n_flat, int num_experts, int* counts,
                      int* bucket_start, int* send_order, int* dst_slot, void* stream);

// Largest n_flat the entry point accepts.
int b200_plan_noalloc_max(void);

#ifdef __cplusplus
}
#endif
