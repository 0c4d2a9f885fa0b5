// An entry point for callers that are not allowed to allocate.
//
// This function has no counterpart in the reference.  It exists for hosts of
// this library that must not call cudaMalloc (or anything that does) at the
// moment they need a reduction: code running while a CUDA graph is being
// captured elsewhere in the process, plugins living inside another runtime's
// memory budget, real-time loops where an allocation may stall behind the
// driver's lock.  Everything else in this library gets its staging memory from
// the engine at start-up; here the staging memory is a fixed array inside the
// library image.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Sums `world` fp32 buffers of `numel` elements element-wise and leaves the
// sum in every one of them (an all-reduce whose ranks are buffers on the
// current device), using the one-shot kernel with its staging, flags and
// bookkeeping placed in a static device array of about 1.3 MiB.  Every GPU
// that loads the library holds that array until the process exits.
//
//   bufs    host array of `world` device pointers (fp32, `numel` elements each,
//           on the current device -- checked; the buffers must not overlap)
//   world   2..8
//   numel   1..4096
//   stream  a cudaStream_t of the current device (0 for the default stream)
//   check   non-zero: wait for the stream and report a device-side time-out
//   err     optional buffer that receives a message when the call fails
//
// Returns 0 on success, 1 for a bad argument (too many buffers, too many
// elements, null pointer: nothing has been launched), 2 for a CUDA error and 3
// if `check` was set and a wait inside the kernel ran into its two-second limit.
//
// Calls no cudaMalloc/cudaFree and no allocating library routine.  The first
// call on a device looks up the address of the static array, writes the
// bookkeeping tables for every `world` from 2 to 8 into it and synchronises the
// stream; make that first call before any stream capture begins.  Every later
// call on that device, whatever its `world`, only clears the flags (a memset
// on the stream) and launches the kernel.
// All calls share the one array, and each call first clears the flags and
// counters in it: two calls whose kernels overlap on the GPU (different
// streams, no dependency) race with each other.  Issue them on one stream, or
// order them yourself.
int fairring_allreduce_f32_noalloc(float* const* bufs, int world, long long numel, void* stream,
                                   int check, char* err, unsigned long err_len);

#ifdef __cplusplus
}
#endif
