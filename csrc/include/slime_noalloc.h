// Batched copy for callers that must not allocate.
//
// This entry point has no counterpart in the reference. It exists for hosts that embed the
// library where the CUDA allocator is off limits at call time: a serving process that has
// handed its whole memory budget to its own pool and treats any later cudaMalloc as a bug,
// a plug-in running inside a framework that forbids allocation on the request path, a
// tool started with almost no free device memory. The regular batched transfer
// (slime_nvlink_ep_transfer) keeps a per-endpoint staging table and counters that it
// allocates on first use; this variant keeps the same bookkeeping in a fixed array that is
// part of the library image instead.
//
//   slime_copy_batch_noalloc(dst, src, len, n, stream)
//     dst, src  host arrays of n device addresses (destination / source of each segment;
//               peer-mapped addresses are fine)
//     len       host array of n byte counts
//     n         0 .. SLIME_NOALLOC_MAX_SEGMENTS
//     stream    cudaStream_t as void*
//   Returns 0 on success, a negative value otherwise (slime_last_error() has the text).
//   A batch larger than SLIME_NOALLOC_MAX_SEGMENTS is refused; split it and call again.
//
// What a caller needs to know:
//  * Nothing is allocated: no cudaMalloc / cudaFree, no pinned-memory allocation, no library
//    routine that allocates. The price is SLIME_NOALLOC_SCRATCH_BYTES of device memory on
//    every GPU that loads the library, held until the process exits.
//  * The first call on each device looks up the device address of that array (one query,
//    cached per device). Make that first call during start-up, outside any stream capture.
//  * The segment table is built from the caller's host arrays while the call runs and copied
//    to the device with ordinary asynchronous copies from pageable memory, which have finished
//    reading their source when the call returns. For the same reason a stream that is being
//    captured is refused with an error.
//  * Zero-length segments are allowed anywhere in the batch and move nothing.
//  * Every call on a device uses the same array. Calls whose kernels could overlap on the
//    GPU (different streams, no ordering between them) would overwrite each other's table:
//    issue them on one stream, or order them with events.
#pragma once

#define SLIME_NOALLOC_MAX_SEGMENTS 4096
// 32 bytes per table entry plus one 256-byte block for counters
#define SLIME_NOALLOC_SCRATCH_BYTES (SLIME_NOALLOC_MAX_SEGMENTS * 32 + 256)

#ifdef __cplusplus
extern "C" {
#endif

int slime_copy_batch_noalloc(const unsigned long long* dst, const unsigned long long* src, const unsigned long long* len,
                             int n, void* stream);
int slime_copy_batch_noalloc_max_segments(void);

#ifdef __cplusplus
}
#endif
