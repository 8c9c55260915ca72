// Allocation-free INT4 matrix-vector product.
//
// This entry point has no counterpart in the reference: it exists for callers of this
// library that are not allowed to allocate device memory at the point where they need a
// projection -- a plug-in running inside another runtime's callback that forbids
// cudaMalloc/cudaFree (they synchronise the device and may dead-lock against the host
// runtime's own allocator lock), a service that must stay inside a memory budget fixed at
// start-up, or code on a latency path where an implicit device synchronisation is not
// acceptable.  The regular entry point (b2_gemv_int4) expects the caller to bring a
// scratch buffer for the split-K partial sums and arrival counters; this one brings its
// own, a fixed block of B2_NOALLOC_SCRATCH_BYTES that lives in the library image on every
// GPU that loads the library, from load until the process exits.
//
// What it computes: out[r][n] = sum_k x[r][k] * W[k][n] for r < rows, fp16 in / fp16 out,
// fp32 accumulation, W given in this library's packed fragment layout
// (mi50grad_b200/ops/packing.py: qfrag, szfrag).  The caller passes inputs and outputs only.
//
// Rules:
//  * It calls no cudaMalloc, cudaFree or any allocating library routine.
//  * The first call on a device looks up the device address of the built-in scratch block
//    (once per device, with that device current).  Make that first call outside any stream
//    capture.
//  * Problem sizes whose split-K partials or counters do not fit in the block are refused
//    with B2_NOALLOC_ERR_TOO_LARGE; nothing is launched.
//  * Alignment: x must be 4-byte aligned and ldx even (activations are read as fp16 pairs), out
//    2-byte aligned, qfrag 16-byte and szfrag 8-byte aligned (tensors from any CUDA allocator
//    are).  Anything else is refused with B2_NOALLOC_ERR_BAD_ARGUMENT before a launch: a misaligned
//    device access would otherwise fault and leave the context unusable.
//  * The first call on each device of a process also opts the kernel in to its shared-memory size
//    on that device; calls from several threads are serialised for that step.
//  * All calls share the one block.  The arrival counters are cleared in stream order at
//    the start of every call; the partial sums are fully overwritten before they are read.
//    Two calls that overlap on the GPU (different streams, or graphs replayed
//    concurrently) race on the block: serialise them.
#pragma once
#include <cuda_runtime.h>

#define B2_NOALLOC_SCRATCH_BYTES (4u << 20)   // 4 MiB per GPU, of which the first 4 KiB are counters

#define B2_NOALLOC_OK 0
#define B2_NOALLOC_ERR_BAD_ARGUMENT (-1)      // null pointer, rows outside 1..8, K % 8, unsupported group size, misalignment
#define B2_NOALLOC_ERR_TOO_LARGE (-2)         // needs more scratch than B2_NOALLOC_SCRATCH_BYTES
#define B2_NOALLOC_ERR_SYMBOL (-3)            // the scratch block's device address could not be obtained
// positive return values are cudaError_t codes from the launch

#ifdef __cplusplus
extern "C" {
#endif

// qfrag/szfrag: packed weights of a [K x N] projection (N = real outputs), x: [rows][ldx] fp16,
// out: [rows][ldo] fp16.  group_size in {32, 64, 128, 256}; group_offset: k-elements of the first
// quantisation group that precede row 0 (0 unless the matrix is a row shard), multiple of 32.
int b2_gemv_int4_noalloc(const void* qfrag, const void* szfrag, const void* x, int ldx, void* out, int ldo,
                         int rows, int K, int N, int group_size, int group_offset, cudaStream_t stream);

// Human-readable text for a return value of b2_gemv_int4_noalloc.
const char* b2_gemv_int4_noalloc_strerror(int code);

// Scratch bytes a problem needs (to check against B2_NOALLOC_SCRATCH_BYTES beforehand).
size_t b2_gemv_int4_noalloc_required(int rows, int K, int N);

#ifdef __cplusplus
}
#endif
