// An entry point for callers that must not allocate device memory.
//
// This function has no counterpart in the reference project: it exists for users of this
// library whose process cannot call cudaMalloc when it wants a result.  Two kinds of caller are
// meant.  One has handed all device memory to an allocator of its own at start-up (a serving
// process with a fixed memory plan, a host framework that owns the pool) and has no way to ask
// this library's usual helpers for a scratch buffer.  The other sits in a latency-critical loop
// where cudaMalloc or cudaFree would stall the whole device behind an implicit synchronisation.
// Both still own their inputs and outputs and pass them in; only the scratch is ours.
//
// mg_argmax_wide_noalloc computes what mg_argmax_wide computes (per row of 32-bit logits, the
// lowest index among the largest values, ids >= limit excluded), but keeps the intermediate
// per-slice maxima in a fixed array that is part of the loaded library instead of in scratch
// buffers passed by the caller.
//
//  * Limit: rows * ceil(vocab / 2048) <= MG_NOALLOC_MAX_PARTS (8192 slice results).  That is
//    256 rows of a 50304-wide vocabulary, or 64 rows of a 262144-wide one.  Larger requests are
//    refused with MG_ERR_ARG and a message from mg_last_error(); nothing is launched.
//  * Cost: 64 KiB of device memory on every GPU that loads the library, held until exit.
//  * It calls no cudaMalloc, cudaFree, or any routine that allocates (none of torch's either).
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and remembers it; make that first call outside any stream capture.
//  * All calls on a device share the one array.  The kernel overwrites every slot it later
//    reads, so nothing has to be cleared between calls, but two calls that overlap on the GPU
//    (different streams, no ordering between them) race on it: order them.
#pragma once

#define MG_NOALLOC_MAX_PARTS 8192

#ifdef __cplusplus
extern "C" {
#endif

// logits: [rows, vocab] float32 on the current device; out: [rows] int32; limit <= 0 means the
// whole vocabulary; stream: a cudaStream_t of the current device.  Returns 0 on success.
int mg_argmax_wide_noalloc(const float* logits, int* out, int rows, int vocab, int limit, void* stream);

#ifdef __cplusplus
}
#endif
