// Greedy-token selection for callers that may not allocate device memory.
//
// This entry point has no counterpart in the reference runtime; it exists for hosts of this
// library that fix their device-memory layout at start-up and then forbid allocation: a serving
// process whose memory is fully divided into weight, KV-page and arena budgets, a caller that
// cannot tolerate the device-wide synchronisation cudaMalloc/cudaFree imply while other streams
// are decoding, or an embedding application that simply owns no allocator it may call.  Such a
// caller passes only its input (the logits) and its outputs; the scratch space the two-level
// arg-max needs lives in a fixed array inside the library image.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Limits of the built-in scratch area (about 132 KB of device memory, held by every GPU that
// loads the library until the process exits).
#define FB_NOALLOC_ARGMAX_MAX_ROWS 256
#define FB_NOALLOC_ARGMAX_CHUNKS 64

// out_id[r] = index of the largest finite logit of row r (ties -> lower index, -1 if none),
// out_val[r] = that logit (out_val may be NULL).  Same result as fb_argmax_chunked.
//
//   logits : device pointer, fp32 [rows, vocab], row pitch ldl elements (multiple of 4), 16-byte aligned
//   rows   : 1 .. FB_NOALLOC_ARGMAX_MAX_ROWS; more rows are refused with FB_ERR_LIMIT (nothing runs)
//   stream : CUDA stream (as void*) the work is enqueued on
//
// Returns FB_OK, FB_ERR_LIMIT (rows beyond the built-in scratch), FB_ERR_SHAPE / FB_ERR_ALIGN (bad
// arguments), FB_ERR_RUNTIME (the scratch symbol could not be resolved on this device) or
// FB_ERR_LAUNCH.
//
// The call never allocates: no cudaMalloc, cudaFree or allocating library routine.  The first call
// on each device resolves the device address of the scratch array (cudaGetSymbolAddress, with that
// device current); make that first call before starting any stream capture.  All calls on a device
// share the one scratch array, which keeps the previous call's contents: the per-row counters are
// cleared on the stream at the start of every call, everything else is overwritten before it is
// read.  Two calls that overlap on the GPU (different streams without an ordering between them)
// race on the scratch and give undefined results; order them.
int fb_argmax_noalloc(const float* logits, long long ldl, int rows, int vocab, int* out_id,
                      float* out_val, void* stream);

#ifdef __cplusplus
}
#endif
