// Routing top-k for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (which has no router at all). It exists
// for hosts that drive the library from contexts where cudaMalloc is off limits: a serving loop
// that has handed every byte of the device to its own pool, a real-time thread that may not take
// the allocator's locks, or code running while allocation is frozen. Such callers pass their own
// input and output buffers; the intermediate histogram and rank tables live in a fixed array
// inside the library image instead of in memory obtained at call time.
//
// Limits (checked, see fastb_route_topk_noalloc_limits): at most 16384 tokens, 256 experts,
// top-8. The array costs 640 KiB on every GPU that loads the library, until the process exits.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// logits [T, E] fp32 (device), bias [E] fp32 (device) or NULL,
// topk_idx [T, K] int32 (out), topk_w [T, K] fp32 (out), expert_counts [E] int32 (out: tokens
// routed to each expert). `stream` is a cudaStream_t. Returns 0 on success, else a cudaError_t
// value; fastb_noalloc_last_error() then describes what was refused.
//
// The first call on each device looks up the device address of the internal array (no allocation,
// but a runtime query): make that first call outside any stream capture. All calls on one device
// share the array, so two calls whose kernels may overlap on the GPU (different streams without
// an ordering between them) race on it; calls on one stream are safe. The array keeps whatever
// the previous call left; this routine reads no word it has not written in the same call.
// Host threads: the function may be called from several threads at once (the per-device address
// cache is atomic and the error text is per thread); the device-side race above still applies to
// their kernels unless their streams are ordered.
int fastb_route_topk_noalloc(const float* logits, const float* bias, int T, int E, int K, int* topk_idx, float* topk_w, int* expert_counts,
                             void* stream);

// Writes the maxima accepted above.
void fastb_route_topk_noalloc_limits(int* max_tokens, int* max_experts, int* max_top_k);

// Message of the last refusal on the calling thread ("" if none).
const char* fastb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
