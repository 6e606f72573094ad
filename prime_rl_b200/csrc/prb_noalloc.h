// Allocation-free entry point of the fused LM head (no counterpart in the reference).
//
// For callers that must not, or cannot, allocate device memory at call time: a worker that
// has already handed every free byte of the GPU to its KV-cache pool (any later cudaMalloc
// fails or fragments), a host program that reaches this library through the bare C ABI and
// has no tensor allocator at hand, or a latency-critical path that is not allowed to enter
// the driver's allocator. The regular entry point (prb_lmhead_fwd) asks the caller for
// scratch buffers sized from T and V; this one keeps its scratch in a fixed array inside the
// library image instead.
//
// Limits and rules
//   * T <= PRB_NOALLOC_MAX_TOKENS rows per call; the vocabulary is cut into at most
//     PRB_NOALLOC_MAX_SPLITS slices. Larger T is rejected with PRB_NOALLOC_TOO_LARGE and
//     nothing is launched.
//   * The scratch array (about 6.3 MB) exists once per GPU that loads the library and stays
//     until the process exits.
//   * All calls on a device share it and it keeps what the last call left there; the entry
//     point clears the part that has to start at zero. Two calls that overlap on the GPU
//     (different streams) race on it: keep calls on one device in stream order.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and sets a kernel attribute; make that
//     first call before starting any stream capture.
//   * No cudaMalloc / cudaFree / allocating library routine is called. Inputs and outputs are
//     the caller's device buffers, exactly as for prb_lmhead_fwd.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define PRB_NOALLOC_MAX_TOKENS 8192
#define PRB_NOALLOC_MAX_SPLITS 64
#define PRB_NOALLOC_TOO_LARGE (-20)

// h: bf16 [T, H] (row pitch ldh elements); W: bf16 [V, H] (pitch ldw); labels: int32 [T] (ids
// outside [0, V) give logprob 0); inv_temp: fp32 [T] or NULL. Outputs, fp32 [T] each: logprob,
// entropy, lse. status: device int that receives a non-zero code if a bounded wait inside the
// kernel ran out. Returns 0 when the work was enqueued on `stream`.
int prb_lmhead_fwd_noalloc(const void* h, const void* W, const int* labels, const float* inv_temp, float* logprob,
                           float* entropy, float* lse, int T, int V, int H, long long ldh, long long ldw,
                           int* status, void* stream);

#ifdef __cplusplus
}
#endif
