// Allocation-free entry point of the fused LM head: same kernels as prb_lmhead_fwd
// (gemm.cu), scratch in a fixed device array of this translation unit. See prb_noalloc.h
// for who needs it, the limits and the rules of use.
#include "common.cuh"
#include "prb_noalloc.h"
#include <stdio.h>

#include <atomic>

extern "C" int prb_lmhead_num_splits(int T, int V);
extern "C" int prb_lmhead_fwd(const void* h, const void* W, const int* labels, const float* inv_temp, float* part_m,
                              float* part_s, float* part_t, float* target, float* logprob, float* entropy,
                              float* lse, int T, int V, int H, long long ldh, long long ldw, int splits, int* status,
                              void* stream_);

namespace prb {
// part_m | part_s | part_t : [PRB_NOALLOC_MAX_SPLITS, PRB_NOALLOC_MAX_TOKENS] each, then target [MAX_TOKENS]
constexpr size_t kNoAllocPart = static_cast<size_t>(PRB_NOALLOC_MAX_SPLITS) * PRB_NOALLOC_MAX_TOKENS;
static __device__ __align__(256) float g_lmhead_scratch[3 * kNoAllocPart + PRB_NOALLOC_MAX_TOKENS];

// Device address of the scratch array on the current device. In host code the array's name
// is only a stand-in for the symbol, so the address is asked from the runtime once per device.
static float* noalloc_scratch_ptr(int* rc) {
  static std::atomic<float*> ptrs[64];      // zero-initialised; host threads may race to fill a slot with the same value
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *rc = -21; return nullptr; }
  float* p = ptrs[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_lmhead_scratch) != cudaSuccess || p == nullptr) {
      *rc = -22;
      return nullptr;
    }
    ptrs[dev].store(p, std::memory_order_release);
  }
  *rc = 0;
  return p;
}
}  // namespace prb

PRB_API int prb_lmhead_fwd_noalloc(const void* h, const void* W, const int* labels, const float* inv_temp,
                                   float* logprob, float* entropy, float* lse, int T, int V, int H, long long ldh,
                                   long long ldw, int* status, void* stream) {
  using namespace prb;
  if (T <= 0) return 0;
  if (T > PRB_NOALLOC_MAX_TOKENS) {
    fprintf(stderr, "prb_lmhead_fwd_noalloc: T = %d exceeds the built-in scratch (%d rows); use prb_lmhead_fwd\n", T,
            PRB_NOALLOC_MAX_TOKENS);
    return PRB_NOALLOC_TOO_LARGE;
  }
  int rc = 0;
  float* scratch = noalloc_scratch_ptr(&rc);
  if (scratch == nullptr) return rc;
  int splits = prb_lmhead_num_splits(T, V);
  if (splits > PRB_NOALLOC_MAX_SPLITS) {
    // Fewer slices than the scheduler would like: spread the 256-column vocabulary tiles again so
    // that no slice is empty. An empty slice writes no partial row, and the merge kernel would
    // then read what an earlier call left in the shared array.
    const int tiles_n = (V + 255) / 256;
    const int per = (tiles_n + PRB_NOALLOC_MAX_SPLITS - 1) / PRB_NOALLOC_MAX_SPLITS;
    splits = (tiles_n + per - 1) / per;
  }
  // the partial arrays are fully overwritten for rows < T and slices < `splits`; the target
  // logit array is the part that must start at zero (prb_lmhead_fwd clears it)
  float* part_m = scratch;
  float* part_s = scratch + kNoAllocPart;
  float* part_t = scratch + 2 * kNoAllocPart;
  float* target = scratch + 3 * kNoAllocPart;
  return prb_lmhead_fwd(h, W, labels, inv_temp, part_m, part_s, part_t, target, logprob, entropy, lse, T, V, H, ldh,
                        ldw, splits, status, stream);
}
