// Token sampling for the rollout engine in one pass over the logits (the un-truncated case:
// temperature only). One CTA per row: every thread streams its share of the vocabulary once and keeps
//   - the running (max, sum exp) of z = logit / T for the log-softmax normaliser, and
//   - the arg-max of z + g with g ~ Gumbel(0, 1) drawn from a counter-based generator, which IS a sample
//     from softmax(z) (Gumbel-max); rows with T <= 0 take the arg-max of z itself (greedy).
// Outputs the token and its log-probability log softmax(z)[token]. The PyTorch path this replaces
// makes five passes over [B, V] fp32 (scale, log-softmax, exp, multinomial, gather).
//
// Reference behaviour: vLLM's sampler with processed logprobs
// (packages/prime-rl-configs/src/prime_rl/configs/inference.py:602-654).
#include "common.cuh"

namespace prb {

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

// 32-bit finaliser (three multiplies) over the element index mixed with a per-row seed: enough for 24 random bits
// per element, and a third of the instructions of the 64-bit hash above.
__device__ __forceinline__ unsigned mix32(unsigned x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}

struct SampleState {
  float m, s;        // running max and sum of exp(z - m)
  float key, z;      // best perturbed score and the unperturbed z of that token
  int idx;
};

__device__ __forceinline__ SampleState sample_merge(const SampleState& a, const SampleState& b) {
  SampleState r;
  r.m = fmaxf(a.m, b.m);
  r.s = (a.m == -INFINITY ? 0.f : a.s * __expf(a.m - r.m)) + (b.m == -INFINITY ? 0.f : b.s * __expf(b.m - r.m));
  const bool take_b = b.key > a.key || (b.key == a.key && b.idx < a.idx && b.idx >= 0);
  r.key = take_b ? b.key : a.key;
  r.z = take_b ? b.z : a.z;
  r.idx = take_b ? b.idx : a.idx;
  return r;
}

__global__ void __launch_bounds__(1024)
sample_gumbel_kernel(const float* __restrict__ logits, const float* __restrict__ temperature, long long ld,
                     unsigned long long seed, int* __restrict__ tokens, float* __restrict__ logprobs, int V) {
  const int row = blockIdx.x;
  const float T = temperature[row];
  const bool greedy = T <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / T;
  const float* z_row = logits + static_cast<long long>(row) * ld;
  const unsigned long long base = splitmix64(seed ^ (0x51ed270b0f3a9d1bull * (row + 1)));
  SampleState st{-INFINITY, 0.f, -INFINITY, 0.f, -1};
  const unsigned row_key = static_cast<unsigned>(base) ^ static_cast<unsigned>(base >> 32);
  auto take = [&](float z, int i) {
    float key = z;
    if (!greedy) {
      // 24 random bits -> u in (0, 1), g = -log(-log(u))
      const unsigned h = mix32(static_cast<unsigned>(i) * 0x9e3779b1u ^ row_key);
      const float u = (static_cast<float>(h >> 8) + 0.5f) * (1.f / 16777216.f);
      key = z - __logf(-__logf(u));
    }
    if (key > st.key) {
      st.key = key;
      st.z = z;
      st.idx = i;
    }
  };
  // rows whose start is 16-byte aligned are read four elements at a time; the log-sum-exp is updated once per group
  const bool vec = (reinterpret_cast<uintptr_t>(z_row) & 15) == 0;
  const int v4 = vec ? V / 4 : 0;
  for (int g4 = threadIdx.x; g4 < v4; g4 += blockDim.x) {
    const float4 q = reinterpret_cast<const float4*>(z_row)[g4];
    const float z0 = q.x * inv_t, z1 = q.y * inv_t, z2 = q.z * inv_t, z3 = q.w * inv_t;
    const float gm = fmaxf(fmaxf(z0, z1), fmaxf(z2, z3));
    if (gm > st.m) {
      st.s *= __expf(st.m - gm);                  // exp(-inf) = 0 on the first group
      st.m = gm;
    }
    if (gm > -INFINITY)                            // a group of -inf logits adds nothing (and -inf - -inf is NaN)
      st.s += __expf(z0 - st.m) + __expf(z1 - st.m) + __expf(z2 - st.m) + __expf(z3 - st.m);
    const int i = g4 * 4;
    take(z0, i); take(z1, i + 1); take(z2, i + 2); take(z3, i + 3);
  }
  for (int i = v4 * 4 + threadIdx.x; i < V; i += blockDim.x) {
    const float z = z_row[i] * inv_t;
    if (z > st.m) {
      st.s = st.s * __expf(st.m - z) + 1.f;
      st.m = z;
    } else if (z > -INFINITY) {
      st.s += __expf(z - st.m);
    }
    take(z, i);
  }
  // warp, then block reduction
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    SampleState other;
    other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, st.s, o);
    other.key = __shfl_xor_sync(0xffffffffu, st.key, o);
    other.z = __shfl_xor_sync(0xffffffffu, st.z, o);
    other.idx = __shfl_xor_sync(0xffffffffu, st.idx, o);
    st = sample_merge(st, other);
  }
  __shared__ SampleState part[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) part[warp] = st;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    st = lane < nw ? part[lane] : SampleState{-INFINITY, 0.f, -INFINITY, 0.f, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      SampleState other;
      other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
      other.s = __shfl_xor_sync(0xffffffffu, st.s, o);
      other.key = __shfl_xor_sync(0xffffffffu, st.key, o);
      other.z = __shfl_xor_sync(0xffffffffu, st.z, o);
      other.idx = __shfl_xor_sync(0xffffffffu, st.idx, o);
      st = sample_merge(st, other);
    }
    if (lane == 0) {
      tokens[row] = st.idx;
      logprobs[row] = st.z - (st.m + __logf(st.s));
    }
  }
}

}  // namespace prb

// logits fp32 [B, V] (row pitch ld), temperature fp32 [B] (<= 0: greedy), tokens int32 [B], logprobs fp32 [B].
PRB_API int prb_sample_gumbel(const float* logits, const float* temperature, long long ld, unsigned long long seed,
                              int* tokens, float* logprobs, int B, int V, void* stream) {
  if (B <= 0) return 0;
  if (V <= 0) return -3;
  prb::sample_gumbel_kernel<<<B, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(logits, temperature, ld, seed, tokens,
                                                                                  logprobs, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
