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


// ---------------------------------------------------------------------------------------------------------
// Truncated sampling (top-k and / or top-p) without a sort. One CTA per row:
//   pass 0   max and sum of exp of z = logit / T (the softmax normaliser: top-p is a statement about probability)
//   4 passes radix descent over an order-preserving 32-bit key of z, 8 bits per pass: a 256-bin histogram of
//            (count, probability mass) of the elements that match the prefix found so far, then the lowest bin
//            whose elements can still be kept: fewer than k elements and less than p of the mass lie strictly
//            above it. After the fourth pass the prefix is the key of the smallest kept logit.
//   pass 5   Gumbel-max over the kept elements (key >= threshold), their normaliser for the reported
//            log-probability, and optionally their ids (unordered, at most mask_cap per row).
// A sorted-order rule "keep element i while the mass before it is below p and i < k" keeps exactly the elements at
// or above that threshold (elements equal to the threshold value are all kept). The row is read six times from
// the L2 (600 KB for a 152 k vocabulary) instead of being sorted through HBM.
__device__ __forceinline__ unsigned order_key(float z) {
  const unsigned u = __float_as_uint(z);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);       // larger float <=> larger key
}

__global__ void __launch_bounds__(1024)
sample_truncated_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                        const int* __restrict__ top_k, const float* __restrict__ top_p, long long ld,
                        unsigned long long seed, int* __restrict__ tokens, float* __restrict__ logprobs,
                        int* __restrict__ mask_ids, int* __restrict__ mask_count, int mask_cap, int V) {
  const int row = blockIdx.x;
  const float T = temperature[row];
  const bool greedy = T <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / T;
  const float* z_row = logits + static_cast<long long>(row) * ld;
  const int k_lim = (top_k[row] > 0 && top_k[row] < V) ? top_k[row] : V;
  const float p_lim = top_p[row];
  const bool use_p = p_lim < 1.f;
  __shared__ float red_a[32], red_b[32];
  __shared__ unsigned h_mass[256];          // probability mass per bin in fixed point (kMassScale = 1.0)
  __shared__ unsigned h_cnt[256];
  constexpr float kMassScale = 67108864.f;   // 2^26: the probabilities of a row add up to 1, so a bin fits 32 bits
  __shared__ unsigned s_prefix, s_cnt_above;
  __shared__ float s_mass_above, s_m, s_inv_sum;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;

  // ---- pass 0: max, then sum of exp
  float m = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, z_row[i] * inv_t);
  m = warp_max(m);
  if (lane == 0) red_a[warp] = m;
  __syncthreads();
  if (warp == 0) {
    m = lane < nw ? red_a[lane] : -INFINITY;
    m = warp_max(m);
    if (lane == 0) s_m = m;
  }
  __syncthreads();
  m = s_m;
  float sum = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) sum += __expf(z_row[i] * inv_t - m);
  sum = warp_sum(sum);
  if (lane == 0) red_b[warp] = sum;
  __syncthreads();
  if (warp == 0) {
    sum = lane < nw ? red_b[lane] : 0.f;
    sum = warp_sum(sum);
    if (lane == 0) {
      s_inv_sum = 1.f / sum;
      s_prefix = 0u;
      s_cnt_above = 0u;
      s_mass_above = 0.f;
    }
  }
  __syncthreads();
  const float inv_sum = s_inv_sum;

  // ---- radix descent
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int b = threadIdx.x; b < 256; b += blockDim.x) { h_mass[b] = 0u; h_cnt[b] = 0u; }
    __syncthreads();
    const unsigned prefix = s_prefix;
    // Logits crowd into a few bins (the first pass splits by sign and exponent), so lanes of a warp that hit the
    // same bin combine first (match + masked reduce) and one of them does the shared-memory atomics.
    for (int base = 0; base < V; base += blockDim.x) {
      const int i = base + threadIdx.x;
      unsigned bin = 0xffffffffu, fixed = 0u;
      if (i < V) {
        const float z = z_row[i] * inv_t;
        const unsigned key = order_key(z);
        if (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8))) {
          bin = (key >> shift) & 0xffu;
          if (use_p) fixed = __float2uint_rn(__expf(z - m) * inv_sum * kMassScale);
        }
      }
      const unsigned peers = __match_any_sync(0xffffffffu, bin);
      const unsigned msum = __reduce_add_sync(peers, fixed);
      if (bin != 0xffffffffu && lane == __ffs(peers) - 1) {
        atomicAdd(&h_cnt[bin], static_cast<unsigned>(__popc(peers)));
        if (use_p) atomicAdd(&h_mass[bin], msum);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned cnt = s_cnt_above;
      float mass = s_mass_above;
      int chosen = -1;
      unsigned chosen_cnt = cnt;
      float chosen_mass = mass;
      const float inv_scale = 1.f / kMassScale;
      for (int b = 255; b >= 0; --b) {
        if (h_cnt[b] == 0u) continue;
        if (cnt >= static_cast<unsigned>(k_lim) || (use_p && mass >= p_lim)) break;   // nothing at or below b is kept
        chosen = b;
        chosen_cnt = cnt;
        chosen_mass = mass;
        cnt += h_cnt[b];
        mass += static_cast<float>(h_mass[b]) * inv_scale;
      }
      if (chosen < 0) {                       // cannot happen (the top element is always kept); keep the top bin
        for (int b = 255; b >= 0; --b)
          if (h_cnt[b]) { chosen = b; break; }
      }
      s_prefix = prefix | (static_cast<unsigned>(chosen) << shift);
      s_cnt_above = chosen_cnt;
      s_mass_above = chosen_mass;
    }
    __syncthreads();
  }
  const unsigned thr = s_prefix;

  // ---- pass 5: sample among the kept
  const unsigned long long base = splitmix64(seed ^ (0x51ed270b0f3a9d1bull * (row + 1)));
  const unsigned row_key = static_cast<unsigned>(base) ^ static_cast<unsigned>(base >> 32);
  SampleState st{-INFINITY, 0.f, -INFINITY, 0.f, -1};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float z = z_row[i] * inv_t;
    if (order_key(z) < thr) continue;
    if (mask_ids != nullptr) {
      const int slot = atomicAdd(&mask_count[row], 1);
      if (slot < mask_cap) mask_ids[static_cast<long long>(row) * mask_cap + slot] = i;
    }
    if (z > st.m) {
      st.s = st.s * __expf(st.m - z) + 1.f;
      st.m = z;
    } else {
      st.s += __expf(z - st.m);
    }
    float key = z;
    if (!greedy) {
      const unsigned h = mix32(static_cast<unsigned>(i) * 0x9e3779b1u ^ row_key);
      const float u = (static_cast<float>(h >> 8) + 0.5f) * (1.f / 16777216.f);
      key = z - __logf(-__logf(u));
    }
    if (key > st.key) { st.key = key; st.z = z; st.idx = i; }
  }
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
  if (lane == 0) part[warp] = st;
  __syncthreads();
  if (warp == 0) {
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

// Top-k / top-p sampling: top_k int32 [B] (<= 0: off), top_p fp32 [B] (>= 1: off). mask_ids (optional, int32
// [B, mask_cap]) receives the ids of the kept tokens in no particular order and mask_count (int32 [B], zeroed by
// the caller) how many there are (it may exceed mask_cap; only the first mask_cap are stored).
PRB_API int prb_sample_truncated(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                                 long long ld, unsigned long long seed, int* tokens, float* logprobs, int* mask_ids,
                                 int* mask_count, int mask_cap, int B, int V, void* stream) {
  if (B <= 0) return 0;
  if (V <= 0 || (mask_ids != nullptr && (mask_count == nullptr || mask_cap <= 0))) return -3;
  prb::sample_truncated_kernel<<<B, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, temperature, top_k, top_p, ld, seed, tokens, logprobs, mask_ids, mask_count, mask_cap, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
