// Depthwise causal convolution over the tokens of a packed stream (Mamba-2 and gated delta-net
// mixers): y[t, c] = act(bias[c] + sum_s w[c, K-1-s] * x[t-s, c]) where tap s only counts when token
// t-s belongs to the same document (pos[t] >= s). x, y bf16 [T, C]; w bf16 [C, K] (K <= 4);
// pos int32 [T]. A thread handles 8 channels (16-byte loads) of several tokens with the taps in registers; memory-bound.
//
// Backward recomputes the pre-activation, then
//   dx[t, c]     = sum_s w[c, K-1-s] * dpre[t+s, c]     (token t+s in the same document: pos[t+s] >= s)
//   dw[c, K-1-s] = sum_t dpre[t, c] * x[t-s, c]          (fp32 atomics after a per-block reduction over tokens)
//   dbias[c]     = sum_t dpre[t, c]
//
// The reference calls fla.modules.conv.causal_conv1d (Triton) here
// (src/prime_rl/trainer/models/nemotron_h/mamba.py:201-207, qwen3_5/gated_delta_net.py:75-82).
#include "common.cuh"

namespace prb {

constexpr int kConvMaxK = 4;
constexpr int kConvTok = 32;   // tokens per block in the backward kernel

__device__ __forceinline__ void conv_load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}

__device__ __forceinline__ void conv_store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16(v[0], v[1]); u.y = pack_bf16(v[2], v[3]); u.z = pack_bf16(v[4], v[5]); u.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// pre-activation of 8 channels [c0, c0 + 8) of token t
__device__ __forceinline__ void conv_pre(const __nv_bfloat16* x, const float (&w)[kConvMaxK][8], const float (&b)[8],
                                         const int* pos, long long t, int c0, int C, int K, float (&pre)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) pre[j] = b[j];
  const int pt = pos[t];
  for (int s = 0; s < K; ++s) {
    if (pt < s) break;
    float v[8];
    conv_load8(x + (t - s) * C + c0, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) pre[j] = fmaf(w[K - 1 - s][j], v[j], pre[j]);
  }
}

__device__ __forceinline__ void conv_load_w(const __nv_bfloat16* w, const __nv_bfloat16* bias, int c0, int K,
                                            float (&wr)[kConvMaxK][8], float (&br)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    br[j] = bias ? __bfloat162float(bias[c0 + j]) : 0.f;
    for (int k = 0; k < K; ++k) wr[k][j] = __bfloat162float(w[(c0 + j) * K + k]);
  }
}

// grid: (channel groups of 32 vectors, token blocks of kConvFwdTok); block: 32 x 8 threads (x = channel
// vector, y = token lane). A thread keeps the taps of its 8 channels in registers and walks
// kConvFwdTok / 8 tokens, so the weights are read once per 8 tokens instead of once per token.
constexpr int kConvFwdTok = 64;

__global__ void __launch_bounds__(256)
conv1d_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                  const __nv_bfloat16* __restrict__ bias, const int* __restrict__ pos, __nv_bfloat16* __restrict__ y,
                  long long T, int C, int K, int silu) {
  const int cvec = blockIdx.x * 32 + threadIdx.x;
  if (cvec >= C / 8) return;
  const int c0 = cvec * 8;
  float wr[kConvMaxK][8], br[8];
  conv_load_w(w, bias, c0, K, wr, br);
  const long long t_blk = static_cast<long long>(blockIdx.y) * kConvFwdTok;
#pragma unroll 2
  for (int it = 0; it < kConvFwdTok / 8; ++it) {
    const long long t = t_blk + it * 8 + threadIdx.y;
    if (t >= T) break;
    float pre[8];
    conv_pre(x, wr, br, pos, t, c0, C, K, pre);
    if (silu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) pre[j] = pre[j] / (1.f + __expf(-pre[j]));
    }
    conv_store8(y + t * C + c0, pre);
  }
}

// grid: (C / 8 / 32 channel groups of 32 vectors, token blocks of kConvTok); block: 32 x 8 threads
// (x = channel vector, y = token lane). Each thread walks kConvTok / 8 tokens.
__global__ void __launch_bounds__(256)
conv1d_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                  const __nv_bfloat16* __restrict__ bias, const int* __restrict__ pos,
                  const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                  float* __restrict__ dbias, long long T, int C, int K, int silu) {
  const int cvec = blockIdx.x * 32 + threadIdx.x;
  const bool live_c = cvec < C / 8;
  const int c0 = (live_c ? cvec : 0) * 8;
  float wr[kConvMaxK][8], br[8];
  conv_load_w(w, bias, c0, K, wr, br);
  float gw[kConvMaxK][8], gb[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    gb[j] = 0.f;
#pragma unroll
    for (int k = 0; k < kConvMaxK; ++k) gw[k][j] = 0.f;
  }
  const long long t_blk = static_cast<long long>(blockIdx.y) * kConvTok;
  for (int it = 0; it < kConvTok / 8; ++it) {
    const long long t = t_blk + it * 8 + threadIdx.y;
    if (t >= T || !live_c) continue;
    // dx[t] needs dpre of tokens t .. t+K-1; dw / dbias take dpre[t] itself
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < K; ++s) {
      const long long u = t + s;
      if (u >= T || pos[u] < s) continue;          // token u is in another document or too early in its own
      float pre[8], g[8];
      conv_pre(x, wr, br, pos, u, c0, C, K, pre);
      conv_load8(dy + u * C + c0, g);
      if (silu) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float sg = 1.f / (1.f + __expf(-pre[j]));
          g[j] *= sg * (1.f + pre[j] * (1.f - sg));
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(wr[K - 1 - s][j], g[j], acc[j]);
      if (s == 0) {
        const int pt = pos[t];
#pragma unroll
        for (int j = 0; j < 8; ++j) gb[j] += g[j];
        for (int s2 = 0; s2 < K; ++s2) {
          if (pt < s2) break;
          float xv[8];
          conv_load8(x + (t - s2) * C + c0, xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) gw[K - 1 - s2][j] = fmaf(g[j], xv[j], gw[K - 1 - s2][j]);
        }
      }
    }
    conv_store8(dx + t * C + c0, acc);
  }
  // reduce the weight / bias gradients over the 8 token lanes, then one atomic per value and block
  __shared__ float red[8][32][8];
  for (int k = 0; k <= K; ++k) {
#pragma unroll
    for (int j = 0; j < 8; ++j) red[threadIdx.y][threadIdx.x][j] = (k < K) ? gw[k][j] : gb[j];
    __syncthreads();
    if (threadIdx.y == 0 && live_c) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float sum = 0.f;
#pragma unroll
        for (int l = 0; l < 8; ++l) sum += red[l][threadIdx.x][j];
        if (k < K) atomicAdd(dw + (c0 + j) * K + k, sum);
        else if (dbias) atomicAdd(dbias + c0 + j, sum);
      }
    }
    __syncthreads();
  }
}

}  // namespace prb

PRB_API int prb_conv1d_fwd(const void* x, const void* w, const void* bias, const int* pos, void* y, long long T, int C,
                           int K, int silu, void* stream) {
  if (T <= 0) return 0;
  if (C % 8 || K < 1 || K > prb::kConvMaxK) return -3;
  dim3 grid((C / 8 + 31) / 32, static_cast<unsigned>((T + prb::kConvFwdTok - 1) / prb::kConvFwdTok));
  prb::conv1d_fwd_kernel<<<grid, dim3(32, 8), 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),
      reinterpret_cast<const __nv_bfloat16*>(bias), pos, reinterpret_cast<__nv_bfloat16*>(y), T, C, K, silu);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// dw [C, K] and dbias [C] (fp32) must be zero on entry.
PRB_API int prb_conv1d_bwd(const void* x, const void* w, const void* bias, const int* pos, const void* dy, void* dx,
                           float* dw, float* dbias, long long T, int C, int K, int silu, void* stream) {
  if (T <= 0) return 0;
  if (C % 8 || K < 1 || K > prb::kConvMaxK) return -3;
  dim3 grid((C / 8 + 31) / 32, static_cast<unsigned>((T + prb::kConvTok - 1) / prb::kConvTok));
  prb::conv1d_bwd_kernel<<<grid, dim3(32, 8), 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),
      reinterpret_cast<const __nv_bfloat16*>(bias), pos, reinterpret_cast<const __nv_bfloat16*>(dy),
      reinterpret_cast<__nv_bfloat16*>(dx), dw, dbias, T, C, K, silu);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
