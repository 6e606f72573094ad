// Group RMSNorm combined with a gate (Mamba-2 and gated delta-net output norms), bf16 in / out:
//
//   gate_first = 1:  u = x * silu(g);  y = u * rsqrt(mean_group(u^2) + eps) * w          (Mamba-2)
//   gate_first = 0:  y = x * rsqrt(mean_group(x^2) + eps) * w * silu(g)                  (gated delta-net)
//
// x, g, y: [rows, cols]; the norm runs over groups of `group` consecutive channels (cols % group == 0,
// group % 8 == 0, group <= 8192); w: [cols] when gate_first (one weight per channel) or [group] otherwise
// is passed with `w_len` (the weight index is channel % w_len). One warp per (row, group), 8
// channels per 16-byte load. The backward recomputes the statistics and writes dx, dg (bf16); every
// warp keeps one group and walks over rows, so its lanes own fixed channels and the weight gradient
// is summed in registers and added to dw (fp32) once per warp (groups of at most 1024 channels).
//
// The reference computes these with PyTorch ops / fla's FusedRMSNormGated
// (src/prime_rl/trainer/models/nemotron_h/mamba.py:56-76, qwen3_5/gated_delta_net.py:41-45).
#include "common.cuh"

namespace prb {

constexpr int kGnWarps = 8;           // warps (row-groups) per CTA

__device__ __forceinline__ void gn_load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}

__device__ __forceinline__ void gn_store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16(v[0], v[1]); u.y = pack_bf16(v[2], v[3]); u.z = pack_bf16(v[4], v[5]); u.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ float gn_silu(float z) { return z / (1.f + __expf(-z)); }
__device__ __forceinline__ float gn_dsilu(float z) {
  const float s = 1.f / (1.f + __expf(-z));
  return s * (1.f + z * (1.f - s));
}

__global__ void __launch_bounds__(kGnWarps * 32)
gated_norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                      const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, long long items, int cols,
                      int group, int w_len, float eps, int gate_first) {
  const long long item = static_cast<long long>(blockIdx.x) * kGnWarps + (threadIdx.x >> 5);
  if (item >= items) return;
  const int lane = threadIdx.x & 31;
  const int groups = cols / group;
  const long long row = item / groups;
  const int c_base = static_cast<int>(item - row * groups) * group;
  const long long off = row * cols + c_base;
  const int nvec = group / 8;
  float ss = 0.f;
  for (int v = lane; v < nvec; v += 32) {
    float xv[8], gv[8];
    gn_load8(x + off + v * 8, xv);
    if (gate_first) {
      gn_load8(g + off + v * 8, gv);
#pragma unroll
      for (int j = 0; j < 8; ++j) xv[j] *= gn_silu(gv[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss = fmaf(xv[j], xv[j], ss);
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / static_cast<float>(group) + eps);
  for (int v = lane; v < nvec; v += 32) {
    float xv[8], gv[8], wv[8], o[8];
    gn_load8(x + off + v * 8, xv);
    gn_load8(g + off + v * 8, gv);
    gn_load8(w + (c_base + v * 8) % w_len, wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = gn_silu(gv[j]);
      o[j] = gate_first ? xv[j] * sg * rstd * wv[j] : xv[j] * rstd * wv[j] * sg;
    }
    gn_store8(y + off + v * 8, o);
  }
}

// Warp `wid` of the grid owns group wid % groups and the rows wid / groups, + rows_par, + 2 rows_par, ...
// (the host launches groups * rows_par warps). dw: fp32 [w_len], zero on entry.
__global__ void __launch_bounds__(kGnWarps * 32)
gated_norm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                      const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ dy,
                      __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dg, float* __restrict__ dw,
                      long long rows, int cols, int group, int w_len, int rows_par, float eps, int gate_first) {
  const long long wid = static_cast<long long>(blockIdx.x) * kGnWarps + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int groups = cols / group;
  const int gi = static_cast<int>(wid % groups);
  const int c_base = gi * group;
  const int nvec = group / 8;
  constexpr int kOwn = 4;                                   // vectors per lane: group <= 4 * 32 * 8
  float wacc[kOwn][8];
#pragma unroll
  for (int i = 0; i < kOwn; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) wacc[i][j] = 0.f;
  for (long long row = wid / groups; row < rows; row += rows_par) {
    const long long off = row * cols + c_base;
    // pass 1: statistics. u = normalised input (x silu(g) or x); t = dy * w (* silu(g) when the gate comes last)
    float ss = 0.f, dot = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float xv[8], gv[8], wv[8], dv[8];
      gn_load8(x + off + v * 8, xv);
      gn_load8(g + off + v * 8, gv);
      gn_load8(w + (c_base + v * 8) % w_len, wv);
      gn_load8(dy + off + v * 8, dv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sg = gn_silu(gv[j]);
        const float u = gate_first ? xv[j] * sg : xv[j];
        const float t = gate_first ? dv[j] * wv[j] : dv[j] * wv[j] * sg;
        ss = fmaf(u, u, ss);
        dot = fmaf(u, t, dot);
      }
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float rstd = rsqrtf(ss / static_cast<float>(group) + eps);
    const float coef = dot * rstd * rstd * rstd / static_cast<float>(group);
#pragma unroll
    for (int i = 0; i < kOwn; ++i) {
      const int v = lane + i * 32;
      if (v >= nvec) break;
      float xv[8], gv[8], wv[8], dv[8], ox[8], og[8];
      gn_load8(x + off + v * 8, xv);
      gn_load8(g + off + v * 8, gv);
      gn_load8(w + (c_base + v * 8) % w_len, wv);
      gn_load8(dy + off + v * 8, dv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sg = gn_silu(gv[j]), dsg = gn_dsilu(gv[j]);
        const float u = gate_first ? xv[j] * sg : xv[j];
        const float t = gate_first ? dv[j] * wv[j] : dv[j] * wv[j] * sg;
        const float du = t * rstd - u * coef;               // gradient with respect to the normalised input
        if (gate_first) {
          ox[j] = du * sg;
          og[j] = du * xv[j] * dsg;
          wacc[i][j] = fmaf(dv[j], u * rstd, wacc[i][j]);
        } else {
          ox[j] = du;
          og[j] = dv[j] * xv[j] * rstd * wv[j] * dsg;
          wacc[i][j] = fmaf(dv[j] * sg, u * rstd, wacc[i][j]);
        }
      }
      gn_store8(dx + off + v * 8, ox);
      gn_store8(dg + off + v * 8, og);
    }
  }
#pragma unroll
  for (int i = 0; i < kOwn; ++i) {
    const int v = lane + i * 32;
    if (v >= nvec) break;
    const int wc = (c_base + v * 8) % w_len;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dw + wc + j, wacc[i][j]);
  }
}

}  // namespace prb

PRB_API int prb_gated_norm_fwd(const void* x, const void* g, const void* w, void* y, long long rows, int cols, int group,
                               int w_len, float eps, int gate_first, void* stream) {
  if (rows <= 0) return 0;
  if (group <= 0 || cols % group || group % 8 || group > 8192 || w_len % 8 || (w_len != cols && w_len != group)) return -3;
  const long long items = rows * (cols / group);
  prb::gated_norm_fwd_kernel<<<static_cast<unsigned>((items + prb::kGnWarps - 1) / prb::kGnWarps), prb::kGnWarps * 32, 0,
                               reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(g),
      reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(y), items, cols, group, w_len, eps,
      gate_first);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// dw: fp32 [w_len], zero on entry. Groups of at most 1024 channels.
PRB_API int prb_gated_norm_bwd(const void* x, const void* g, const void* w, const void* dy, void* dx, void* dg, float* dw,
                               long long rows, int cols, int group, int w_len, float eps, int gate_first, void* stream) {
  if (rows <= 0) return 0;
  if (group <= 0 || cols % group || group % 8 || group > 1024 || w_len % 8 || (w_len != cols && w_len != group)) return -3;
  const int groups = cols / group;
  // groups * rows_par warps, rows_par a multiple of the warps per CTA so that the grid is whole CTAs
  long long rows_par = (148LL * 16 * prb::kGnWarps + groups - 1) / groups;
  if (rows_par > rows) rows_par = rows;
  rows_par = (rows_par + prb::kGnWarps - 1) / prb::kGnWarps * prb::kGnWarps;
  const long long warps = rows_par * groups;
  prb::gated_norm_bwd_kernel<<<static_cast<unsigned>(warps / prb::kGnWarps), prb::kGnWarps * 32, 0,
                               reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(g),
      reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<const __nv_bfloat16*>(dy),
      reinterpret_cast<__nv_bfloat16*>(dx), reinterpret_cast<__nv_bfloat16*>(dg), dw, rows, cols, group, w_len,
      static_cast<int>(rows_par), eps, gate_first);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
