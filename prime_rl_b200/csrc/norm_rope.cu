// RMSNorm forward/backward (optionally fused with the residual add) and the fused per-head
// QK-RMSNorm + rotary embedding, bf16 activations with fp32 math. Bandwidth-bound kernels:
// one warp owns one row, 16-byte vector loads, the row stays in registers between the
// reduction and the write.
//
// Replaces layers/norms.py:29-47 (quack.rmsnorm) and layers/rotary_emb.py:83-118 +
// the q/k norm in layers/attn.py:141-152 of the reference.
#include "common.cuh"

namespace prb {

constexpr int kNormThreads = 256;

// Sum over the TPR threads that share one row (TPR = 32: one warp; TPR = 128: four warps
// through shared memory). Every thread of the CTA must call it.
template <int TPR>
__device__ __forceinline__ float row_group_sum(float v, float* scratch) {
  v = warp_sum(v);
  if (TPR == 32) return v;
  const int warp = threadIdx.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[warp] = v;
  __syncthreads();
  const int g0 = (warp / (TPR / 32)) * (TPR / 32);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < TPR / 32; ++i) s += scratch[g0 + i];
  return s;
}

__device__ __forceinline__ void load8(const uint4& a, float* f) {
  float2 f0 = unpack_bf16(a.x), f1 = unpack_bf16(a.y), f2 = unpack_bf16(a.z), f3 = unpack_bf16(a.w);
  f[0] = f0.x; f[1] = f0.y; f[2] = f1.x; f[3] = f1.y; f[4] = f2.x; f[5] = f2.y; f[6] = f3.x; f[7] = f3.y;
}
__device__ __forceinline__ uint4 store8(const float* f) {
  uint4 o;
  o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]); o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
  return o;
}

// ---------------------------------------------------------------- RMSNorm forward
// h = x (+ residual); y = h * rsqrt(mean(h^2) + eps) * w; optionally writes h back
// (residual stream) and rstd. TPR threads share a row, VPL 16-byte vectors per thread.
template <int TPR, int VPL>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, long long rows, int cols,
                   float eps) {
  __shared__ float scratch[kNormThreads / 32];
  const int rl = threadIdx.x % TPR;
  const long long row = static_cast<long long>(blockIdx.x) * (kNormThreads / TPR) + threadIdx.x / TPR;
  const bool active = row < rows;
  const int nvec = cols >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (active ? row : 0) * cols);
  const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + (active ? row : 0) * cols) : nullptr;
  float v[VPL][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = rl + i * TPR;
    if (active && vi < nvec) {
      load8(xr[vi], v[i]);
      if (rr) {
        float g[8];
        load8(rr[vi], g);
#pragma unroll
        for (int t = 0; t < 8; ++t) v[i][t] += g[t];
        // the residual stream is stored in bf16: normalise what is stored
        const uint4 o = store8(v[i]);
        if (h_out) reinterpret_cast<uint4*>(h_out + row * cols)[vi] = o;
        load8(o, v[i]);
      }
#pragma unroll
      for (int t = 0; t < 8; ++t) ss += v[i][t] * v[i][t];
    }
  }
  ss = row_group_sum<TPR>(ss, scratch);
  const float rstd = rsqrtf(ss / static_cast<float>(cols) + eps);
  if (active && rl == 0 && rstd_out) rstd_out[row] = rstd;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + (active ? row : 0) * cols);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int vi = rl + i * TPR;
    if (active && vi < nvec) {
      float wv[8], o[8];
      load8(wr[vi], wv);
#pragma unroll
      for (int t = 0; t < 8; ++t) o[t] = v[i][t] * rstd * wv[t];
      yr[vi] = store8(o);
    }
  }
}

// ---------------------------------------------------------------- RMSNorm backward
// dx = rstd * (dy*w) - x * rstd^3 * mean(dy*w*x)  (+ dres);  dw partial per CTA.
// dw_partial has shape [gridDim.x, cols] fp32; a second kernel sums it.
template <int TPR, int VPL>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, long long rows, int cols, int rows_per_cta) {
  extern __shared__ float s_dw[];  // [cols]
  __shared__ float scratch[kNormThreads / 32];
  constexpr int RPI = kNormThreads / TPR;  // rows per iteration
  const int rl = threadIdx.x % TPR;
  const int rslot = threadIdx.x / TPR;
  const int nvec = cols >> 3;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) s_dw[i] = 0.f;
  __syncthreads();
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  float dwacc[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i)
#pragma unroll
    for (int t = 0; t < 8; ++t) dwacc[i][t] = 0.f;

  const long long row0 = static_cast<long long>(blockIdx.x) * rows_per_cta;
  for (int r = 0; r < rows_per_cta; r += RPI) {
    const long long row = row0 + r + rslot;
    const bool active = (r + rslot < rows_per_cta) && row < rows;
    const float rstd = active ? rstd_in[row] : 0.f;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (active ? row : 0) * cols);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (active ? row : 0) * cols);
    float xv[VPL][8], gv[VPL][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = rl + i * TPR;
      if (active && vi < nvec) {
        float wv[8];
        load8(xr[vi], xv[i]);
        load8(gr[vi], gv[i]);
        load8(wr[vi], wv);
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          dwacc[i][t] += gv[i][t] * xv[i][t] * rstd;
          gv[i][t] *= wv[t];
          dot += gv[i][t] * xv[i][t];
        }
      }
    }
    dot = row_group_sum<TPR>(dot, scratch);
    const float c = dot * rstd * rstd * rstd / static_cast<float>(cols);
    uint4* dxr = reinterpret_cast<uint4*>(dx + (active ? row : 0) * cols);
    const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + (active ? row : 0) * cols) : nullptr;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = rl + i * TPR;
      if (active && vi < nvec) {
        float o[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) o[t] = gv[i][t] * rstd - xv[i][t] * c;
        if (rr) {
          float b[8];
          load8(rr[vi], b);
#pragma unroll
          for (int t = 0; t < 8; ++t) o[t] += b[t];
        }
        dxr[vi] = store8(o);
      }
    }
  }
  if (dw_partial) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = rl + i * TPR;
      if (vi < nvec) {
#pragma unroll
        for (int t = 0; t < 8; ++t) atomicAdd(&s_dw[vi * 8 + t], dwacc[i][t]);
      }
    }
    __syncthreads();
    float* out = dw_partial + static_cast<long long>(blockIdx.x) * cols;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) out[i] = s_dw[i];
  }
}

__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int nparts, int cols,
                              int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int i = 0; i < nparts; ++i) s += partial[static_cast<long long>(i) * cols + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ---------------------------------------------------------------- QK-norm + RoPE
// One warp per (token, head). x is [T, heads, D] with token pitch `ld` elements; D in
// {64, 128, 256}. y = rope(rmsnorm(x) * w) with the half-split rotation
// (x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin), angle = pos * inv_freq[i], i < D/2.
// w == nullptr skips the norm (plain RoPE, used for models without QK-norm).
template <int D, bool BWD>
__global__ void __launch_bounds__(256)
qknorm_rope_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gin,
                   const __nv_bfloat16* __restrict__ w, const int* __restrict__ pos,
                   const float* __restrict__ inv_freq, __nv_bfloat16* __restrict__ out, float* __restrict__ rstd_io,
                   float* __restrict__ dw, long long T, int heads, long long ld_x, long long ld_out, long long ld_dx,
                   float eps) {
  constexpr int EPL = D / 32;  // elements per lane, contiguous
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  __shared__ float s_dw[D];
  if (BWD && dw) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) s_dw[i] = 0.f;
    __syncthreads();
  }
  const bool active = item < T * heads;
  if (active) {
    const long long t = item / heads;
    const int h = static_cast<int>(item - t * heads);
    const int e0 = lane * EPL;
    const float p = static_cast<float>(pos[t]);
    float cs[EPL], sn[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int fi = (e0 + i) % (D / 2);
      sincosf(p * inv_freq[fi], &sn[i], &cs[i]);
    }
    const bool upper = e0 >= D / 2;
    float xv[EPL];
    {
      const __nv_bfloat16* src = x + t * ld_x + static_cast<long long>(h) * D + e0;
#pragma unroll
      for (int i = 0; i < EPL; ++i) xv[i] = __bfloat162float(src[i]);
    }
    if (!BWD) {
      float rstd = 1.f;
      if (w) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) ss += xv[i] * xv[i];
        ss = warp_sum(ss);
        rstd = rsqrtf(ss / D + eps);
        if (lane == 0 && rstd_io) rstd_io[item] = rstd;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          // the normalised value is rounded to bf16 before the rotation, as a separate
          // norm module would produce it
          xv[i] = __bfloat162float(__float2bfloat16(xv[i] * rstd * __bfloat162float(w[e0 + i])));
        }
      }
      __nv_bfloat16* dst = out + t * ld_out + static_cast<long long>(h) * D + e0;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, xv[i], 16);
        const float r = upper ? (xv[i] * cs[i] + other * sn[i]) : (xv[i] * cs[i] - other * sn[i]);
        dst[i] = __float2bfloat16(r);
      }
    } else {
      // gin = dL/dy. Undo the rotation (transpose), then the norm backward.
      float gv[EPL];
      const __nv_bfloat16* gsrc = gin + t * ld_out + static_cast<long long>(h) * D + e0;
#pragma unroll
      for (int i = 0; i < EPL; ++i) gv[i] = __bfloat162float(gsrc[i]);
      float gn[EPL];
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, gv[i], 16);
        gn[i] = upper ? (gv[i] * cs[i] - other * sn[i]) : (gv[i] * cs[i] + other * sn[i]);
      }
      __nv_bfloat16* dst = out + t * ld_dx + static_cast<long long>(h) * D + e0;
      if (w) {
        const float rstd = rstd_io[item];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          const float wi = __bfloat162float(w[e0 + i]);
          if (dw) atomicAdd(&s_dw[e0 + i], gn[i] * xv[i] * rstd);
          gn[i] *= wi;
          dot += gn[i] * xv[i];
        }
        dot = warp_sum(dot);
        const float c = dot * rstd * rstd * rstd / D;
#pragma unroll
        for (int i = 0; i < EPL; ++i) dst[i] = __float2bfloat16(gn[i] * rstd - xv[i] * c);
      } else {
#pragma unroll
        for (int i = 0; i < EPL; ++i) dst[i] = __float2bfloat16(gn[i]);
      }
    }
  }
  if (BWD && dw) {
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(&dw[i], s_dw[i]);
  }
}


// Inference: the packed projection qkv [T, (nq + 2 nkv) * D] -> q [T, nq, D] (norm + rotary) and, in the same
// launch, K (norm + rotary) and V written into the paged cache at slot[t] (cache rows of nkv * D elements) and,
// when k_out / v_out are given, also as contiguous [T, nkv, D] tensors. One warp per (token, head); the
// arithmetic is the one of qknorm_rope_kernel, so the engine and the trainer see the same values.
// EPL contiguous bf16 values of one lane as one 4 / 8 / 16-byte access (the addresses are multiples of EPL * 2 bytes:
// rows of D elements, lane offsets of EPL elements, 16-byte aligned bases).
template <int EPL>
__device__ __forceinline__ void rope_load(const __nv_bfloat16* src, float (&x)[EPL]) {
  if constexpr (EPL == 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(src);
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  } else if constexpr (EPL == 2) {
    const float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(src));
    x[0] = a.x; x[1] = a.y;
  } else {
    const uint4 u = *reinterpret_cast<const uint4*>(src);
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y; x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
  }
}

template <int EPL>
__device__ __forceinline__ void rope_store(__nv_bfloat16* dst, const __nv_bfloat16 (&r)[EPL]) {
  if constexpr (EPL == 4) {
    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(r);
  } else if constexpr (EPL == 2) {
    *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(r);
  } else {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(r);
  }
}

constexpr int kRopeHeadsPerWarp = 4;   // rows a warp has in flight at once (one 256-byte row alone cannot cover DRAM latency)

template <int D>
__global__ void __launch_bounds__(256)
qkv_rope_cache_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ qw,
                      const __nv_bfloat16* __restrict__ kw, const int* __restrict__ pos,
                      const float* __restrict__ inv_freq, const long long* __restrict__ slot,
                      __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                      __nv_bfloat16* __restrict__ v_out, __nv_bfloat16* __restrict__ k_cache,
                      __nv_bfloat16* __restrict__ v_cache, long long T, int nq, int nkv, float eps) {
  constexpr int EPL = D / 32;
  constexpr int HPW = kRopeHeadsPerWarp;
  constexpr int kTok = 9;                    // the 8 consecutive (token, head group) items of a CTA touch at most 9 tokens
  __shared__ float s_cs[kTok][D / 2], s_sn[kTok][D / 2];
  const int lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const int groups = (heads + HPW - 1) / HPW;          // items per token
  const long long item0 = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5);
  const long long t0 = item0 / groups;
  // the sine / cosine table of the CTA's tokens, computed once instead of once per head
  for (int i = threadIdx.x; i < kTok * (D / 2); i += blockDim.x) {
    const int which = i / (D / 2), fi = i - which * (D / 2);
    const long long tt = t0 + which;
    if (tt < T && tt * groups < item0 + (blockDim.x >> 5))
      sincosf(static_cast<float>(pos[tt]) * inv_freq[fi], &s_sn[which][fi], &s_cs[which][fi]);
  }
  __syncthreads();
  const long long item = item0 + (threadIdx.x >> 5);
  if (item >= T * groups) return;
  const long long t = item / groups;
  const int h0 = static_cast<int>(item - t * groups) * HPW;
  const int tw = static_cast<int>(t - t0);
  const int e0 = lane * EPL;
  const bool upper = e0 >= D / 2;
  float cs[EPL], sn[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int fi = (e0 + i) % (D / 2);
    cs[i] = s_cs[tw][fi];
    sn[i] = s_sn[tw][fi];
  }
  // all rows of the group are requested before the first one is used
  float xv[HPW][EPL];
  const __nv_bfloat16* row = qkv + t * (static_cast<long long>(heads) * D) + e0;
#pragma unroll
  for (int j = 0; j < HPW; ++j)
    if (h0 + j < heads) rope_load<EPL>(row + static_cast<long long>(h0 + j) * D, xv[j]);
  const long long cache_row = slot[t] * nkv;
#pragma unroll
  for (int j = 0; j < HPW; ++j) {
    const int h = h0 + j;
    if (h >= heads) break;
    const bool is_q = h < nq, is_v = h >= nq + nkv;
    const int hk = is_q ? h : (is_v ? h - nq - nkv : h - nq);      // head index inside its own tensor
    __align__(16) __nv_bfloat16 res[EPL];
    if (is_v) {
#pragma unroll
      for (int i = 0; i < EPL; ++i) res[i] = __float2bfloat16(xv[j][i]);
    } else {
      const __nv_bfloat16* w = is_q ? qw : kw;
      if (w) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) ss += xv[j][i] * xv[j][i];
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / D + eps);
#pragma unroll
        for (int i = 0; i < EPL; ++i)
          xv[j][i] = __bfloat162float(__float2bfloat16(xv[j][i] * rstd * __bfloat162float(w[e0 + i])));
      }
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, xv[j][i], 16);
        const float r = upper ? (xv[j][i] * cs[i] + other * sn[i]) : (xv[j][i] * cs[i] - other * sn[i]);
        res[i] = __float2bfloat16(r);
      }
    }
    if (is_q) {
      rope_store<EPL>(q_out + (t * nq + hk) * D + e0, res);
      continue;
    }
    __nv_bfloat16* lin = is_v ? v_out : k_out;
    if (lin != nullptr) rope_store<EPL>(lin + (t * nkv + hk) * D + e0, res);
    rope_store<EPL>((is_v ? v_cache : k_cache) + (cache_row + hk) * D + e0, res);
  }
}

}  // namespace prb

using namespace prb;

// TPR = 32 for narrow rows, 128 otherwise; VPL covers cols / 8 / TPR vectors per thread.
#define PRB_VPL_DISPATCH(cols, CALL)                           \
  do {                                                         \
    const int nvec_ = (cols) / 8;                              \
    if (nvec_ <= 32) { CALL(32, 1); }                          \
    else if (nvec_ <= 64) { CALL(32, 2); }                     \
    else if (nvec_ <= 128) { CALL(32, 4); }                    \
    else if (nvec_ <= 256) { CALL(128, 2); }                   \
    else if (nvec_ <= 512) { CALL(128, 4); }                   \
    else if (nvec_ <= 1024) { CALL(128, 8); }                  \
    else return -2;                                            \
  } while (0)

// x, residual (nullable), w, y, h_out (nullable): bf16; rstd (nullable): fp32 [rows].
// cols must be a multiple of 8 and at most 8192.
PRB_API int prb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out, float* rstd,
                            long long rows, int cols, float eps, void* stream) {
  if (cols % 8) return -1;
  if (rows == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define CALL(TPR, V)                                                                                      \
  rmsnorm_fwd_kernel<TPR, V><<<static_cast<unsigned>((rows + (kNormThreads / TPR) - 1) / (kNormThreads / TPR)), \
                              kNormThreads, 0, s>>>(                                                        \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, \
      (__nv_bfloat16*)h_out, rstd, rows, cols, eps)
  PRB_VPL_DISPATCH(cols, CALL);
#undef CALL
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// dw_partial: fp32 scratch [prb_rmsnorm_bwd_parts(rows), cols] (nullable when dw is not
// wanted); dw: fp32 [cols] (overwritten, or accumulated into when accumulate_dw != 0).
PRB_API int prb_rmsnorm_bwd_parts(long long rows) {
  long long parts = (rows + 63) / 64;
  if (parts > 1184) parts = 1184;  // 148 SMs x 8
  return static_cast<int>(parts < 1 ? 1 : parts);
}

PRB_API int prb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                            void* dx, float* dw_partial, float* dw, int accumulate_dw, long long rows, int cols,
                            void* stream) {
  if (cols % 8) return -1;
  if (rows == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int parts = prb_rmsnorm_bwd_parts(rows);
  const int rows_per_cta = static_cast<int>((rows + parts - 1) / parts);
  const size_t smem = sizeof(float) * cols;
#define CALL(TPR, V)                                                                                    \
  rmsnorm_bwd_kernel<TPR, V><<<parts, kNormThreads, smem, s>>>(                                           \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,                   \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, dw ? dw_partial : nullptr, rows, cols, rows_per_cta)
  PRB_VPL_DISPATCH(cols, CALL);
#undef CALL
  if (dw) colsum_kernel<<<(cols + 255) / 256, 256, 0, s>>>(dw_partial, dw, parts, cols, accumulate_dw);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Forward: out = rope(norm(x)), out pitch ld_out. Backward (bwd != 0): out (= dx, pitch
// ld_dx) from gin (= dy, pitch ld_out), x (pitch ld_x) and the saved rstd; dw (fp32 [D],
// accumulated) may be null. Pitches are in elements per token.
PRB_API int prb_qknorm_rope(const void* x, const void* gin, const void* w, const int* pos, const float* inv_freq,
                            void* out, float* rstd, float* dw, long long T, int heads, int D, long long ld_x,
                            long long ld_out, long long ld_dx, float eps, int bwd, void* stream) {
  if (T == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long items = T * heads;
  const unsigned grid = static_cast<unsigned>((items + 7) / 8);
#define LAUNCH(DD, B)                                                                                     \
  qknorm_rope_kernel<DD, B><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gin,        \
                                                  (const __nv_bfloat16*)w, pos, inv_freq, (__nv_bfloat16*)out, \
                                                  rstd, dw, T, heads, ld_x, ld_out, ld_dx, eps)
  if (D == 128) { if (bwd) LAUNCH(128, true); else LAUNCH(128, false); }
  else if (D == 64) { if (bwd) LAUNCH(64, true); else LAUNCH(64, false); }
  else if (D == 256) { if (bwd) LAUNCH(256, true); else LAUNCH(256, false); }
  else return -2;
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// qkv bf16 [T, (nq + 2 nkv) * D] contiguous; qw / kw bf16 [D] or null (no QK norm); pos int32 [T]; slot int64 [T]
// (row of the flattened cache [pages * page_size, nkv, D]); k_out / v_out may be null.
PRB_API int prb_qkv_rope_cache(const void* qkv, const void* qw, const void* kw, const int* pos, const float* inv_freq,
                               const long long* slot, void* q_out, void* k_out, void* v_out, void* k_cache,
                               void* v_cache, long long T, int nq, int nkv, int D, float eps, void* stream) {
  if (T == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long items = T * ((nq + 2 * nkv + prb::kRopeHeadsPerWarp - 1) / prb::kRopeHeadsPerWarp);
  const unsigned grid = static_cast<unsigned>((items + 7) / 8);
#define LAUNCH(DD)                                                                                                  \
  prb::qkv_rope_cache_kernel<DD><<<grid, 256, 0, s>>>(                                                               \
      (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, pos, inv_freq, slot,           \
      (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out, (__nv_bfloat16*)k_cache,                 \
      (__nv_bfloat16*)v_cache, T, nq, nkv, eps)
  if (D == 128) LAUNCH(128);
  else if (D == 64) LAUNCH(64);
  else if (D == 256) LAUNCH(256);
  else return -2;
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
