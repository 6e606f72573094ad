// Bandwidth-bound elementwise kernels: gated activations (SwiGLU, clamped SwiGLU, ReLU^2)
// forward/backward, the flat-buffer fused AdamW step with device-side gradient clipping,
// squared-norm reduction and the per-token RL loss.
//
// Replaces layers/activations.py:12-43, torch.optim.AdamW(fused=True)
// (trainer/optim/__init__.py:133-140), clip_grad_norm_ (trainer/utils.py:77-97) and the
// per-token losses of trainer/rl/loss.py:140-276 of the reference.
#include "common.cuh"

namespace prb {

enum ActKind : int { kSwiGLU = 0, kSwiGLUClamped = 1, kReLU2 = 2 };

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// y[r, c] = act(g[r, c]) * u[r, c];   g / u are column windows of rows with pitch ld_in.
// ReLU^2 has no `up` input: y = relu(g)^2.
template <int ACT>
__global__ void __launch_bounds__(256)
glu_fwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
               __nv_bfloat16* __restrict__ y, long long rows, int cols, long long ld_in, long long ld_out,
               float limit, float alpha_act) {
  const int vec_per_row = cols >> 3;
  const long long total = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;
    const uint4 gv = *reinterpret_cast<const uint4*>(g + r * ld_in + c);
    uint4 uv = make_uint4(0, 0, 0, 0);
    if (ACT != kReLU2) uv = *reinterpret_cast<const uint4*>(u + r * ld_in + c);
    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
    const uint32_t uw[4] = {uv.x, uv.y, uv.z, uv.w};
    uint32_t ow[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 gg = unpack_bf16(gw[k]);
      float2 uu = unpack_bf16(uw[k]);
      float o0, o1;
      if (ACT == kSwiGLU) {
        o0 = gg.x * sigmoidf_(gg.x) * uu.x;
        o1 = gg.y * sigmoidf_(gg.y) * uu.y;
      } else if (ACT == kSwiGLUClamped) {
        // GPT-OSS style: gate clamped from above, up clamped to [-limit, limit],
        // y = gate * sigmoid(alpha * gate) * (up + 1)
        const float g0 = fminf(gg.x, limit), g1 = fminf(gg.y, limit);
        const float u0 = fminf(fmaxf(uu.x, -limit), limit), u1 = fminf(fmaxf(uu.y, -limit), limit);
        o0 = g0 * sigmoidf_(alpha_act * g0) * (u0 + 1.f);
        o1 = g1 * sigmoidf_(alpha_act * g1) * (u1 + 1.f);
      } else {
        const float r0 = fmaxf(gg.x, 0.f), r1 = fmaxf(gg.y, 0.f);
        o0 = r0 * r0;
        o1 = r1 * r1;
      }
      ow[k] = pack_bf16(o0, o1);
    }
    *reinterpret_cast<uint4*>(y + r * ld_out + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

// Row-masked variant for the padded row space of grouped experts in inference: one warp per row, the
// validity of a row is looked up once, padding rows (row_valid < 0) cost one load.
template <int ACT>
__global__ void __launch_bounds__(256)
glu_fwd_rows_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                    __nv_bfloat16* __restrict__ y, long long rows, int cols, long long ld_in, long long ld_out,
                    float limit, float alpha_act, const int* __restrict__ row_valid) {
  const int lane = threadIdx.x & 31;
  const int vec_per_row = cols >> 3;
  for (long long r = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); r < rows;
       r += static_cast<long long>(gridDim.x) * 8) {
    if (row_valid[r] < 0) continue;
    for (int vi = lane; vi < vec_per_row; vi += 32) {
      const int c = vi * 8;
      const uint4 gv = *reinterpret_cast<const uint4*>(g + r * ld_in + c);
      uint4 uv = make_uint4(0, 0, 0, 0);
      if (ACT != kReLU2) uv = *reinterpret_cast<const uint4*>(u + r * ld_in + c);
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
      const uint32_t uw[4] = {uv.x, uv.y, uv.z, uv.w};
      uint32_t ow[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 gg = unpack_bf16(gw[k]);
        float2 uu = unpack_bf16(uw[k]);
        float o0, o1;
        if (ACT == kSwiGLU) {
          o0 = gg.x * sigmoidf_(gg.x) * uu.x;
          o1 = gg.y * sigmoidf_(gg.y) * uu.y;
        } else if (ACT == kSwiGLUClamped) {
          const float g0 = fminf(gg.x, limit), g1 = fminf(gg.y, limit);
          const float u0 = fminf(fmaxf(uu.x, -limit), limit), u1 = fminf(fmaxf(uu.y, -limit), limit);
          o0 = g0 * sigmoidf_(alpha_act * g0) * (u0 + 1.f);
          o1 = g1 * sigmoidf_(alpha_act * g1) * (u1 + 1.f);
        } else {
          const float r0 = fmaxf(gg.x, 0.f), r1 = fmaxf(gg.y, 0.f);
          o0 = r0 * r0;
          o1 = r1 * r1;
        }
        ow[k] = pack_bf16(o0, o1);
      }
      *reinterpret_cast<uint4*>(y + r * ld_out + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
  }
}

template <int ACT>
__global__ void __launch_bounds__(256)
glu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ g,
               const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ dg, __nv_bfloat16* __restrict__ du,
               long long rows, int cols, long long ld_in, long long ld_dy, long long ld_dout, float limit,
               float alpha_act) {
  const int vec_per_row = cols >> 3;
  const long long total = rows * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;
    const uint4 gv = *reinterpret_cast<const uint4*>(g + r * ld_in + c);
    const uint4 dv = *reinterpret_cast<const uint4*>(dy + r * ld_dy + c);
    uint4 uv = make_uint4(0, 0, 0, 0);
    if (ACT != kReLU2) uv = *reinterpret_cast<const uint4*>(u + r * ld_in + c);
    const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
    const uint32_t uw[4] = {uv.x, uv.y, uv.z, uv.w};
    const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w};
    uint32_t ogw[4], ouw[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 gg = unpack_bf16(gw[k]);
      const float2 uu = unpack_bf16(uw[k]);
      const float2 dd = unpack_bf16(dw[k]);
      float dgv[2], duv[2];
      const float gs[2] = {gg.x, gg.y}, us[2] = {uu.x, uu.y}, ds[2] = {dd.x, dd.y};
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (ACT == kSwiGLU) {
          const float s = sigmoidf_(gs[t]);
          dgv[t] = ds[t] * us[t] * s * (1.f + gs[t] * (1.f - s));
          duv[t] = ds[t] * gs[t] * s;
        } else if (ACT == kSwiGLUClamped) {
          const float gc = fminf(gs[t], limit);
          const float uc = fminf(fmaxf(us[t], -limit), limit);
          const float s = sigmoidf_(alpha_act * gc);
          const float dglu = s * (1.f + alpha_act * gc * (1.f - s));
          dgv[t] = (gs[t] <= limit) ? ds[t] * (uc + 1.f) * dglu : 0.f;
          duv[t] = (us[t] >= -limit && us[t] <= limit) ? ds[t] * gc * s : 0.f;
        } else {
          dgv[t] = gs[t] > 0.f ? 2.f * gs[t] * ds[t] : 0.f;
          duv[t] = 0.f;
        }
      }
      ogw[k] = pack_bf16(dgv[0], dgv[1]);
      ouw[k] = pack_bf16(duv[0], duv[1]);
    }
    *reinterpret_cast<uint4*>(dg + r * ld_dout + c) = make_uint4(ogw[0], ogw[1], ogw[2], ogw[3]);
    if (ACT != kReLU2) *reinterpret_cast<uint4*>(du + r * ld_dout + c) = make_uint4(ouw[0], ouw[1], ouw[2], ouw[3]);
  }
}

// ---------------------------------------------------------------- squared norm
// out[0] += sum(x^2). fp32 or bf16 input; `out` must be zeroed by the caller.
template <typename T>
__global__ void __launch_bounds__(256) sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
  float acc = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v;
    if (sizeof(T) == 2) v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
    else v = reinterpret_cast<const float*>(x)[i];
    acc += v * v;
  }
  __shared__ float s[8];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 8) {
    float v = s[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) v += __shfl_xor_sync(0xffu, v, o);
    if (threadIdx.x == 0) atomicAdd(out, v);
  }
}

// clip_coef[0] = min(1, max_norm / (sqrt(sumsq) + 1e-6)); norm_out[0] = sqrt(sumsq)
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm, float* __restrict__ coef,
                                 float* __restrict__ norm_out) {
  const float n = sqrtf(sumsq[0]);
  norm_out[0] = n;
  coef[0] = (max_norm > 0.f) ? fminf(1.f, max_norm / (n + 1e-6f)) : 1.f;
}

// ---------------------------------------------------------------- fused AdamW on flat buffers
// master (fp32), m, v (fp32), grad (fp32 or bf16), optional bf16 compute copy.
//   g = grad * grad_scale * clip_coef[0]
//   p = p * (1 - lr*wd);  m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2
//   p -= (lr / bc1) * m / (sqrt(v)/sqrt(bc2) + eps)
// lr is read from device memory so that a captured graph can be replayed across steps.
template <typename GT>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, const GT* __restrict__ grad,
             __nv_bfloat16* __restrict__ p_bf16, long long n, const float* __restrict__ hyper /*lr,bc1,bc2s*/,
             float b1, float b2, float eps, float wd, float grad_scale, const float* __restrict__ clip_coef) {
  const float lr = hyper[0], bc1 = hyper[1], bc2_sqrt = hyper[2];
  const float gs = grad_scale * (clip_coef ? clip_coef[0] : 1.f);
  const float step = lr / bc1;
  const float decay = 1.f - lr * wd;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    if (i + 4 <= n) {
      float4 pp = *reinterpret_cast<float4*>(p + i);
      float4 mm = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      float g[4];
      if (sizeof(GT) == 2) {
        const uint2 gw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(grad) + i);
        const float2 a = unpack_bf16(gw.x), b = unpack_bf16(gw.y);
        g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
      } else {
        const float4 gg = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grad) + i);
        g[0] = gg.x; g[1] = gg.y; g[2] = gg.z; g[3] = gg.w;
      }
      float pa[4] = {pp.x, pp.y, pp.z, pp.w}, ma[4] = {mm.x, mm.y, mm.z, mm.w}, va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float gt = g[t] * gs;
        ma[t] = b1 * ma[t] + (1.f - b1) * gt;
        va[t] = b2 * va[t] + (1.f - b2) * gt * gt;
        pa[t] = pa[t] * decay - step * ma[t] / (sqrtf(va[t]) / bc2_sqrt + eps);
      }
      *reinterpret_cast<float4*>(p + i) = make_float4(pa[0], pa[1], pa[2], pa[3]);
      *reinterpret_cast<float4*>(m + i) = make_float4(ma[0], ma[1], ma[2], ma[3]);
      *reinterpret_cast<float4*>(v + i) = make_float4(va[0], va[1], va[2], va[3]);
      if (p_bf16) {
        uint2 o;
        o.x = pack_bf16(pa[0], pa[1]);
        o.y = pack_bf16(pa[2], pa[3]);
        *reinterpret_cast<uint2*>(p_bf16 + i) = o;
      }
    } else {
      for (long long j = i; j < n; ++j) {
        float gt;
        if (sizeof(GT) == 2) gt = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[j]);
        else gt = reinterpret_cast<const float*>(grad)[j];
        gt *= gs;
        const float mj = b1 * m[j] + (1.f - b1) * gt;
        const float vj = b2 * v[j] + (1.f - b2) * gt * gt;
        const float pj = p[j] * decay - step * mj / (sqrtf(vj) / bc2_sqrt + eps);
        m[j] = mj; v[j] = vj; p[j] = pj;
        if (p_bf16) p_bf16[j] = __float2bfloat16(pj);
      }
    }
  }
}

// ---------------------------------------------------------------- per-token RL loss
// kind 0 (IPO):    keep = |pi - mu| <= eps_clip
//                  loss = -keep * adv_tau * A * ratio + kl_tau * log_ratio^2
// kind 1 (IcePop): keep = ratio in [lo, hi];  loss = -keep * adv_tau * A * ratio + kl_tau * log_ratio^2
// where ratio = exp(lp - old_lp). Writes the masked per-token loss scaled by `scale[0]`
// (1 / global token count), d(loss)/d(lp), and accumulates sums for metrics:
// stats[0] += loss, [1] += mismatch_kl (r - log r - 1), [2] += masked-out count, [3] += tokens.
__global__ void __launch_bounds__(256)
rl_loss_kernel(const float* __restrict__ lp, const float* __restrict__ old_lp, const float* __restrict__ adv,
               const float* __restrict__ weight /*loss mask or per-token weight*/, float* __restrict__ dlp,
               float* __restrict__ stats, long long n, int kind, float p0, float p1, float adv_tau, float kl_tau,
               const float* __restrict__ scale) {
  const float sc = scale[0];
  float s_loss = 0.f, s_kl = 0.f, s_masked = 0.f, s_tok = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float w = weight[i];
    float d = 0.f;
    if (w != 0.f) {
      const float lr = lp[i] - old_lp[i];
      const float ratio = __expf(lr);
      bool keep;
      if (kind == 0) {
        const float pi = __expf(lp[i]), mu = __expf(old_lp[i]);
        keep = fabsf(pi - mu) <= p0;
      } else {
        keep = ratio >= p0 && ratio <= p1;
      }
      const float a = adv[i];
      const float pg = keep ? -adv_tau * a * ratio : 0.f;
      const float loss = pg + kl_tau * lr * lr;
      d = (pg + 2.f * kl_tau * lr) * w * sc;  // d(ratio)/d(lp) = ratio
      s_loss += loss * w * sc;
      s_kl += (ratio - lr - 1.f) * w;
      s_masked += keep ? 0.f : w;
      s_tok += w;
    }
    dlp[i] = d;
  }
  s_loss = warp_sum(s_loss); s_kl = warp_sum(s_kl); s_masked = warp_sum(s_masked); s_tok = warp_sum(s_tok);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(&stats[0], s_loss);
    atomicAdd(&stats[1], s_kl);
    atomicAdd(&stats[2], s_masked);
    atomicAdd(&stats[3], s_tok);
  }
}

}  // namespace prb

using namespace prb;

static inline unsigned ew_grid(long long work_items, int per_thread = 1) {
  long long b = (work_items / per_thread + 255) / 256;
  const long long cap = 148LL * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<unsigned>(b);
}

// g, u: bf16 [rows, cols] windows with row pitch ld_in; y: bf16 pitch ld_out; cols % 8 == 0.
static int glu_fwd_launch(const void* g, const void* u, void* y, long long rows, int cols, long long ld_in,
                          long long ld_out, int act, float limit, float alpha_act, const int* row_valid, void* stream) {
  if (cols % 8 || ld_in % 8 || ld_out % 8) return -1;
  if (rows == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (row_valid != nullptr) {
    long long blocks = (rows + 7) / 8;
    if (blocks > 148LL * 64) blocks = 148LL * 64;
#define LR(A) glu_fwd_rows_kernel<A><<<static_cast<unsigned>(blocks), 256, 0, s>>>(                                 \
      (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)y, rows, cols, ld_in, ld_out, limit, alpha_act, \
      row_valid)
    if (act == kSwiGLU) LR(kSwiGLU); else if (act == kSwiGLUClamped) LR(kSwiGLUClamped); else LR(kReLU2);
#undef LR
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }
  const unsigned grid = ew_grid(rows * (cols / 8));
#define L(A) glu_fwd_kernel<A><<<grid, 256, 0, s>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)u, \
                                                     (__nv_bfloat16*)y, rows, cols, ld_in, ld_out, limit, alpha_act)
  if (act == kSwiGLU) L(kSwiGLU); else if (act == kSwiGLUClamped) L(kSwiGLUClamped); else L(kReLU2);
#undef L
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_glu_fwd(const void* g, const void* u, void* y, long long rows, int cols, long long ld_in,
                        long long ld_out, int act, float limit, float alpha_act, void* stream) {
  return glu_fwd_launch(g, u, y, rows, cols, ld_in, ld_out, act, limit, alpha_act, nullptr, stream);
}

// Rows r with row_valid[r] < 0 (padding rows of a grouped inference pass) are skipped.
PRB_API int prb_glu_fwd_rowmask(const void* g, const void* u, void* y, long long rows, int cols, long long ld_in,
                                long long ld_out, int act, float limit, float alpha_act, const int* row_valid,
                                void* stream) {
  return glu_fwd_launch(g, u, y, rows, cols, ld_in, ld_out, act, limit, alpha_act, row_valid, stream);
}

PRB_API int prb_glu_bwd(const void* dy, const void* g, const void* u, void* dg, void* du, long long rows, int cols,
                        long long ld_in, long long ld_dy, long long ld_dout, int act, float limit, float alpha_act,
                        void* stream) {
  if (cols % 8 || ld_in % 8 || ld_dy % 8 || ld_dout % 8) return -1;
  if (rows == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = ew_grid(rows * (cols / 8));
#define L(A) glu_bwd_kernel<A><<<grid, 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)g,           \
                                                     (const __nv_bfloat16*)u, (__nv_bfloat16*)dg, (__nv_bfloat16*)du, \
                                                     rows, cols, ld_in, ld_dy, ld_dout, limit, alpha_act)
  if (act == kSwiGLU) L(kSwiGLU); else if (act == kSwiGLUClamped) L(kSwiGLUClamped); else L(kReLU2);
#undef L
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_sumsq(const void* x, long long n, int is_bf16, float* out, void* stream) {
  if (n == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = ew_grid(n, 8);
  if (is_bf16) sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, n, out);
  else sumsq_kernel<float><<<grid, 256, 0, s>>>((const float*)x, n, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_clip_coef(const float* sumsq, float max_norm, float* coef, float* norm_out, void* stream) {
  clip_coef_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sumsq, max_norm, coef, norm_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// hyper: device fp32 [3] = {lr, 1 - b1^t, sqrt(1 - b2^t)}.
PRB_API int prb_adamw(float* p, float* m, float* v, const void* grad, int grad_is_bf16, void* p_bf16, long long n,
                      const float* hyper, float b1, float b2, float eps, float wd, float grad_scale,
                      const float* clip_coef, void* stream) {
  if (n == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = ew_grid(n, 4);
  if (grad_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(p, m, v, (const __nv_bfloat16*)grad, (__nv_bfloat16*)p_bf16, n,
                                                     hyper, b1, b2, eps, wd, grad_scale, clip_coef);
  else
    adamw_kernel<float><<<grid, 256, 0, s>>>(p, m, v, (const float*)grad, (__nv_bfloat16*)p_bf16, n, hyper, b1, b2,
                                             eps, wd, grad_scale, clip_coef);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_rl_loss(const float* lp, const float* old_lp, const float* adv, const float* weight, float* dlp,
                        float* stats, long long n, int kind, float p0, float p1, float adv_tau, float kl_tau,
                        const float* scale, void* stream) {
  if (n == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  rl_loss_kernel<<<ew_grid(n), 256, 0, s>>>(lp, old_lp, adv, weight, dlp, stats, n, kind, p0, p1, adv_tau, kl_tau,
                                            scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
