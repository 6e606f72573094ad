// One-token recurrence steps of the state-carrying sequence mixers, for the rollout engine's decode steps: every
// running sequence owns a slot of a state pool per layer, and one launch advances all of them in place.
//
//   Mamba-2:            S = exp(dt A) S + dt x B^T,          y = S C + D x           S [H, P, N] per sequence
//   gated delta rule:   S = a S;  S += beta k (v - k^T S)^T,  o = S^T q              S [H, dk, dv] per sequence
//
// Both are bound by one read and one write of the state (fp32). The reference gets these steps from its serving
// stack (vLLM's `selective_state_update` Triton kernel and fla's fused recurrent delta rule).
#include "common.cuh"

namespace prb {

// grid (H, n): one CTA per (sequence, head); a warp owns rows p = warp, warp + W, ...; a lane owns the state
// columns n = lane * 4 + 128 * i (float4), N a multiple of 4.
__global__ void __launch_bounds__(256)
mamba2_step_kernel(float* __restrict__ pool, const int* __restrict__ slots, const float* __restrict__ x,
                   const float* __restrict__ dt, const float* __restrict__ A, const float* __restrict__ B,
                   const float* __restrict__ C, const float* __restrict__ D, float* __restrict__ y, int H, int P, int N,
                   int G) {
  const int h = blockIdx.x, s = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int g = h / (H / G);
  const float dtv = dt[s * H + h];
  const float dA = __expf(dtv * A[h]);
  const float* Bv = B + (static_cast<long long>(s) * G + g) * N;
  const float* Cv = C + (static_cast<long long>(s) * G + g) * N;
  float* S = pool + (static_cast<long long>(slots[s]) * H + h) * P * N;
  const float* xv = x + (static_cast<long long>(s) * H + h) * P;
  float* yv = y + (static_cast<long long>(s) * H + h) * P;
  const float skip = D ? D[h] : 0.f;
  for (int p = warp; p < P; p += nwarps) {
    const float xp = xv[p];
    const float dx = dtv * xp;
    float acc = 0.f;
    float4* row = reinterpret_cast<float4*>(S + static_cast<long long>(p) * N);
    for (int c = lane; c < N / 4; c += 32) {
      float4 st = row[c];
      const float4 b = reinterpret_cast<const float4*>(Bv)[c];
      const float4 cc = reinterpret_cast<const float4*>(Cv)[c];
      st.x = st.x * dA + dx * b.x; st.y = st.y * dA + dx * b.y;
      st.z = st.z * dA + dx * b.z; st.w = st.w * dA + dx * b.w;
      row[c] = st;
      acc += st.x * cc.x + st.y * cc.y + st.z * cc.z + st.w * cc.w;
    }
    acc = warp_sum(acc);
    if (lane == 0) yv[p] = acc + skip * xp;
  }
}

// grid (H, n), one thread per value column v (dv <= 1024); q, k already normalised / scaled by the caller.
__global__ void __launch_bounds__(1024)
delta_step_kernel(float* __restrict__ pool, const int* __restrict__ slots, const float* __restrict__ q,
                  const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ g,
                  const float* __restrict__ beta, float* __restrict__ o, int H, int dk, int dv) {
  extern __shared__ float sm[];            // q [dk], k [dk]
  const int h = blockIdx.x, s = blockIdx.y, col = threadIdx.x;
  const long long sh = static_cast<long long>(s) * H + h;
  for (int i = threadIdx.x; i < dk; i += blockDim.x) {
    sm[i] = q[sh * dk + i];
    sm[dk + i] = k[sh * dk + i];
  }
  __syncthreads();
  if (col >= dv) return;
  const float a = __expf(g[sh]), bt = beta[sh];
  float* S = pool + (static_cast<long long>(slots[s]) * H + h) * dk * dv + col;
  float pred = 0.f;
  for (int i = 0; i < dk; ++i) pred += sm[dk + i] * S[static_cast<long long>(i) * dv];
  pred *= a;
  const float corr = bt * (v[sh * dv + col] - pred);
  float out = 0.f;
  for (int i = 0; i < dk; ++i) {
    const float sn = a * S[static_cast<long long>(i) * dv] + sm[dk + i] * corr;
    S[static_cast<long long>(i) * dv] = sn;
    out += sm[i] * sn;
  }
  o[sh * dv + col] = out;
}

}  // namespace prb

// pool: fp32 [slots_total, H, P, N]; slots: int32 [n] (distinct); x [n, H, P], dt [n, H], A [H], B / C [n, G, N],
// D [H] or null, y [n, H, P]: all fp32 and contiguous. N % 4 == 0, H % G == 0.
PRB_API int prb_mamba2_step(float* pool, const int* slots, const float* x, const float* dt, const float* A,
                            const float* B, const float* C, const float* D, float* y, int n, int H, int P, int N, int G,
                            void* stream) {
  if (n <= 0) return 0;
  if (N % 4 || G <= 0 || H % G || P <= 0) return -2;
  prb::mamba2_step_kernel<<<dim3(H, n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(pool, slots, x, dt, A, B, C, D,
                                                                                         y, H, P, N, G);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// pool: fp32 [slots_total, H, dk, dv]; q, k [n, H, dk] (normalised, q scaled), v [n, H, dv], g (log-decay) and beta
// [n, H], o [n, H, dv]: fp32, contiguous. dv <= 1024.
PRB_API int prb_delta_rule_step(float* pool, const int* slots, const float* q, const float* k, const float* v,
                                const float* g, const float* beta, float* o, int n, int H, int dk, int dv,
                                void* stream) {
  if (n <= 0) return 0;
  if (dv > 1024 || dv <= 0 || dk <= 0) return -2;
  const int threads = (dv + 31) / 32 * 32;
  prb::delta_step_kernel<<<dim3(H, n), threads, 2 * dk * sizeof(float), reinterpret_cast<cudaStream_t>(stream)>>>(
      pool, slots, q, k, v, g, beta, o, H, dk, dv);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
