// MoE routing and token permutation without any host synchronisation.
//
//   router_topk : scores (softmax | sigmoid) over E experts, top-k selection (optionally on
//                 scores + selection bias), weight normalisation, per-expert histogram.
//   plan        : exclusive scan of the 128-padded per-expert counts -> expert_offset[E+1],
//                 block_expert[max_blocks] (-1 past the end) and cursor reset.
//   scatter     : slot[t, j] = position of (token t, choice j) in the expert-sorted, padded
//                 row space; row_src[pos] = t * k + j (-1 for padding rows).
//   gather_rows : permuted[pos, :] = row_src[pos] >= 0 ? x[row_src[pos] / k, :] * (w?) : 0
//   combine     : y[t, :] = sum_j w[t, j] * permuted_out[slot[t, j], :]   (+ residual)
//   combine_bwd_w: dw[t, j] = <dy[t, :], permuted_out[slot[t, j], :]>
//
// Every expert's row range starts on a 128-row boundary so that a grouped-GEMM tile never
// straddles two experts and the k-grouped weight-gradient GEMM can reduce over whole
// 64-row slabs; padding rows are zero.
//
// Replaces TokenChoiceTopKRouter (layers/moe.py:182-322) and the local reorder / permute /
// scatter-add of trainer/distributed/token_dispatcher.py:97-165 in the reference.
#include "common.cuh"

namespace prb {

constexpr int kMaxExperts = 512;
constexpr int kMaxTopK = 16;

// Scores, top-k and weights of token t by one warp; the chosen experts are counted in s_hist (shared memory).
// logits fp32 [T, E]. score_func: 0 softmax, 1 sigmoid. sel_bias (nullable, fp32 [E]) is added for
// selection only. When `forced` (nullable, int32 [T, k]) is given those experts are used instead of
// the top-k (router replay).
__device__ __forceinline__ void router_token(const float* __restrict__ logits, const float* __restrict__ sel_bias,
                                             const int* __restrict__ forced, int* __restrict__ topk_idx,
                                             float* __restrict__ topk_w, float* __restrict__ scores_out, int* s_hist,
                                             long long t, int lane, int E, int k, int score_func, int norm_topk,
                                             float route_scale) {
  constexpr int MAXPL = kMaxExperts / 32;
  float sc[MAXPL];
  const int pl = (E + 31) / 32;
  const float* row = logits + t * E;
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAXPL; ++i) {
    const int e = lane + i * 32;
    sc[i] = (i < pl && e < E) ? row[e] : -INFINITY;
    mx = fmaxf(mx, sc[i]);
  }
  if (score_func == 0) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) {
      const int e = lane + i * 32;
      sc[i] = (i < pl && e < E) ? __expf(sc[i] - mx) : 0.f;
      sum += sc[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) sc[i] *= inv;
  } else {
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) {
      const int e = lane + i * 32;
      sc[i] = (i < pl && e < E) ? 1.f / (1.f + __expf(-sc[i])) : 0.f;
    }
  }
  if (scores_out) {
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) {
      const int e = lane + i * 32;
      if (i < pl && e < E) scores_out[t * E + e] = sc[i];
    }
  }
  float sel[MAXPL];
#pragma unroll
  for (int i = 0; i < MAXPL; ++i) {
    const int e = lane + i * 32;
    sel[i] = (i < pl && e < E) ? sc[i] + (sel_bias ? sel_bias[e] : 0.f) : -INFINITY;
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_e = 0;
  for (int j = 0; j < k; ++j) {
    int be;
    float bw;
    if (forced) {
      be = forced[t * k + j];
      // fetch the score of expert `be` from the lane that holds it
      float cand = 0.f;
#pragma unroll
      for (int i = 0; i < MAXPL; ++i)
        if (lane + i * 32 == be) cand = sc[i];
      bw = __shfl_sync(0xffffffffu, cand, be & 31);
    } else {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < MAXPL; ++i) {
        const int e = lane + i * 32;
        if (sel[i] > bv) {
          bv = sel[i];
          bi = e;
        }
      }
      // warp arg-max; ties resolve to the lowest expert index (matches torch.topk order
      // closely enough for replay, which is exact by construction)
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
          bv = ov;
          bi = oi;
        }
      }
      be = bi;
      float cand = 0.f;
#pragma unroll
      for (int i = 0; i < MAXPL; ++i) {
        if (lane + i * 32 == be) {
          cand = sc[i];
          sel[i] = -INFINITY;
        }
      }
      bw = __shfl_sync(0xffffffffu, cand, be & 31);
    }
    wsum += bw;
    if (lane == j) {
      my_w = bw;
      my_e = be;
    }
  }
  if (lane < k) {
    float w = my_w;
    if (norm_topk) w = w / (wsum + 1e-20f);
    w *= route_scale;
    topk_idx[t * k + lane] = my_e;
    topk_w[t * k + lane] = w;
    atomicAdd(&s_hist[my_e], 1);
  }
}

// One warp per token.
__global__ void __launch_bounds__(256)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ sel_bias,
                   const int* __restrict__ forced, int* __restrict__ topk_idx, float* __restrict__ topk_w,
                   float* __restrict__ scores_out, int* __restrict__ counts, long long T, int E, int k,
                   int score_func, int norm_topk, float route_scale) {
  __shared__ int s_hist[kMaxExperts];
  for (int i = threadIdx.x; i < E; i += blockDim.x) s_hist[i] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long t = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t < T)
    router_token(logits, sel_bias, forced, topk_idx, topk_w, scores_out, s_hist, t, lane, E, k, score_func, norm_topk,
                 route_scale);
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x)
    if (s_hist[i]) atomicAdd(&counts[i], s_hist[i]);
}

// Single CTA. counts[E] -> expert_offset[E+1] (padded to 128), block_expert[max_blocks],
// cursor[E] = 0, total_rows[0] = padded total.
__global__ void __launch_bounds__(512)
moe_plan_kernel(const int* __restrict__ counts, int* __restrict__ expert_offset, int* __restrict__ block_expert,
                int* __restrict__ cursor, int* __restrict__ total_rows, int E, int max_blocks) {
  __shared__ int s_off[kMaxExperts + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + 127) / 128 * 128;
    }
    s_off[E] = acc;
    total_rows[0] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    expert_offset[e] = s_off[e];
    if (e < E) cursor[e] = 0;
  }
  for (int b = threadIdx.x; b < max_blocks; b += blockDim.x) {
    const int row = b * 128;
    int ex = -1;
    if (row < s_off[E]) {
      int lo = 0, hi = E;  // largest e with s_off[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid;
      }
      ex = lo;
      // skip experts with zero rows that share the same offset
      while (ex + 1 < E && s_off[ex + 1] <= row) ++ex;
    }
    block_expert[b] = ex;
  }
}

__global__ void __launch_bounds__(256)
moe_scatter_kernel(const int* __restrict__ topk_idx, const int* __restrict__ expert_offset, int* __restrict__ cursor,
                   int* __restrict__ slot, int* __restrict__ row_src, long long n /* T*k */, int e_lo, int E) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = topk_idx[i] - e_lo;          // experts outside [e_lo, e_lo + E) live on another rank
  if (e < 0 || e >= E) { slot[i] = -1; return; }
  const int pos = expert_offset[e] + atomicAdd(&cursor[e], 1);
  slot[i] = pos;
  row_src[pos] = static_cast<int>(i);
}

// Deterministic variant of the scatter: one CTA per expert walks the (t, j) pairs in index
// order, so that the position of a pair inside its expert does not depend on thread timing.
__global__ void __launch_bounds__(256)
moe_scatter_sorted_kernel(const int* __restrict__ topk_idx, const int* __restrict__ expert_offset,
                          int* __restrict__ slot, int* __restrict__ row_src, long long n, int e_lo) {
  const int e = blockIdx.x;
  __shared__ int s_base;
  __shared__ int s_warp[8];
  if (threadIdx.x == 0) s_base = expert_offset[e];
  __syncthreads();
  for (long long i0 = 0; i0 < n; i0 += blockDim.x) {
    const long long i = i0 + threadIdx.x;
    const bool hit = i < n && topk_idx[i] - e_lo == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, total = 0;
    for (int w = 0; w < 8; ++w) {
      if (w < warp) before += s_warp[w];
      total += s_warp[w];
    }
    if (hit) {
      const int pos = s_base + before + __popc(ballot & ((1u << lane) - 1));
      slot[i] = pos;
      row_src[pos] = static_cast<int>(i);
    }
    __syncthreads();
    if (threadIdx.x == 0) s_base += total;
    __syncthreads();
  }
}

// Decode-sized batches (T * k pairs that one CTA walks in a few rounds): router scores + top-k + histogram +
// padded expert offsets + block -> expert table + row_src fill + scatter in ONE launch of one CTA, instead of a
// fill, the router kernel, a memset, the plan kernel and the scatter kernel. counts need not be zeroed.
__global__ void __launch_bounds__(1024)
moe_route_plan_small_kernel(const float* __restrict__ logits, const float* __restrict__ sel_bias,
                            const int* __restrict__ forced, int* __restrict__ topk_idx, float* __restrict__ topk_w,
                            float* __restrict__ scores_out, int* __restrict__ counts, int* __restrict__ expert_offset,
                            int* __restrict__ block_expert, int* __restrict__ total_rows, int* __restrict__ slot,
                            int* __restrict__ row_src, long long T, int E, int k, int max_blocks, int score_func,
                            int norm_topk, float route_scale) {
  __shared__ int s_hist[kMaxExperts];
  __shared__ int s_off[kMaxExperts + 1];
  __shared__ int s_cur[kMaxExperts];
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    s_hist[i] = 0;
    s_cur[i] = 0;
  }
  // padding marker for the whole row space (valid rows are overwritten by the scatter below)
  for (int i = threadIdx.x; i < max_blocks * 128; i += blockDim.x) row_src[i] = -1;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  for (long long t = threadIdx.x >> 5; t < T; t += blockDim.x >> 5)
    router_token(logits, sel_bias, forced, topk_idx, topk_w, scores_out, s_hist, t, lane, E, k, score_func, norm_topk,
                 route_scale);
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = acc;
      acc += (s_hist[e] + 127) / 128 * 128;
    }
    s_off[E] = acc;
    total_rows[0] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    expert_offset[e] = s_off[e];
    if (e < E) counts[e] = s_hist[e];
  }
  for (int b = threadIdx.x; b < max_blocks; b += blockDim.x) {
    const int row = b * 128;
    int ex = -1;
    if (row < s_off[E]) {
      int lo = 0, hi = E;  // largest e with s_off[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid;
      }
      ex = lo;
      while (ex + 1 < E && s_off[ex + 1] <= row) ++ex;   // skip experts without rows that share the offset
    }
    block_expert[b] = ex;
  }
  // the expert ids were written to global memory by this CTA before the barriers above
  const long long n = T * k;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = topk_idx[i];
    const int pos = s_off[e] + atomicAdd(&s_cur[e], 1);
    slot[i] = pos;
    row_src[pos] = static_cast<int>(i);
  }
}

// out[pos, :] = src row (row_src[pos] / k) of x, scaled by w[row_src[pos]] when w != null;
// zero for padding rows and rows past total_rows. One warp per row, 16-byte vectors.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_src,
                       const float* __restrict__ w, __nv_bfloat16* __restrict__ out, long long max_rows, int cols,
                       int k, const int* __restrict__ total_rows, int zero_pad) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  const int total = total_rows[0];
  for (long long pos = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); pos < max_rows;
       pos += static_cast<long long>(gridDim.x) * 8) {
    if (pos >= total) break;  // rows past the padded total are never read by the grouped GEMM
    const int src = row_src[pos];
    uint4* dst = reinterpret_cast<uint4*>(out + pos * cols);
    if (src < 0) {
      if (zero_pad)
        for (int v = lane; v < nvec; v += 32) dst[v] = make_uint4(0, 0, 0, 0);
    } else {
      const uint4* s = reinterpret_cast<const uint4*>(x + static_cast<long long>(src / k) * cols);
      if (w) {
        const float ww = w[src];
        for (int v = lane; v < nvec; v += 32) {
          uint4 a = s[v];
          float2 f0 = unpack_bf16(a.x), f1 = unpack_bf16(a.y), f2 = unpack_bf16(a.z), f3 = unpack_bf16(a.w);
          a.x = pack_bf16(f0.x * ww, f0.y * ww); a.y = pack_bf16(f1.x * ww, f1.y * ww);
          a.z = pack_bf16(f2.x * ww, f2.y * ww); a.w = pack_bf16(f3.x * ww, f3.y * ww);
          dst[v] = a;
        }
      } else {
        for (int v = lane; v < nvec; v += 32) dst[v] = s[v];
      }
    }
  }
}

// y[t, :] = (residual[t, :]) + sum_j w[t, j] * p[slot[t, j], :];  w == null -> weights of 1.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ p, const int* __restrict__ slot, const float* __restrict__ w,
                   const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ y, long long T, int cols,
                   int k) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  for (long long t = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); t < T;
       t += static_cast<long long>(gridDim.x) * 8) {
    int sl[kMaxTopK];
    float ww[kMaxTopK];
    for (int j = 0; j < k; ++j) {
      sl[j] = slot[t * k + j];               // < 0: the pair's expert lives on another rank (its term comes from there)
      ww[j] = w ? w[t * k + j] : 1.f;
    }
    // blockIdx.y splits the columns when there are few tokens (decode), so that the gather is spread over the SMs
    for (int v = blockIdx.y * 32 + lane; v < nvec; v += 32 * gridDim.y) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (residual) {
        const uint4 a = reinterpret_cast<const uint4*>(residual + t * cols)[v];
        float2 f0 = unpack_bf16(a.x), f1 = unpack_bf16(a.y), f2 = unpack_bf16(a.z), f3 = unpack_bf16(a.w);
        acc[0] = f0.x; acc[1] = f0.y; acc[2] = f1.x; acc[3] = f1.y;
        acc[4] = f2.x; acc[5] = f2.y; acc[6] = f3.x; acc[7] = f3.y;
      }
      for (int j = 0; j < k; ++j) {
        if (sl[j] < 0) continue;
        const uint4 a = reinterpret_cast<const uint4*>(p + static_cast<long long>(sl[j]) * cols)[v];
        float2 f0 = unpack_bf16(a.x), f1 = unpack_bf16(a.y), f2 = unpack_bf16(a.z), f3 = unpack_bf16(a.w);
        acc[0] += ww[j] * f0.x; acc[1] += ww[j] * f0.y; acc[2] += ww[j] * f1.x; acc[3] += ww[j] * f1.y;
        acc[4] += ww[j] * f2.x; acc[5] += ww[j] * f2.y; acc[6] += ww[j] * f3.x; acc[7] += ww[j] * f3.y;
      }
      uint4 o;
      o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
      o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
      reinterpret_cast<uint4*>(y + t * cols)[v] = o;
    }
  }
}

// dw[t, j] = <dy[t, :], p[slot[t, j], :]>  — one warp per (t, j).
__global__ void __launch_bounds__(256)
moe_combine_bwd_w_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ p,
                         const int* __restrict__ slot, float* __restrict__ dw, long long n /* T*k */, int cols,
                         int k) {
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 3;
  for (long long i = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); i < n;
       i += static_cast<long long>(gridDim.x) * 8) {
    const long long t = i / k;
    const uint4* a = reinterpret_cast<const uint4*>(dy + t * cols);
    if (slot[i] < 0) {                       // the pair's expert lives on another rank
      if (lane == 0) dw[i] = 0.f;
      continue;
    }
    const uint4* b = reinterpret_cast<const uint4*>(p + static_cast<long long>(slot[i]) * cols);
    float acc = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 x = a[v], y = b[v];
      float2 x0 = unpack_bf16(x.x), x1 = unpack_bf16(x.y), x2 = unpack_bf16(x.z), x3 = unpack_bf16(x.w);
      float2 y0 = unpack_bf16(y.x), y1 = unpack_bf16(y.y), y2 = unpack_bf16(y.z), y3 = unpack_bf16(y.w);
      acc += x0.x * y0.x + x0.y * y0.y + x1.x * y1.x + x1.y * y1.y + x2.x * y2.x + x2.y * y2.y + x3.x * y3.x +
             x3.y * y3.y;
    }
    acc = warp_sum(acc);
    if (lane == 0) dw[i] = acc;
  }
}

}  // namespace prb

using namespace prb;

static inline unsigned row_grid(long long rows) {
  long long b = (rows + 7) / 8;
  const long long cap = 148LL * 32;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<unsigned>(b);
}

// counts (int32 [E]) must be zeroed by the caller before the call.
PRB_API int prb_router_topk(const float* logits, const float* sel_bias, const int* forced, int* topk_idx,
                            float* topk_w, float* scores_out, int* counts, long long T, int E, int k,
                            int score_func, int norm_topk, float route_scale, void* stream) {
  if (E > kMaxExperts || k > kMaxTopK || k > 32) return -1;
  if (T == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  router_topk_kernel<<<static_cast<unsigned>((T + 7) / 8), 256, 0, s>>>(
      logits, sel_bias, forced, topk_idx, topk_w, scores_out, counts, T, E, k, score_func, norm_topk, route_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Builds expert_offset[E+1], block_expert[max_blocks], slot[T*k], row_src[max_blocks*128]
// from topk_idx and counts. row_src is filled with -1 first. `deterministic` selects the
// order-preserving scatter.
//
// Range form: this rank owns the E experts [e_lo, e_lo + E) of a larger set. `topk_idx` holds global ids, `counts`
// points at the owned experts' counts; pairs of other experts get slot = -1 and no row (the combine skips them),
// `block_expert` holds local ids (0 .. E-1).
PRB_API int prb_moe_plan_range(const int* topk_idx, const int* counts, int* expert_offset, int* block_expert,
                               int* cursor, int* total_rows, int* slot, int* row_src, long long T, int E, int k,
                               int max_blocks, int deterministic, int e_lo, void* stream) {
  if (E > kMaxExperts || E <= 0 || e_lo < 0) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaMemsetAsync(row_src, 0xff, sizeof(int) * static_cast<size_t>(max_blocks) * 128, s);
  moe_plan_kernel<<<1, 512, 0, s>>>(counts, expert_offset, block_expert, cursor, total_rows, E, max_blocks);
  const long long n = T * k;
  if (n > 0) {
    if (deterministic) {
      cudaMemsetAsync(slot, 0xff, sizeof(int) * static_cast<size_t>(n), s);       // pairs no CTA claims stay at -1
      moe_scatter_sorted_kernel<<<E, 256, 0, s>>>(topk_idx, expert_offset, slot, row_src, n, e_lo);
    } else {
      moe_scatter_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(topk_idx, expert_offset, cursor, slot,
                                                                               row_src, n, e_lo, E);
    }
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_moe_plan(const int* topk_idx, const int* counts, int* expert_offset, int* block_expert, int* cursor,
                         int* total_rows, int* slot, int* row_src, long long T, int E, int k, int max_blocks,
                         int deterministic, void* stream) {
  return prb_moe_plan_range(topk_idx, counts, expert_offset, block_expert, cursor, total_rows, slot, row_src, T, E, k,
                            max_blocks, deterministic, 0, stream);
}

PRB_API int prb_moe_gather_rows(const void* x, const int* row_src, const float* w, void* out, long long max_rows,
                                int cols, int k, const int* total_rows, void* stream) {
  if (cols % 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  moe_gather_rows_kernel<<<row_grid(max_rows), 256, 0, s>>>((const __nv_bfloat16*)x, row_src, w,
                                                            (__nv_bfloat16*)out, max_rows, cols, k, total_rows, 1);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Inference variant: padding rows of `out` are left as they are (the grouped GEMMs that follow are told, with the
// same row_src, not to store those rows).
PRB_API int prb_moe_gather_rows_nopad(const void* x, const int* row_src, const float* w, void* out, long long max_rows,
                                      int cols, int k, const int* total_rows, void* stream) {
  if (cols % 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  moe_gather_rows_kernel<<<row_grid(max_rows), 256, 0, s>>>((const __nv_bfloat16*)x, row_src, w,
                                                            (__nv_bfloat16*)out, max_rows, cols, k, total_rows, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_moe_combine(const void* p, const int* slot, const float* w, const void* residual, void* y,
                            long long T, int cols, int k, void* stream) {
  if (cols % 8 || k > kMaxTopK) return -1;
  if (T == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // few tokens: one warp per (token, 256-column slice) instead of one warp per token
  int col_split = 1;
  if (T <= 148 * 8 * 2) {
    col_split = (cols / 8 + 31) / 32;
    if (col_split > 16) col_split = 16;
  }
  moe_combine_kernel<<<dim3(row_grid(T), col_split), 256, 0, s>>>((const __nv_bfloat16*)p, slot, w,
                                                                  (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, T,
                                                                  cols, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_moe_combine_bwd_w(const void* dy, const void* p, const int* slot, float* dw, long long T, int cols,
                                  int k, void* stream) {
  if (cols % 8) return -1;
  if (T == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  moe_combine_bwd_w_kernel<<<row_grid(T * k), 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)p, slot,
                                                           dw, T * k, cols, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// One launch for router + plan when T * k <= 8192 (decode steps). Outputs as prb_router_topk + prb_moe_plan;
// counts / row_src need no initialisation.
PRB_API int prb_moe_route_plan_small(const float* logits, const float* sel_bias, const int* forced, int* topk_idx,
                                     float* topk_w, float* scores_out, int* counts, int* expert_offset,
                                     int* block_expert, int* total_rows, int* slot, int* row_src, long long T, int E,
                                     int k, int max_blocks, int score_func, int norm_topk, float route_scale,
                                     void* stream) {
  if (E > kMaxExperts || k > kMaxTopK || k > 32 || T * k > 8192) return -1;
  if (T == 0) return 0;
  moe_route_plan_small_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      logits, sel_bias, forced, topk_idx, topk_w, scores_out, counts, expert_offset, block_expert, total_rows, slot,
      row_src, T, E, k, max_blocks, score_func, norm_topk, route_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
