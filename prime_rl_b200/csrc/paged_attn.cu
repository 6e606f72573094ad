// Paged-attention decode: one query token per sequence against its paged bf16 KV cache
// (pages of `page_size` tokens, per-sequence block tables), GQA aware: the G query heads
// that share a KV head are processed together so that K and V are streamed from HBM once.
// Bandwidth-bound; optional split of the context over several CTAs (partials merged by a
// second kernel) keeps all SMs busy when batch x kv_heads is small.
//
// Per 32-key chunk and warp:
//   phase A  lane <-> key   : the lane reads its key's whole 256-byte K row, dots it with the
//                             G query rows held in shared memory (broadcast reads), then the
//                             warp does the online-softmax bookkeeping per head
//   phase B  lane <-> 4 dims: V rows are read coalesced, every lane accumulates its 4 output
//                             dims for all G heads with the probabilities staged in shared memory
//
// Takes the place of vLLM's paged attention kernel in the reference's inference stack.
#include "common.cuh"

namespace prb {

constexpr int kPdD = 128;
constexpr int kPdWarps = 4;

struct PagedParams {
  const __nv_bfloat16* q;       // [B, Hq, D]
  const __nv_bfloat16* kpool;   // [pages, page_size, Hkv, D]
  const __nv_bfloat16* vpool;
  const int* block_tables;      // [B, max_blocks]
  const int* ctx_lens;          // [B]
  __nv_bfloat16* out;           // [B, Hq, D]
  float* o_part;                // [B, Hq, S, D]   (S > 1)
  float* ml_part;               // [B, Hq, S, 2]
  float scale;
  int B, Hq, Hkv, page_size, max_blocks, splits;
};

template <int G>
__global__ void __launch_bounds__(kPdWarps * 32)
paged_decode_kernel(const PagedParams p) {
  __shared__ float s_q[G][kPdD];
  __shared__ float s_p[kPdWarps][G][32];
  __shared__ float s_m[kPdWarps][G], s_l[kPdWarps][G];
  __shared__ float s_o[kPdWarps][G][kPdD];
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctx = p.ctx_lens[b];
  // this CTA's key range (32-key chunks are dealt to the splits round robin by ranges)
  const int chunks = (ctx + 31) / 32;
  const int per = (chunks + p.splits - 1) / p.splits;
  const int c_begin = split * per, c_end = min(chunks, c_begin + per);

  for (int i = threadIdx.x; i < G * kPdD; i += blockDim.x) {
    const int g = i / kPdD, d = i - g * kPdD;
    s_q[g][d] = __bfloat162float(p.q[(static_cast<long long>(b) * p.Hq + kvh * G + g) * kPdD + d]) * p.scale;
  }
  __syncthreads();

  float m[G], l[G], o[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
    o[g][0] = o[g][1] = o[g][2] = o[g][3] = 0.f;
  }
  const int* table = p.block_tables + static_cast<long long>(b) * p.max_blocks;
  const long long row_stride = static_cast<long long>(p.Hkv) * kPdD;

  for (int c = c_begin + warp; c < c_end; c += kPdWarps) {
    const int key = c * 32 + lane;
    const bool valid = key < ctx;
    long long base = 0;
    if (valid) {
      const int page = table[key / p.page_size];
      base = (static_cast<long long>(page) * p.page_size + key % p.page_size) * row_stride +
             static_cast<long long>(kvh) * kPdD;
    }
    // ---- phase A: scores of this lane's key for all G heads
    float sc[G];
#pragma unroll
    for (int g = 0; g < G; ++g) sc[g] = 0.f;
    if (valid) {
      const uint4* kr = reinterpret_cast<const uint4*>(p.kpool + base);
#pragma unroll 4
      for (int ch = 0; ch < kPdD / 8; ++ch) {
        const uint4 kv = kr[ch];
        const float2 k0 = unpack_bf16(kv.x), k1 = unpack_bf16(kv.y), k2 = unpack_bf16(kv.z), k3 = unpack_bf16(kv.w);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float4 qa = *reinterpret_cast<const float4*>(&s_q[g][ch * 8]);
          const float4 qb = *reinterpret_cast<const float4*>(&s_q[g][ch * 8 + 4]);
          sc[g] += qa.x * k0.x + qa.y * k0.y + qa.z * k1.x + qa.w * k1.y + qb.x * k2.x + qb.y * k2.y + qb.z * k3.x +
                   qb.w * k3.y;
        }
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float s = valid ? sc[g] : -INFINITY;
      const float mn = fmaxf(m[g], warp_max(s));
      const float pr = valid ? __expf(s - mn) : 0.f;
      const float alpha = __expf(m[g] - mn);      // m = -inf on the first chunk -> 0
      l[g] = l[g] * alpha + warp_sum(pr);
      o[g][0] *= alpha; o[g][1] *= alpha; o[g][2] *= alpha; o[g][3] *= alpha;
      m[g] = mn;
      s_p[warp][g][lane] = pr;
    }
    __syncwarp();
    // ---- phase B: accumulate V, lane owns dims [4 lane, 4 lane + 4)
    const int nvalid = min(32, ctx - c * 32);
    for (int i = 0; i < nvalid; ++i) {
      const long long vb = __shfl_sync(0xffffffffu, base, i);
      const uint2 vv = *reinterpret_cast<const uint2*>(p.vpool + vb + lane * 4);
      const float2 v0 = unpack_bf16(vv.x), v1 = unpack_bf16(vv.y);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pg = s_p[warp][g][i];
        o[g][0] += pg * v0.x; o[g][1] += pg * v0.y; o[g][2] += pg * v1.x; o[g][3] += pg * v1.y;
      }
    }
    __syncwarp();
  }

  // ---- combine the warps of this CTA
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
    *reinterpret_cast<float4*>(&s_o[warp][g][lane * 4]) = make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * kPdD; i += blockDim.x) {
    const int g = i / kPdD, d = i - g * kPdD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kPdWarps; ++w) M = fmaxf(M, s_m[w][g]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kPdWarps; ++w) {
      const float a = (s_m[w][g] == -INFINITY) ? 0.f : __expf(s_m[w][g] - M);
      L += s_l[w][g] * a;
      O += s_o[w][g][d] * a;
    }
    const long long head = static_cast<long long>(b) * p.Hq + kvh * G + g;
    if (p.splits == 1) {
      p.out[head * kPdD + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
    } else {
      p.o_part[(head * p.splits + split) * kPdD + d] = O;
      if (d == 0) {
        p.ml_part[(head * p.splits + split) * 2] = M;
        p.ml_part[(head * p.splits + split) * 2 + 1] = L;
      }
    }
  }
}

__global__ void __launch_bounds__(kPdD)
paged_decode_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                          __nv_bfloat16* __restrict__ out, int splits) {
  const long long head = blockIdx.x;
  const int d = threadIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, ml_part[(head * splits + s) * 2]);
  float L = 0.f, O = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = ml_part[(head * splits + s) * 2];
    const float a = (ms == -INFINITY) ? 0.f : __expf(ms - M);
    L += ml_part[(head * splits + s) * 2 + 1] * a;
    O += o_part[(head * splits + s) * kPdD + d] * a;
  }
  out[head * kPdD + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
}

}  // namespace prb

// q: bf16 [B, Hq, 128]; kpool / vpool: bf16 [pages, page_size, Hkv, 128]; block_tables: int32
// [B, max_blocks]; ctx_lens: int32 [B]; out: bf16 [B, Hq, 128]. For splits > 1 the caller gives
// o_part fp32 [B, Hq, splits, 128] and ml_part fp32 [B, Hq, splits, 2].
PRB_API int prb_paged_decode(const void* q, const void* kpool, const void* vpool, const int* block_tables,
                             const int* ctx_lens, void* out, float* o_part, float* ml_part, int B, int Hq, int Hkv,
                             int head_dim, int page_size, int max_blocks, int splits, float scale, void* stream_) {
  using namespace prb;
  if (head_dim != kPdD || Hq % Hkv) return -2;
  if (B <= 0) return 0;
  if (splits < 1 || (splits > 1 && (o_part == nullptr || ml_part == nullptr))) return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  PagedParams p;
  p.q = (const __nv_bfloat16*)q; p.kpool = (const __nv_bfloat16*)kpool; p.vpool = (const __nv_bfloat16*)vpool;
  p.block_tables = block_tables; p.ctx_lens = ctx_lens; p.out = (__nv_bfloat16*)out;
  p.o_part = o_part; p.ml_part = ml_part; p.scale = scale;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size; p.max_blocks = max_blocks; p.splits = splits;
  dim3 grid(B, Hkv, splits);
  const int G = Hq / Hkv;
  switch (G) {
    case 1: paged_decode_kernel<1><<<grid, kPdWarps * 32, 0, stream>>>(p); break;
    case 2: paged_decode_kernel<2><<<grid, kPdWarps * 32, 0, stream>>>(p); break;
    case 4: paged_decode_kernel<4><<<grid, kPdWarps * 32, 0, stream>>>(p); break;
    case 8: paged_decode_kernel<8><<<grid, kPdWarps * 32, 0, stream>>>(p); break;
    default: return -4;
  }
  if (splits > 1)
    paged_decode_merge_kernel<<<static_cast<unsigned>(B) * Hq, kPdD, 0, stream>>>(o_part, ml_part,
                                                                                 (__nv_bfloat16*)out, splits);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
