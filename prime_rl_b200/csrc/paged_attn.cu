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
  // Shared-prefix decode (optional, tensor-core kernels only). Sequences whose leading pages are the same
  // physical pages (samples of one prompt) form groups of up to 8: the group kernel reads those pages once
  // for all members and leaves a partial result per member in split slots [splits, splits + prefix_splits);
  // the per-sequence kernel then starts at page page_begin[b]. The merge kernel folds both.
  const int* page_begin;        // [B] first page the per-sequence kernel reads (nullptr = 0 everywhere)
  const int* group_seqs;        // [groups, 8] member sequence indices, -1 = unused slot
  const int* group_pages;       // [groups] number of leading pages the members share (0 = no group in this slot)
  int prefix_splits, total_splits;
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


// ---------------------------------------------------------------------------------------------
// Tensor-core variant for 16-token pages and up to 8 query heads per KV head. With a GQA group
// of 8 the op needs 8 FLOP per KV byte, more than the fp32 pipes deliver at HBM speed, so the
// scores and the P V product run on mma.sync m16n8k16 (rows 8..15 of the M = 16 tile are zero).
// One CTA = one (sequence, KV head, split), four warps; a warp owns whole pages: it copies the
// page's K and V rows (16 x 256 B each) into its private, double-buffered, XOR-swizzled shared
// memory with cp.async, reads operand fragments with ldmatrix (V transposed), keeps the online
// softmax state of its pages in registers; the warps' partial results are merged at the end.
constexpr int kPmPage = 16;
constexpr int kPmWarpBytes = 2 * 2 * kPmPage * kPdD * 2;   // 2 buffers x (K, V) x 4 KB = 16 KB

__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int G>
__global__ void __launch_bounds__(kPdWarps * 32)
paged_decode_mma_kernel(const PagedParams p) {
  extern __shared__ __align__(128) uint8_t pm_smem[];
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, j = lane & 3;        // fragment row (query head of the group) / column pair
  const int ctx = p.ctx_lens[b];
  const int pages = (ctx + kPmPage - 1) / kPmPage;
  const int first = p.page_begin ? min(p.page_begin[b], pages) : 0;            // pages before it: the group kernel
  const int per = (pages - first + p.splits - 1) / p.splits;
  const int pg_begin = first + split * per, pg_end = min(pages, pg_begin + per);
  const int* table = p.block_tables + static_cast<long long>(b) * p.max_blocks;
  const long long row_stride = static_cast<long long>(p.Hkv) * kPdD;          // elements between keys of a page
  const uint32_t sbase = smem_u32(pm_smem) + warp * kPmWarpBytes;
  const int S = p.total_splits > 0 ? p.total_splits : p.splits;               // slots per head in the partial arrays
  const float scale_log2 = p.scale * 1.4426950408889634f;

  // Q fragments: row g of the A tile is query head g of this KV head's group (rows >= G are zero)
  uint32_t qa[8][2];
  {
    const __nv_bfloat16* qrow = p.q + (static_cast<long long>(b) * p.Hq + kvh * G + (g < G ? g : 0)) * kPdD;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      qa[kk][0] = (g < G) ? *reinterpret_cast<const uint32_t*>(qrow + 16 * kk + 2 * j) : 0u;
      qa[kk][1] = (g < G) ? *reinterpret_cast<const uint32_t*>(qrow + 16 * kk + 8 + 2 * j) : 0u;
    }
  }
  float o[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m = -INFINITY, l = 0.f;                 // running max (log2 domain) / sum of row g

  // copy one page (K and V rows of this KV head) into buffer `buf`: 512 chunks of 16 bytes
  auto issue_page = [&](int pg, int buf) {
    const long long base = static_cast<long long>(table[pg]) * kPmPage * row_stride + static_cast<long long>(kvh) * kPdD;
    const uint32_t kdst = sbase + buf * (2 * kPmPage * kPdD * 2), vdst = kdst + kPmPage * kPdD * 2;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = lane + 32 * i;              // chunk id: key = c / 16, 16-byte chunk of the row = c % 16
      const int key = c >> 4, ch = c & 15;
      const long long off = base + key * row_stride + ch * 8;
      const uint32_t sw = key * 256 + ((ch ^ (key & 7)) << 4);
      cp_async16(kdst + sw, p.kpool + off);
      cp_async16(vdst + sw, p.vpool + off);
    }
    cp_async_commit();
  };

  int pg = pg_begin + warp;
  if (pg < pg_end) issue_page(pg, 0);
  int buf = 0;
  for (; pg < pg_end; pg += kPdWarps, buf ^= 1) {
    const int nxt = pg + kPdWarps;
    if (nxt < pg_end) { issue_page(nxt, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncwarp();
    const uint32_t ks = sbase + buf * (2 * kPmPage * kPdD * 2), vs = ks + kPmPage * kPdD * 2;
    // ---- S = Q K^T for the 16 keys of the page (two n-tiles of 8 keys)
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const int key = 8 * (lane >> 4) + (lane & 7);          // matrices 0, 1 -> keys 0..7; 2, 3 -> keys 8..15
      const int hi = (lane >> 3) & 1;                        // second 8 columns of the k-step
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(ks + key * 256 + (((2 * kk + hi) ^ (key & 7)) << 4), b0, b1, b2, b3);
        mma_16816(s0, qa[kk][0], 0u, qa[kk][1], 0u, b0, b1);
        mma_16816(s1, qa[kk][0], 0u, qa[kk][1], 0u, b2, b3);
      }
    }
    // ---- online softmax of row g: this thread holds keys 2j, 2j+1 (s0) and 8+2j, 9+2j (s1)
    const int k0 = pg * kPmPage + 2 * j;
    float x0 = (k0 < ctx) ? s0[0] * scale_log2 : -INFINITY, x1 = (k0 + 1 < ctx) ? s0[1] * scale_log2 : -INFINITY;
    float x2 = (k0 + 8 < ctx) ? s1[0] * scale_log2 : -INFINITY, x3 = (k0 + 9 < ctx) ? s1[1] * scale_log2 : -INFINITY;
    float mx = fmaxf(fmaxf(x0, x1), fmaxf(x2, x3));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m, mx);                            // finite: key pg * 16 < ctx exists
    const float alpha = exp2f(m - mn);
    const float p0 = exp2f(x0 - mn), p1 = exp2f(x1 - mn), p2 = exp2f(x2 - mn), p3 = exp2f(x3 - mn);
    float rs = p0 + p1 + p2 + p3;
    rs += __shfl_xor_sync(0xffffffffu, rs, 1);
    rs += __shfl_xor_sync(0xffffffffu, rs, 2);
    l = l * alpha + rs;
    m = mn;
    const uint32_t pa0 = pack_bf16(p0, p1), pa2 = pack_bf16(p2, p3);   // A fragment of P (rows 8..15 zero)
    // ---- O = O * alpha + P V
    {
      const int key = 8 * ((lane >> 3) & 1) + (lane & 7);    // matrices 0, 2 -> keys 0..7; 1, 3 -> keys 8..15
      const int sub = lane >> 4;                             // second d tile of the pair
#pragma unroll
      for (int pr = 0; pr < 8; ++pr) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vs + key * 256 + (((2 * pr + sub) ^ (key & 7)) << 4), b0, b1, b2, b3);
        o[2 * pr][0] *= alpha; o[2 * pr][1] *= alpha;
        o[2 * pr + 1][0] *= alpha; o[2 * pr + 1][1] *= alpha;
        mma_16816(o[2 * pr], pa0, 0u, pa2, 0u, b0, b1);
        mma_16816(o[2 * pr + 1], pa0, 0u, pa2, 0u, b2, b3);
      }
    }
    __syncwarp();
  }

  // ---- merge the four warps: row g < G, this thread holds d = 8 n + 2 j, 2 j + 1 of every n-tile
  __syncthreads();                                            // all cp.async traffic is done, smem is reusable
  float* s_m = reinterpret_cast<float*>(pm_smem);             // [warps][8]
  float* s_l = s_m + kPdWarps * 8;
  float* s_o = s_l + kPdWarps * 8;                            // [warps][8][128]
  if (g < G) {
    if (j == 0) { s_m[warp * 8 + g] = m; s_l[warp * 8 + g] = l; }
#pragma unroll
    for (int n = 0; n < 16; ++n)
      *reinterpret_cast<float2*>(&s_o[(warp * 8 + g) * kPdD + 8 * n + 2 * j]) = make_float2(o[n][0], o[n][1]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * kPdD; i += blockDim.x) {
    const int gg = i / kPdD, d = i - gg * kPdD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kPdWarps; ++w) M = fmaxf(M, s_m[w * 8 + gg]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kPdWarps; ++w) {
      const float a = (s_m[w * 8 + gg] == -INFINITY) ? 0.f : exp2f(s_m[w * 8 + gg] - M);
      L += s_l[w * 8 + gg] * a;
      O += s_o[(w * 8 + gg) * kPdD + d] * a;
    }
    const long long head = static_cast<long long>(b) * p.Hq + kvh * G + gg;
    if (S == 1) {
      p.out[head * kPdD + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
    } else {
      p.o_part[(head * S + split) * kPdD + d] = O;
      if (d == 0) {
        // the merge kernel works in the natural-log domain
        p.ml_part[(head * S + split) * 2] = (M == -INFINITY) ? -INFINITY : M * 0.6931471805599453f;
        p.ml_part[(head * S + split) * 2 + 1] = L;
      }
    }
  }
}

// Shared-prefix pass: one CTA = (group, KV head, slice of the shared pages). The four warps own the four
// 16-row query tiles of the group (rows 0..7: the G heads of member 2w, rows 8..15: member 2w + 1), so the full
// M = 16 of the mma tile is used; K and V pages are copied into shared memory ONCE per CTA (four pages per
// stage, double buffered) and read by all four warps. Every key of a shared page is valid for every member
// (shared pages are full), so no masking. Results are per-member partials in slots [splits, splits + prefix_splits).
constexpr int kPxPages = 4;                                         // pages per stage
constexpr int kPxPageBytes = 2 * kPmPage * kPdD * 2;                // K and V rows of one page: 8 KB
constexpr int kPxStageBytes = kPxPages * kPxPageBytes;              // 32 KB

template <int G>
__global__ void __launch_bounds__(kPdWarps * 32)
paged_prefix_mma_kernel(const PagedParams p) {
  extern __shared__ __align__(128) uint8_t pm_smem[];
  const int grp = blockIdx.x, kvh = blockIdx.y, ps = blockIdx.z;
  const int shared_pages = p.group_pages[grp];
  if (shared_pages <= 0) return;                              // uniform for the CTA: no barrier was reached yet
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, j = lane & 3;
  const int* members = p.group_seqs + grp * 8;
  const int leader = members[0];
  const int seq_a = members[2 * warp], seq_b = members[2 * warp + 1];
  const int per = (shared_pages + p.prefix_splits - 1) / p.prefix_splits;
  const int pg_begin = ps * per, pg_end = min(shared_pages, pg_begin + per);
  const int* table = p.block_tables + static_cast<long long>(leader) * p.max_blocks;
  const long long row_stride = static_cast<long long>(p.Hkv) * kPdD;
  const uint32_t sbase = smem_u32(pm_smem);
  const float scale_log2 = p.scale * 1.4426950408889634f;

  // Q fragments of both members (rows g and g + 8 of the A tile); absent members and heads >= G give zero rows
  uint32_t qa[8][2], qb[8][2];
  {
    const bool va = seq_a >= 0 && g < G, vb = seq_b >= 0 && g < G;
    const __nv_bfloat16* ra = p.q + (static_cast<long long>(va ? seq_a : 0) * p.Hq + kvh * G + (g < G ? g : 0)) * kPdD;
    const __nv_bfloat16* rb = p.q + (static_cast<long long>(vb ? seq_b : 0) * p.Hq + kvh * G + (g < G ? g : 0)) * kPdD;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      qa[kk][0] = va ? *reinterpret_cast<const uint32_t*>(ra + 16 * kk + 2 * j) : 0u;
      qa[kk][1] = va ? *reinterpret_cast<const uint32_t*>(ra + 16 * kk + 8 + 2 * j) : 0u;
      qb[kk][0] = vb ? *reinterpret_cast<const uint32_t*>(rb + 16 * kk + 2 * j) : 0u;
      qb[kk][1] = vb ? *reinterpret_cast<const uint32_t*>(rb + 16 * kk + 8 + 2 * j) : 0u;
    }
  }
  float o[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_a = -INFINITY, l_a = 0.f, m_b = -INFINITY, l_b = 0.f;

  // the CTA copies up to kPxPages pages into stage `buf`: 2 x 256 16-byte chunks per page over 128 threads
  auto issue_stage = [&](int pg0, int buf) {
    const int n_pages = min(kPxPages, pg_end - pg0);
    for (int c = threadIdx.x; c < n_pages * 256; c += kPdWarps * 32) {
      const int page = c >> 8, r = c & 255;                   // r: key = r / 16, 16-byte chunk of the row = r % 16
      const int key = r >> 4, ch = r & 15;
      const long long off = static_cast<long long>(table[pg0 + page]) * kPmPage * row_stride +
                            static_cast<long long>(kvh) * kPdD + key * row_stride + ch * 8;
      const uint32_t kdst = sbase + buf * kPxStageBytes + page * kPxPageBytes;
      const uint32_t sw = key * 256 + ((ch ^ (key & 7)) << 4);
      cp_async16(kdst + sw, p.kpool + off);
      cp_async16(kdst + kPmPage * kPdD * 2 + sw, p.vpool + off);
    }
    cp_async_commit();
  };

  int buf = 0;
  if (pg_begin < pg_end) issue_stage(pg_begin, 0);
  for (int pg0 = pg_begin; pg0 < pg_end; pg0 += kPxPages, buf ^= 1) {
    const int nxt = pg0 + kPxPages;
    if (nxt < pg_end) { issue_stage(nxt, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();                                          // every thread's copies of this stage have landed
    const int n_pages = min(kPxPages, pg_end - pg0);
    if (n_pages == kPxPages) {
      // a full stage: one softmax step over its 64 keys (8 independent score tiles, one rescale of the output)
      static_assert(kPxPages == 4, "the full-stage path is written for four pages of 16 keys");
      float s[8][4];
#pragma unroll
      for (int t = 0; t < 8; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
      {
        const int key = 8 * (lane >> 4) + (lane & 7);
        const int hi = (lane >> 3) & 1;
#pragma unroll
        for (int page = 0; page < 4; ++page) {
          const uint32_t ks = sbase + buf * kPxStageBytes + page * kPxPageBytes;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(ks + key * 256 + (((2 * kk + hi) ^ (key & 7)) << 4), b0, b1, b2, b3);
            mma_16816(s[2 * page], qa[kk][0], qb[kk][0], qa[kk][1], qb[kk][1], b0, b1);
            mma_16816(s[2 * page + 1], qa[kk][0], qb[kk][0], qa[kk][1], qb[kk][1], b2, b3);
          }
        }
      }
      float mxa = -INFINITY, mxb = -INFINITY;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        mxa = fmaxf(mxa, fmaxf(s[t][0], s[t][1]));
        mxb = fmaxf(mxb, fmaxf(s[t][2], s[t][3]));
      }
      mxa = fmaxf(mxa, __shfl_xor_sync(0xffffffffu, mxa, 1));
      mxa = fmaxf(mxa, __shfl_xor_sync(0xffffffffu, mxa, 2));
      mxb = fmaxf(mxb, __shfl_xor_sync(0xffffffffu, mxb, 1));
      mxb = fmaxf(mxb, __shfl_xor_sync(0xffffffffu, mxb, 2));
      const float na = fmaxf(m_a, mxa * scale_log2), nb = fmaxf(m_b, mxb * scale_log2);
      const float alpha_a = exp2f(m_a - na), alpha_b = exp2f(m_b - nb);
      float rsa = 0.f, rsb = 0.f;
      uint32_t pa[8], pb[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const float a0 = exp2f(s[t][0] * scale_log2 - na), a1 = exp2f(s[t][1] * scale_log2 - na);
        const float b0 = exp2f(s[t][2] * scale_log2 - nb), b1 = exp2f(s[t][3] * scale_log2 - nb);
        rsa += a0 + a1;
        rsb += b0 + b1;
        pa[t] = pack_bf16(a0, a1);
        pb[t] = pack_bf16(b0, b1);
      }
      rsa += __shfl_xor_sync(0xffffffffu, rsa, 1);
      rsa += __shfl_xor_sync(0xffffffffu, rsa, 2);
      rsb += __shfl_xor_sync(0xffffffffu, rsb, 1);
      rsb += __shfl_xor_sync(0xffffffffu, rsb, 2);
      l_a = l_a * alpha_a + rsa; m_a = na;
      l_b = l_b * alpha_b + rsb; m_b = nb;
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        o[n][0] *= alpha_a; o[n][1] *= alpha_a; o[n][2] *= alpha_b; o[n][3] *= alpha_b;
      }
      {
        const int key = 8 * ((lane >> 3) & 1) + (lane & 7);
        const int sub = lane >> 4;
#pragma unroll
        for (int page = 0; page < 4; ++page) {
          const uint32_t vs = sbase + buf * kPxStageBytes + page * kPxPageBytes + kPmPage * kPdD * 2;
#pragma unroll
          for (int pr = 0; pr < 8; ++pr) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(vs + key * 256 + (((2 * pr + sub) ^ (key & 7)) << 4), b0, b1, b2, b3);
            mma_16816(o[2 * pr], pa[2 * page], pb[2 * page], pa[2 * page + 1], pb[2 * page + 1], b0, b1);
            mma_16816(o[2 * pr + 1], pa[2 * page], pb[2 * page], pa[2 * page + 1], pb[2 * page + 1], b2, b3);
          }
        }
      }
    } else
    for (int page = 0; page < n_pages; ++page) {
      const uint32_t ks = sbase + buf * kPxStageBytes + page * kPxPageBytes, vs = ks + kPmPage * kPdD * 2;
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      {
        const int key = 8 * (lane >> 4) + (lane & 7);
        const int hi = (lane >> 3) & 1;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(ks + key * 256 + (((2 * kk + hi) ^ (key & 7)) << 4), b0, b1, b2, b3);
          mma_16816(s0, qa[kk][0], qb[kk][0], qa[kk][1], qb[kk][1], b0, b1);
          mma_16816(s1, qa[kk][0], qb[kk][0], qa[kk][1], qb[kk][1], b2, b3);
        }
      }
      // rows g (member a): s0[0..1] = keys 2j, 2j+1 and s1[0..1] = keys 8+2j, 9+2j; rows g + 8 (member b): [2..3]
      const float xa0 = s0[0] * scale_log2, xa1 = s0[1] * scale_log2, xa2 = s1[0] * scale_log2, xa3 = s1[1] * scale_log2;
      const float xb0 = s0[2] * scale_log2, xb1 = s0[3] * scale_log2, xb2 = s1[2] * scale_log2, xb3 = s1[3] * scale_log2;
      float mxa = fmaxf(fmaxf(xa0, xa1), fmaxf(xa2, xa3)), mxb = fmaxf(fmaxf(xb0, xb1), fmaxf(xb2, xb3));
      mxa = fmaxf(mxa, __shfl_xor_sync(0xffffffffu, mxa, 1));
      mxa = fmaxf(mxa, __shfl_xor_sync(0xffffffffu, mxa, 2));
      mxb = fmaxf(mxb, __shfl_xor_sync(0xffffffffu, mxb, 1));
      mxb = fmaxf(mxb, __shfl_xor_sync(0xffffffffu, mxb, 2));
      const float na = fmaxf(m_a, mxa), nb = fmaxf(m_b, mxb);
      const float alpha_a = exp2f(m_a - na), alpha_b = exp2f(m_b - nb);
      const float pa0 = exp2f(xa0 - na), pa1 = exp2f(xa1 - na), pa2 = exp2f(xa2 - na), pa3 = exp2f(xa3 - na);
      const float pb0 = exp2f(xb0 - nb), pb1 = exp2f(xb1 - nb), pb2 = exp2f(xb2 - nb), pb3 = exp2f(xb3 - nb);
      float rsa = pa0 + pa1 + pa2 + pa3, rsb = pb0 + pb1 + pb2 + pb3;
      rsa += __shfl_xor_sync(0xffffffffu, rsa, 1);
      rsa += __shfl_xor_sync(0xffffffffu, rsa, 2);
      rsb += __shfl_xor_sync(0xffffffffu, rsb, 1);
      rsb += __shfl_xor_sync(0xffffffffu, rsb, 2);
      l_a = l_a * alpha_a + rsa; m_a = na;
      l_b = l_b * alpha_b + rsb; m_b = nb;
      // A fragment of P: a0 = (row g, keys 2j..), a1 = (row g + 8, keys 2j..), a2 / a3 the same for keys 8 + 2j..
      const uint32_t fa0 = pack_bf16(pa0, pa1), fa1 = pack_bf16(pb0, pb1), fa2 = pack_bf16(pa2, pa3),
                     fa3 = pack_bf16(pb2, pb3);
      {
        const int key = 8 * ((lane >> 3) & 1) + (lane & 7);
        const int sub = lane >> 4;
#pragma unroll
        for (int pr = 0; pr < 8; ++pr) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(vs + key * 256 + (((2 * pr + sub) ^ (key & 7)) << 4), b0, b1, b2, b3);
          o[2 * pr][0] *= alpha_a; o[2 * pr][1] *= alpha_a; o[2 * pr][2] *= alpha_b; o[2 * pr][3] *= alpha_b;
          o[2 * pr + 1][0] *= alpha_a; o[2 * pr + 1][1] *= alpha_a;
          o[2 * pr + 1][2] *= alpha_b; o[2 * pr + 1][3] *= alpha_b;
          mma_16816(o[2 * pr], fa0, fa1, fa2, fa3, b0, b1);
          mma_16816(o[2 * pr + 1], fa0, fa1, fa2, fa3, b2, b3);
        }
      }
    }
    __syncthreads();                                          // the stage may be overwritten by the next copy
  }
  // each warp owns its rows: the partials of member a (rows g) and member b (rows g + 8) go out directly
  if (g < G) {
    const int S = p.total_splits, slot = p.splits + ps;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int seq = half ? seq_b : seq_a;
      if (seq < 0) continue;
      const float mm = half ? m_b : m_a, ll = half ? l_b : l_a;
      const long long head = static_cast<long long>(seq) * p.Hq + kvh * G + g;
#pragma unroll
      for (int n = 0; n < 16; ++n)
        *reinterpret_cast<float2*>(&p.o_part[(head * S + slot) * kPdD + 8 * n + 2 * j]) =
            make_float2(o[n][2 * half], o[n][2 * half + 1]);
      if (j == 0) {
        p.ml_part[(head * S + slot) * 2] = (mm == -INFINITY) ? -INFINITY : mm * 0.6931471805599453f;
        p.ml_part[(head * S + slot) * 2 + 1] = ll;
      }
    }
  }
}

// One warp per head, eight heads per CTA: lane l owns output channels 4 l .. 4 l + 3 (one float4 per partial).
constexpr int kMergeHeads = 8;
__global__ void __launch_bounds__(32 * kMergeHeads)
paged_decode_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                          __nv_bfloat16* __restrict__ out, int splits, int own_splits, int heads_per_seq,
                          const int* __restrict__ page_begin, long long total_heads) {
  // `splits` slots per head; slots >= own_splits belong to the shared-prefix pass and only count for sequences
  // that are in a group (page_begin > 0): the others never wrote them
  static_assert(kPdD == 128, "one float4 per lane");
  const long long head = static_cast<long long>(blockIdx.x) * kMergeHeads + (threadIdx.x >> 5);
  if (head >= total_heads) return;
  const int lane = threadIdx.x & 31;
  int used = splits;
  if (own_splits < splits && (page_begin == nullptr || page_begin[head / heads_per_seq] <= 0)) used = own_splits;
  float M = -INFINITY;
  for (int s = 0; s < used; ++s) M = fmaxf(M, ml_part[(head * splits + s) * 2]);
  float L = 0.f;
  float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < used; ++s) {
    const float ms = ml_part[(head * splits + s) * 2];
    const float a = (ms == -INFINITY) ? 0.f : __expf(ms - M);
    L += ml_part[(head * splits + s) * 2 + 1] * a;
    const float4 o = *reinterpret_cast<const float4*>(o_part + (head * splits + s) * kPdD + 4 * lane);
    O.x += o.x * a; O.y += o.y * a; O.z += o.z * a; O.w += o.w * a;
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  uint2 packed;
  packed.x = pack_bf16(O.x * inv, O.y * inv);
  packed.y = pack_bf16(O.z * inv, O.w * inv);
  *reinterpret_cast<uint2*>(out + head * kPdD + 4 * lane) = packed;
}

}  // namespace prb

// q: bf16 [B, Hq, 128]; kpool / vpool: bf16 [pages, page_size, Hkv, 128]; block_tables: int32
// [B, max_blocks]; ctx_lens: int32 [B]; out: bf16 [B, Hq, 128]. For splits > 1 the caller gives
// o_part fp32 [B, Hq, splits, 128] and ml_part fp32 [B, Hq, splits, 2].
// Shared-prefix form: group_seqs int32 [num_groups, 8] (-1 = unused), group_pages int32 [num_groups] (0 = slot
// unused), page_begin int32 [B]; prefix_splits >= 1 slices of the shared pages; o_part / ml_part then hold
// splits + prefix_splits slots per head. Needs 16-token pages and a GQA group of at most 8.
PRB_API int prb_paged_decode_prefix(const void* q, const void* kpool, const void* vpool, const int* block_tables,
                                    const int* ctx_lens, void* out, float* o_part, float* ml_part, int B, int Hq,
                                    int Hkv, int head_dim, int page_size, int max_blocks, int splits, float scale,
                                    const int* page_begin, const int* group_seqs, const int* group_pages,
                                    int num_groups, int prefix_splits, void* stream_) {
  using namespace prb;
  if (head_dim != kPdD || Hq % Hkv) return -2;
  if (B <= 0) return 0;
  const int G = Hq / Hkv;
  if (page_size != kPmPage || G > 8 || (G & (G - 1)) != 0) return -5;
  if (splits < 1 || prefix_splits < 1 || num_groups < 1 || o_part == nullptr || ml_part == nullptr ||
      page_begin == nullptr || group_seqs == nullptr || group_pages == nullptr)
    return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  PagedParams p;
  p.q = (const __nv_bfloat16*)q; p.kpool = (const __nv_bfloat16*)kpool; p.vpool = (const __nv_bfloat16*)vpool;
  p.block_tables = block_tables; p.ctx_lens = ctx_lens; p.out = (__nv_bfloat16*)out;
  p.o_part = o_part; p.ml_part = ml_part; p.scale = scale;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size; p.max_blocks = max_blocks; p.splits = splits;
  p.page_begin = page_begin; p.group_seqs = group_seqs; p.group_pages = group_pages;
  p.prefix_splits = prefix_splits; p.total_splits = splits + prefix_splits;
  constexpr int smem = kPdWarps * kPmWarpBytes;       // 64 KB: four per-warp page buffers, or two shared 32 KB stages
  static_assert(2 * kPxStageBytes <= smem, "the shared-prefix stages must fit the same allocation");
#define PRB_PX_LAUNCH(GG)                                                                                       \
  {                                                                                                             \
    static prb::DeviceOnce configured;                                                                          \
    if (configured.pending()) {                                                                                 \
      if (cudaFuncSetAttribute(paged_decode_mma_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != \
              cudaSuccess ||                                                                                    \
          cudaFuncSetAttribute(paged_prefix_mma_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != \
              cudaSuccess)                                                                                      \
        return -10;                                                                                             \
      configured.mark();                                                                                        \
    }                                                                                                           \
    paged_prefix_mma_kernel<GG><<<dim3(num_groups, Hkv, prefix_splits), kPdWarps * 32, smem, stream>>>(p);      \
    paged_decode_mma_kernel<GG><<<dim3(B, Hkv, splits), kPdWarps * 32, smem, stream>>>(p);                      \
  }
  switch (G) {
    case 1: PRB_PX_LAUNCH(1) break;
    case 2: PRB_PX_LAUNCH(2) break;
    case 4: PRB_PX_LAUNCH(4) break;
    default: PRB_PX_LAUNCH(8) break;
  }
#undef PRB_PX_LAUNCH
  {
    const long long heads = static_cast<long long>(B) * Hq;
    paged_decode_merge_kernel<<<static_cast<unsigned>((heads + kMergeHeads - 1) / kMergeHeads), 32 * kMergeHeads, 0,
                                stream>>>(o_part, ml_part, (__nv_bfloat16*)out, p.total_splits, splits, Hq, page_begin,
                                          heads);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_paged_decode(const void* q, const void* kpool, const void* vpool, const int* block_tables,
                             const int* ctx_lens, void* out, float* o_part, float* ml_part, int B, int Hq, int Hkv,
                             int head_dim, int page_size, int max_blocks, int splits, float scale, void* stream_) {
  using namespace prb;
  if (head_dim != kPdD || Hq % Hkv) return -2;
  if (B <= 0) return 0;
  if (splits < 1 || (splits > 1 && (o_part == nullptr || ml_part == nullptr))) return -3;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  PagedParams p;
  p.page_begin = nullptr; p.group_seqs = nullptr; p.group_pages = nullptr; p.prefix_splits = 0; p.total_splits = 0;
  p.q = (const __nv_bfloat16*)q; p.kpool = (const __nv_bfloat16*)kpool; p.vpool = (const __nv_bfloat16*)vpool;
  p.block_tables = block_tables; p.ctx_lens = ctx_lens; p.out = (__nv_bfloat16*)out;
  p.o_part = o_part; p.ml_part = ml_part; p.scale = scale;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page_size; p.max_blocks = max_blocks; p.splits = splits;
  dim3 grid(B, Hkv, splits);
  const int G = Hq / Hkv;
  if (page_size == kPmPage && G <= 8 && (G & (G - 1)) == 0) {
    constexpr int smem = kPdWarps * kPmWarpBytes;     // 64 KB (also holds the 17 KB merge scratch)
#define PRB_PM_LAUNCH(GG)                                                                                       \
    {                                                                                                           \
      static prb::DeviceOnce configured;                                                                           \
      if (configured.pending()) {                                                                                        \
        if (cudaFuncSetAttribute(paged_decode_mma_kernel<GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != \
            cudaSuccess)                                                                                        \
          return -10;                                                                                           \
        configured.mark();                                                                                      \
      }                                                                                                         \
      paged_decode_mma_kernel<GG><<<grid, kPdWarps * 32, smem, stream>>>(p);                                    \
    }
    switch (G) {
      case 1: PRB_PM_LAUNCH(1) break;
      case 2: PRB_PM_LAUNCH(2) break;
      case 4: PRB_PM_LAUNCH(4) break;
      default: PRB_PM_LAUNCH(8) break;
    }
#undef PRB_PM_LAUNCH
    if (splits > 1)
      paged_decode_merge_kernel<<<static_cast<unsigned>((static_cast<long long>(B) * Hq + kMergeHeads - 1) / kMergeHeads),
                                  32 * kMergeHeads, 0, stream>>>(o_part, ml_part, (__nv_bfloat16*)out, splits, splits, Hq,
                                                                 nullptr, static_cast<long long>(B) * Hq);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }
  switch (G) {
    case 1: paged_decode_kernel<1><<<grid, kPdWarps * 32, 0, stream>>>(p); break;
    case 2: paged_decode_kernel<2><<<grid, kPdWarps * 32, 0, stream>>>(p); break;
    case 4: paged_decode_kernel<4><<<grid, kPdWarps * 32, 0, stream>>>(p); break;
    case 8: paged_decode_kernel<8><<<grid, kPdWarps * 32, 0, stream>>>(p); break;
    default: return -4;
  }
  if (splits > 1)
    paged_decode_merge_kernel<<<static_cast<unsigned>((static_cast<long long>(B) * Hq + kMergeHeads - 1) / kMergeHeads),
                                32 * kMergeHeads, 0, stream>>>(o_part, ml_part, (__nv_bfloat16*)out, splits, splits, Hq,
                                                               nullptr, static_cast<long long>(B) * Hq);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
