// Flash attention backward for sm_100a (varlen, causal, optional sliding window, GQA,
// head_dim 128). One CTA owns 128 keys of one KV head inside one document and walks over the
// query heads of its group and the 128-row query blocks that can see those keys. Per query
// block and 64-key half h (all products on tcgen05, accumulators in TMEM):
//
//   S_h   = Q K_h^T                 M128 x N64  x K128
//   dP_h  = dO V_h^T                M128 x N64  x K128
//   P = exp2(S * c - lse), dS = P * (dP - delta) * scale          (8 softmax warps, registers)
//   dV_h^T += dO^T P                M128(d) x N64(key) x K128(row)   A, B MN-major
//   dK_h^T += Q^T dS                M128(d) x N64(key) x K128(row)
//   dQ    (+)= dS K_h               M128 x N128 x K64                 B MN-major
//
// dK^T / dV^T stay in TMEM for the whole CTA and are written once (no atomics, GQA heads are
// reduced in place); dQ is flushed per query block with vector reductions into an fp32
// accumulator. TMEM: S 64 + dP 64 + dQ 128 + dV^T 2x64 + dK^T 2x64 = 512 columns.
// Shared memory: K 32 KB, V 32 KB, (Q, dO) 2 stages x 64 KB, P 16 KB, dS 16 KB.
//
// Warps: 0 = TMA producer, 1 = MMA issuer + TMEM owner, 2..9 = softmax / epilogue (two warps
// per TMEM lane quarter; the pair splits the columns). All waits are bounded.
#include "common.cuh"
#include "tma_host.cuh"

namespace prb {

constexpr int kBwD = 128;
constexpr int kBwBM = 128;   // query rows per block
constexpr int kBwBN = 128;   // keys per CTA (two halves of 64)
constexpr int kBwThreads = 320;

constexpr int kBwKV = kBwBN * kBwD * 2;        // 32 KB
constexpr int kBwQ = kBwBM * kBwD * 2;         // 32 KB
constexpr int kBwP = kBwBM * 64 * 2;           // 16 KB
constexpr int kBwSmem = 2 * kBwKV + 4 * kBwQ + 2 * kBwP + 1024 + 256;

// TMEM column map
constexpr int kTmS = 0, kTmDP = 64, kTmDQ = 128, kTmDV = 256, kTmDK = 384;

struct FaBwdParams {
  const int* cu_seqlens;
  int num_docs, total_q, heads_q, heads_kv;
  const float* lse;        // [heads_q, T] natural log
  const float* delta;      // [heads_q, T] rowsum(dO * O)
  float* dq_acc;           // [T, heads_q, D] fp32, zero-initialised
  __nv_bfloat16* dk;       // [T, heads_kv, D]
  __nv_bfloat16* dv;
  long long ld_dk, ld_dv;  // elements per token
  float scale, scale_log2;
  int window;
  int* status;
};

__device__ __forceinline__ float bw_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));  // pure: let the compiler batch them
  return y;
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

__global__ void __launch_bounds__(kBwThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const FaBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = smem;                    // [half][d-slab] 8 KB each
  uint8_t* v_s = k_s + kBwKV;
  uint8_t* q_s = v_s + kBwKV;             // [stage] 32 KB: two d-slabs of [128 x 64]
  uint8_t* do_s = q_s + 2 * kBwQ;
  uint8_t* p_s = do_s + 2 * kBwQ;
  uint8_t* ds_s = p_s + kBwP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_s + kBwP);
  uint64_t* kv_full = bars;
  uint64_t* q_full = kv_full + 1;         // [2]
  uint64_t* q_empty = q_full + 2;         // [2]
  uint64_t* sdp_full = q_empty + 2;
  uint64_t* sdp_free = sdp_full + 1;
  uint64_t* pds_ready = sdp_free + 1;
  uint64_t* pds_free = pds_ready + 1;
  uint64_t* dq_full = pds_free + 1;
  uint64_t* dq_free = dq_full + 1;
  uint64_t* final_done = dq_free + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(final_done + 1);
  int* s_work = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv_head = blockIdx.y;
  const int group = p.heads_q / p.heads_kv;

  // ------------------------------------------------------------ locate the key block
  if (threadIdx.x == 0) {
    int blk = blockIdx.x, acc = 0, found = 0;
    for (int d = 0; d < p.num_docs; ++d) {
      const int s0 = p.cu_seqlens[d], len = p.cu_seqlens[d + 1] - s0;
      const int nb = (len + kBwBN - 1) / kBwBN;
      if (blk < acc + nb) {
        s_work[0] = s0; s_work[1] = len; s_work[2] = (blk - acc) * kBwBN; found = 1;
        break;
      }
      acc += nb;
    }
    s_work[3] = found;
  }
  __syncthreads();
  if (!s_work[3]) return;
  const int doc_start = s_work[0], doc_len = s_work[1], kv0 = s_work[2];
  const int i_begin = kv0 / kBwBM;
  int i_end = (doc_len + kBwBM - 1) / kBwBM;
  if (p.window > 0) i_end = min(i_end, (kv0 + kBwBN - 1 + p.window - 1) / kBwBM + 1);
  const int iters_per_head = i_end - i_begin;
  const int num_iters = iters_per_head * group;   // >= 1: the diagonal block always exists

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_free, 8);
    mbar_init(pds_ready, 8);
    mbar_init(pds_free, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 8);
    mbar_init(final_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * kBwKV);
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          tma_load_2d(k_s + h * 16384 + s * 8192, &tmK, kv_full, kv_head * kBwD + s * 64, doc_start + kv0 + h * 64);
          tma_load_2d(v_s + h * 16384 + s * 8192, &tmV, kv_full, kv_head * kBwD + s * 64, doc_start + kv0 + h * 64);
        }
      bool ok = true;
      for (int n = 0; n < num_iters && ok; ++n) {
        const int st = n & 1;
        const uint32_t ph = (n >> 1) & 1;
        const int g = n / iters_per_head;
        const int i = i_begin + (n - g * iters_per_head);
        const int head = kv_head * group + g;
        if (!mbar_wait(&q_empty[st], ph ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
        mbar_expect_tx(&q_full[st], 2 * kBwQ);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          tma_load_2d(q_s + st * kBwQ + s * 16384, &tmQ, &q_full[st], head * kBwD + s * 64, doc_start + i * kBwBM);
          tma_load_2d(do_s + st * kBwQ + s * 16384, &tmDO, &q_full[st], head * kBwD + s * 64, doc_start + i * kBwBM);
        }
      }
      if (!ok) __nanosleep(200000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t id_s = umma_idesc(1, 128, 64, false, false);    // S, dP
      constexpr uint32_t id_g = umma_idesc(1, 128, 64, true, true);      // dV^T, dK^T
      constexpr uint32_t id_q = umma_idesc(1, 128, 128, false, true);    // dQ
      const uint32_t k_a = smem_u32(k_s), v_a = smem_u32(v_s), q_a = smem_u32(q_s), do_a = smem_u32(do_s);
      const uint32_t p_a = smem_u32(p_s), ds_a = smem_u32(ds_s);

      auto issue_s_dp = [&](int st, int h) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t ao = st * kBwQ + (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t bo = h * 16384 + (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16(tmem_base + kTmS, umma_smem_desc(q_a + ao, 0, 1024), umma_smem_desc(k_a + bo, 0, 1024), id_s,
                   kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t ao = st * kBwQ + (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t bo = h * 16384 + (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_f16(tmem_base + kTmDP, umma_smem_desc(do_a + ao, 0, 1024), umma_smem_desc(v_a + bo, 0, 1024), id_s,
                   kk != 0);
        }
        umma_commit(sdp_full);
      };

      bool ok = mbar_wait(kv_full, 0, p.status, kTimeoutFullBarrier);
      if (ok) ok = mbar_wait(&q_full[0], 0, p.status, kTimeoutFullBarrier);
      if (ok) {
        tc_fence_after();
        issue_s_dp(0, 0);
      }
      uint32_t u = 0;
      for (int n = 0; n < num_iters && ok; ++n) {
        const int st = n & 1;
        for (int h = 0; h < 2 && ok; ++h, ++u) {
          // the softmax warps hold S_u / dP_u in registers: issue the next half's S / dP
          if (!mbar_wait(sdp_free, u & 1, p.status, kTimeoutTmemEmpty)) { ok = false; break; }
          tc_fence_after();
          if (h == 0) {
            issue_s_dp(st, 1);
          } else if (n + 1 < num_iters) {
            const int nst = (n + 1) & 1;
            if (!mbar_wait(&q_full[nst], ((n + 1) >> 1) & 1, p.status, kTimeoutFullBarrier)) { ok = false; break; }
            tc_fence_after();
            issue_s_dp(nst, 0);
          }
          if (!mbar_wait(pds_ready, u & 1, p.status, kTimeoutPeerFlag)) { ok = false; break; }
          if (h == 0 && n > 0) {
            if (!mbar_wait(dq_free, (n - 1) & 1, p.status, kTimeoutTmemEmpty)) { ok = false; break; }
          }
          tc_fence_after();
          // dV_h^T += dO^T P ; dK_h^T += Q^T dS   (reduction over the 128 query rows)
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t b = umma_smem_desc(p_a + kk * 2048, 8192, 1024);
            const uint64_t a = umma_smem_desc(do_a + st * kBwQ + kk * 2048, 16384, 1024);
            umma_f16(tmem_base + kTmDV + h * 64, a, b, id_g, (n | kk) != 0);
          }
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t b = umma_smem_desc(ds_a + kk * 2048, 8192, 1024);
            const uint64_t a = umma_smem_desc(q_a + st * kBwQ + kk * 2048, 16384, 1024);
            umma_f16(tmem_base + kTmDK + h * 64, a, b, id_g, (n | kk) != 0);
          }
          // dQ (+)= dS K_h   (reduction over the 64 keys of this half)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t a = umma_smem_desc(ds_a + kk * 32, 0, 1024);
            const uint64_t b = umma_smem_desc(k_a + h * 16384 + kk * 2048, 8192, 1024);
            umma_f16(tmem_base + kTmDQ, a, b, id_q, (h | kk) != 0);
          }
          umma_commit(pds_free);
          if (h == 1) {
            umma_commit(dq_full);
            umma_commit(&q_empty[st]);
          }
        }
      }
      if (ok) umma_commit(final_done);
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue warps
    const int w = (warp - 2) >> 2;          // column half handled by this warp (0 or 1)
    const int qtr = warp & 3;
    const int r = qtr * 32 + lane;          // row of the query block / TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    uint8_t* p_row = p_s + r * 128;
    uint8_t* ds_row = ds_s + r * 128;
    bool ok = true;
    uint32_t u = 0;
    for (int n = 0; n < num_iters && ok; ++n) {
      const int g = n / iters_per_head;
      const int i = i_begin + (n - g * iters_per_head);
      const int head = kv_head * group + g;
      const int row = i * kBwBM + r;                      // row in document
      const bool row_ok = row < doc_len;
      const long long stat_idx = static_cast<long long>(head) * p.total_q + doc_start + row;
      const float lse2 = row_ok ? p.lse[stat_idx] * 1.4426950408889634f : 0.f;
      const float delta = row_ok ? p.delta[stat_idx] : 0.f;
      for (int h = 0; h < 2 && ok; ++h, ++u) {
        ok = mbar_wait(sdp_full, u & 1, p.status, kTimeoutTmemFull);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t sv[32], dpv[32];
        tmem_ld_32x32(tmem_base + lane_off + kTmS + 32 * w, sv);
        tmem_ld_32x32(tmem_base + lane_off + kTmDP + 32 * w, dpv);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sdp_free);
        const int col0 = kv0 + h * 64 + 32 * w;           // key index in document
        uint32_t pp[16], dd[16];
        // keep column c of this slab iff lim_lo < c <= lim_hi; branch-free so that the 32
        // exponentials of a row are issued back to back
        const int lim_hi = row_ok ? row - col0 : -1;
        const int lim_lo = (p.window > 0) ? lim_hi - p.window : -1;
        const float neg_lse2 = -lse2;
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float ex = bw_ex2(fmaf(__uint_as_float(sv[c + e]), p.scale_log2, neg_lse2));
            const float pr = ((c + e <= lim_hi) & (c + e > lim_lo)) ? ex : 0.f;
            pv[e] = pr;
            dv[e] = pr * (__uint_as_float(dpv[c + e]) - delta) * p.scale;
          }
          pp[c >> 1] = pack_bf16(pv[0], pv[1]);
          dd[c >> 1] = pack_bf16(dv[0], dv[1]);
        }
        if (u > 0) {
          ok = mbar_wait(pds_free, (u - 1) & 1, p.status, kTimeoutTmemFull);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int chunk = 4 * w + c;
          const int off = (chunk ^ (r & 7)) << 4;
          *reinterpret_cast<uint4*>(p_row + off) = make_uint4(pp[4 * c], pp[4 * c + 1], pp[4 * c + 2], pp[4 * c + 3]);
          *reinterpret_cast<uint4*>(ds_row + off) = make_uint4(dd[4 * c], dd[4 * c + 1], dd[4 * c + 2], dd[4 * c + 3]);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(pds_ready);
      }
      if (!ok) break;
      // ---- dQ of this query block: columns [64 w, 64 w + 64) of this row
      ok = mbar_wait(dq_full, n & 1, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float* dq_dst = p.dq_acc + (static_cast<long long>(doc_start + row) * p.heads_q + head) * kBwD + 64 * w;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t qv[32];
        tmem_ld_32x32(tmem_base + lane_off + kTmDQ + 64 * w + 32 * c, qv);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            red_add_v4(dq_dst + 32 * c + e, __uint_as_float(qv[e]), __uint_as_float(qv[e + 1]),
                       __uint_as_float(qv[e + 2]), __uint_as_float(qv[e + 3]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_free);
    }
    // ---------------------------------------------------------- epilogue: dK^T, dV^T -> dK, dV
    if (ok) {
      ok = mbar_wait(final_done, 0, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      // lane = feature d (quarter qtr), warp pair member w = key half
      const int d = r;
      const int h = w;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* base = which ? p.dk : p.dv;
        const long long ld = which ? p.ld_dk : p.ld_dv;
        const int tm = (which ? kTmDK : kTmDV) + h * 64;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t gv[32];
          tmem_ld_32x32(tmem_base + lane_off + tm + 32 * c, gv);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int key = kv0 + h * 64 + 32 * c + e;
            if (key < doc_len)
              base[static_cast<long long>(doc_start + key) * ld + static_cast<long long>(kv_head) * kBwD + d] =
                  __float2bfloat16(__uint_as_float(gv[e]));
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d]; one warp per (t, h).
__global__ void __launch_bounds__(256)
flash_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                       float* __restrict__ delta, long long T, int heads, long long ld_o, long long ld_do) {
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (item >= T * heads) return;
  const long long t = item / heads;
  const int h = static_cast<int>(item - t * heads);
  const uint2 a = *reinterpret_cast<const uint2*>(o + t * ld_o + static_cast<long long>(h) * kBwD + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(d_o + t * ld_do + static_cast<long long>(h) * kBwD + lane * 4);
  const float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y);
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  s = warp_sum(s);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

__global__ void __launch_bounds__(256)
flash_bwd_convert_dq_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long n) {
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(acc + i);
    uint2 o;
    o.x = pack_bf16(v.x, v.y);
    o.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(dq + i) = o;
  }
}

}  // namespace prb

// q, k, v as in prb_flash_fwd; o / d_o: bf16 [T, heads_q, 128] (pitches ld_o / ld_do); lse: fp32
// [heads_q, T]. Scratch supplied by the caller: delta fp32 [heads_q, T], dq_acc fp32
// [T, heads_q, 128] (zeroed here). Outputs dq (contiguous), dk, dv (pitches ld_dk / ld_dv).
PRB_API int prb_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                          const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                          const int* cu_seqlens, int num_docs, int total_q, int heads_q, int heads_kv, int head_dim,
                          long long ld_q, long long ld_k, long long ld_v, long long ld_o, long long ld_do,
                          long long ld_dk, long long ld_dv, float scale, int window, int max_blocks, int* status,
                          void* stream_) {
  using namespace prb;
  if (head_dim != kBwD || heads_q % heads_kv) return -2;
  if (total_q <= 0 || num_docs <= 0) return 0;
  if ((ld_q % 8) || (ld_k % 8) || (ld_v % 8) || (ld_do % 8)) return -4;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  CUtensorMap tmQ, tmK, tmV, tmDO;
  int rc = make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_q, (uint64_t)heads_q * kBwD,
                        (uint64_t)ld_q, kBwBM, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmDO, d_o, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_q, (uint64_t)heads_q * kBwD,
                    (uint64_t)ld_do, kBwBM, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_q, (uint64_t)heads_kv * kBwD,
                    (uint64_t)ld_k, 64, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_q, (uint64_t)heads_kv * kBwD,
                    (uint64_t)ld_v, 64, 64, true);
  if (rc) return rc;
  const long long items = static_cast<long long>(total_q) * heads_q;
  flash_bwd_delta_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, stream>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, total_q, heads_q, ld_o, ld_do);
  cudaMemsetAsync(dq_acc, 0, sizeof(float) * items * kBwD, stream);
  FaBwdParams p;
  p.cu_seqlens = cu_seqlens; p.num_docs = num_docs; p.total_q = total_q; p.heads_q = heads_q; p.heads_kv = heads_kv;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk); p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.ld_dk = ld_dk; p.ld_dv = ld_dv;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.window = window; p.status = status;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwSmem) != cudaSuccess)
      return -10;
    configured = true;
  }
  dim3 grid(max_blocks, heads_kv);
  flash_bwd_kernel<<<grid, kBwThreads, kBwSmem, stream>>>(tmQ, tmK, tmV, tmDO, p);
  const long long n = items * kBwD;
  flash_bwd_convert_dq_kernel<<<148 * 8, 256, 0, stream>>>(dq_acc, (__nv_bfloat16*)dq, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
