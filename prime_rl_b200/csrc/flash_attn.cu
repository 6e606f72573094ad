// Flash attention forward for sm_100a: varlen (packed documents), causal, optional sliding
// window, GQA, head_dim 128, bf16 in / bf16 out + fp32 log-sum-exp.
//
// One CTA owns 256 query rows of one head inside one document, as two 128-row tiles that
// ping-pong: while one tile's softmax warps work on S, the tensor core runs the other
// tile's MMAs. Per 64-key block and tile:
//     S = Q K^T           tcgen05.mma  M128 x N64 x K128  (Q, K from shared memory, S in TMEM)
//     softmax             4 warps, one thread per row, S read with tcgen05.ld, running max / sum
//                         in registers, P written as bf16 into a 128B-swizzled shared tile,
//                         O (TMEM) rescaled in place when the running max moved
//     O += P V            tcgen05.mma  M128 x N128 x K64   (P from shared memory, V MN-major)
// K and V tiles arrive by TMA (no multicast) through separate 3-stage rings.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer + TMEM owner, 2..5 = softmax of tile 0,
// 6..9 = softmax of tile 1. All waits are bounded and report through the status word.
//
// Replaces flash_attn_varlen_func in the reference (src/prime_rl/trainer/models/layers/attn.py:101-115).
#include "common.cuh"
#include "tma_host.cuh"

namespace prb {

constexpr int kFaD = 128;        // head dim
constexpr int kFaBM = 128;       // rows per tile
constexpr int kFaBN = 64;        // keys per block
constexpr int kFaStages = 3;
constexpr int kFaThreads = 320;

constexpr int kQBytes = kFaBM * kFaD * 2;          // 32 KB per tile (two 16 KB slabs of 64 columns)
constexpr int kKVBytes = kFaBN * kFaD * 2;         // 16 KB per stage (two 8 KB halves)
constexpr int kPBytes = kFaBM * kFaBN * 2;         // 16 KB per tile
constexpr int kFaSmem = 2 * kQBytes + 2 * kFaStages * kKVBytes + 2 * kPBytes + 1024 + 512;

struct FaParams {
  const int* cu_seqlens;  // [num_docs + 1]
  int num_docs;
  int total_q;            // T
  int heads_q, heads_kv;
  __nv_bfloat16* out;     // [T, heads_q, D]
  long long ld_out;       // elements per token
  float* lse;             // [heads_q, T]
  float scale_log2;       // softmax scale * log2(e)
  int window;             // <= 0: none; else a query attends keys with q - k < window
  int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kFaThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + 2 * kQBytes;
  uint8_t* v_s = k_s + kFaStages * kKVBytes;
  uint8_t* p_s = v_s + kFaStages * kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 2 * kPBytes);
  uint64_t* q_full = bars;                      // 1
  uint64_t* k_full = q_full + 1;                // stages
  uint64_t* k_empty = k_full + kFaStages;
  uint64_t* v_full = k_empty + kFaStages;
  uint64_t* v_empty = v_full + kFaStages;
  uint64_t* s_full = v_empty + kFaStages;       // 2
  uint64_t* p_ready = s_full + 2;               // 2
  uint64_t* o_ready = p_ready + 2;              // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_ready + 2);
  int* s_work = reinterpret_cast<int*>(tmem_slot + 1);  // doc_start, doc_len, row0 (in doc)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kv_head = head / (p.heads_q / p.heads_kv);

  // ------------------------------------------------------------ locate this CTA's work
  if (threadIdx.x == 0) {
    int pair = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
    int found = 0;
    // pairs are numbered document by document; walk documents from the last one so that
    // the numbering matches the reversed launch order
    int acc = 0;
    for (int d = 0; d < p.num_docs; ++d) {
      const int s0 = p.cu_seqlens[d], s1 = p.cu_seqlens[d + 1];
      const int len = s1 - s0;
      const int np = (len + 2 * kFaBM - 1) / (2 * kFaBM);
      if (pair < acc + np) {
        s_work[0] = s0;
        s_work[1] = len;
        s_work[2] = (pair - acc) * 2 * kFaBM;
        found = 1;
        break;
      }
      acc += np;
    }
    s_work[3] = found;
  }
  __syncthreads();
  if (!s_work[3]) return;
  const int doc_start = s_work[0];
  const int doc_len = s_work[1];
  const int row0 = s_work[2];

  // rows [q0_t, q1_t) of the document for each tile and the key blocks they need
  int q0[2], q1[2], nblk[2], blk0[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    q0[t] = row0 + t * kFaBM;
    q1[t] = min(q0[t] + kFaBM, doc_len);
    nblk[t] = (q1[t] > q0[t]) ? (q1[t] + kFaBN - 1) / kFaBN : 0;
    blk0[t] = 0;
    if (p.window > 0 && nblk[t] > 0) blk0[t] = max(0, q0[t] - p.window + 1) / kFaBN;
  }
  const int j_begin = min(blk0[0], nblk[1] > 0 ? blk0[1] : blk0[0]);
  const int j_end = max(nblk[0], nblk[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kFaStages; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
      mbar_init(&o_ready[i], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
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
      mbar_expect_tx(q_full, 2 * kQBytes);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int s = 0; s < 2; ++s)
          tma_load_2d(q_s + t * kQBytes + s * (kQBytes / 2), &tmQ, q_full, head * kFaD + s * 64,
                      doc_start + q0[t]);
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0;
      bool ok = true;
      for (int j = j_begin; j < j_end && ok; ++j) {
        const int krow = doc_start + j * kFaBN;
        if (!mbar_wait(&k_empty[ks], kph ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
        mbar_expect_tx(&k_full[ks], kKVBytes);
        tma_load_2d(k_s + ks * kKVBytes, &tmK, &k_full[ks], kv_head * kFaD, krow);
        tma_load_2d(k_s + ks * kKVBytes + kKVBytes / 2, &tmK, &k_full[ks], kv_head * kFaD + 64, krow);
        if (++ks == kFaStages) { ks = 0; kph ^= 1; }
        if (!mbar_wait(&v_empty[vs], vph ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
        mbar_expect_tx(&v_full[vs], kKVBytes);
        tma_load_2d(v_s + vs * kKVBytes, &tmV, &v_full[vs], kv_head * kFaD, krow);
        tma_load_2d(v_s + vs * kKVBytes + kKVBytes / 2, &tmV, &v_full[vs], kv_head * kFaD + 64, krow);
        if (++vs == kFaStages) { vs = 0; vph ^= 1; }
      }
      if (!ok) __nanosleep(200000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, kFaBM, kFaBN, false, false);
      constexpr uint32_t idesc_pv = umma_idesc(1, kFaBM, kFaD, false, true);
      const uint32_t q_addr = smem_u32(q_s), k_addr = smem_u32(k_s), v_addr = smem_u32(v_s), p_addr = smem_u32(p_s);
      bool ok = mbar_wait(q_full, 0, p.status, kTimeoutFullBarrier);
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0;
      uint32_t cnt[2] = {0, 0};  // blocks issued per tile (phase source)

      auto issue_qk = [&](int t, int stage) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t a = umma_smem_desc(q_addr + t * kQBytes + (kk >> 2) * (kQBytes / 2) + (kk & 3) * 32, 0, 1024);
          const uint64_t b = umma_smem_desc(k_addr + stage * kKVBytes + (kk >> 2) * (kKVBytes / 2) + (kk & 3) * 32, 0, 1024);
          umma_f16(tmem_base + t * 256, a, b, idesc_qk, kk != 0);
        }
        umma_commit(&s_full[t]);
      };

      // prologue: S for the first block of both tiles
      if (ok && j_begin < j_end) {
        ok = mbar_wait(&k_full[ks], kph, p.status, kTimeoutFullBarrier);
        if (ok) {
          tc_fence_after();
          for (int t = 0; t < 2; ++t)
            if (j_begin >= blk0[t] && j_begin < nblk[t]) issue_qk(t, ks);
          umma_commit(&k_empty[ks]);
          if (++ks == kFaStages) { ks = 0; kph ^= 1; }
        }
      }
      for (int j = j_begin; j < j_end && ok; ++j) {
        const bool has_next = (j + 1 < j_end);
        bool k_next_ready = false;
        if (!mbar_wait(&v_full[vs], vph, p.status, kTimeoutFullBarrier)) { ok = false; break; }
        for (int t = 0; t < 2 && ok; ++t) {
          const bool active = (j >= blk0[t] && j < nblk[t]);
          if (active) {
            // P_j of this tile is in shared memory and its O has been rescaled
            if (!mbar_wait(&p_ready[t], cnt[t] & 1, p.status, kTimeoutPeerFlag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t a = umma_smem_desc(p_addr + t * kPBytes + kk * 32, 0, 1024);
              const uint64_t b = umma_smem_desc(v_addr + vs * kKVBytes + kk * 2048, 8192, 1024);
              umma_f16(tmem_base + t * 256 + 128, a, b, idesc_pv, (cnt[t] | kk) != 0);
            }
            umma_commit(&o_ready[t]);
            ++cnt[t];
          }
          // S of this tile is free again (its softmax finished block j before arriving on
          // p_ready, or the tile has not started yet): issue the next Q K^T right away
          const bool next_active = has_next && (j + 1 >= blk0[t] && j + 1 < nblk[t]);
          if (next_active) {
            if (!k_next_ready) {
              if (!mbar_wait(&k_full[ks], kph, p.status, kTimeoutFullBarrier)) { ok = false; break; }
              tc_fence_after();
              k_next_ready = true;
            }
            issue_qk(t, ks);
          }
        }
        if (!ok) break;
        umma_commit(&v_empty[vs]);
        if (++vs == kFaStages) { vs = 0; vph ^= 1; }
        if (has_next) {
          if (!k_next_ready) {
            // no tile needs block j+1 (cannot happen for j+1 < j_end, kept for symmetry)
            if (!mbar_wait(&k_full[ks], kph, p.status, kTimeoutFullBarrier)) break;
          }
          umma_commit(&k_empty[ks]);
          if (++ks == kFaStages) { ks = 0; kph ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int t = (warp - 2) >> 2;          // tile
    const int qtr = warp & 3;               // TMEM lane quarter
    const int r = qtr * 32 + lane;          // row in tile
    const int row = q0[t] + r;              // row in document
    const bool row_ok = row < q1[t];
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    const uint32_t s_tm = tmem_base + t * 256 + lane_off;
    const uint32_t o_tm = s_tm + 128;
    uint8_t* p_row = p_s + t * kPBytes + r * 128;
    float m = -INFINITY, l = 0.f;
    uint32_t it = 0;
    bool ok = true;
    for (int j = blk0[t]; j < nblk[t]; ++j, ++it) {
      ok = mbar_wait(&s_full[t], it & 1, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[2][32];
      tmem_ld_32x32(s_tm, sv[0]);
      tmem_ld_32x32(s_tm + 32, sv[1]);
      tmem_ld_wait();
      const int col0 = j * kFaBN;
      const bool need_mask = (col0 + kFaBN - 1 > q0[t]) || (p.window > 0 && q1[t] - 1 - col0 >= p.window);
      // raw scores; masked entries become -inf. The running reference `m` (log2 domain) only
      // moves when the block maximum exceeds it by more than 8: P then stays below 2^8, and
      // most blocks need no rescale of O at all.
      float s[64];
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        float x = __uint_as_float(sv[c >> 5][c & 31]);
        if (need_mask) {
          const int col = col0 + c;
          const bool keep = (col <= row) && (p.window <= 0 || row - col < p.window);
          x = keep ? x : -INFINITY;
        }
        s[c] = x;
        mx = fmaxf(mx, x);
      }
      const float m_blk = mx * p.scale_log2;          // scale > 0, so max commutes with it
      float alpha = 1.f;
      if (m_blk > m + 8.f) {                          // also true on the first unmasked block (m = -inf)
        alpha = ex2(m - m_blk);                       // m = -inf -> 0
        m = m_blk;
      }
      // rows without any valid key so far keep m = -inf: use 0 so that no NaN appears
      const float neg_m = (m == -INFINITY) ? 0.f : -m;
      float sum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = ex2(fmaf(s[c], p.scale_log2, neg_m)), p1 = ex2(fmaf(s[c + 1], p.scale_log2, neg_m));
        sum += p0 + p1;
        pk[c >> 1] = pack_bf16(p0, p1);
      }
      l = l * alpha + sum;
      if (it > 0) {
        // O holds blocks < j: wait for the last PV, then rescale in place
        ok = mbar_wait(&o_ready[t], (it - 1) & 1, p.status, kTimeoutTmemFull);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const bool skip = __all_sync(0xffffffffu, alpha == 1.f);
        if (!skip) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t ov[32];
            tmem_ld_32x32(o_tm + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st_32x32(o_tm + c * 32, ov);
          }
          tmem_st_wait();
        }
      }
      // P row: 8 chunks of 16 bytes, 128B swizzle (chunk ^ (row & 7))
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 val = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        *reinterpret_cast<uint4*>(p_row + ((c ^ (r & 7)) << 4)) = val;
      }
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
    }
    // ---------------------------------------------------------- epilogue: O / l, LSE
    if (ok && nblk[t] > blk0[t]) {
      ok = mbar_wait(&o_ready[t], (it - 1) & 1, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
        __nv_bfloat16* dst = p.out + static_cast<long long>(doc_start + row) * p.ld_out +
                             static_cast<long long>(head) * kFaD;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(o_tm + c * 32, ov);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(ov[8 * i + 0]) * inv_l, __uint_as_float(ov[8 * i + 1]) * inv_l);
              o.y = pack_bf16(__uint_as_float(ov[8 * i + 2]) * inv_l, __uint_as_float(ov[8 * i + 3]) * inv_l);
              o.z = pack_bf16(__uint_as_float(ov[8 * i + 4]) * inv_l, __uint_as_float(ov[8 * i + 5]) * inv_l);
              o.w = pack_bf16(__uint_as_float(ov[8 * i + 6]) * inv_l, __uint_as_float(ov[8 * i + 7]) * inv_l);
              *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = o;
            }
          }
        }
        if (row_ok)
          p.lse[static_cast<long long>(head) * p.total_q + doc_start + row] =
              (m + log2f(l)) * 0.6931471805599453f;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace prb

// q: bf16 [T, heads_q, 128] (token pitch ld_q elements), k / v: bf16 [T, heads_kv, 128] (pitches
// ld_k / ld_v; views into a packed qkv projection are fine), out: bf16 [T, heads_q, 128],
// lse: fp32 [heads_q, T] (natural log). max_pairs bounds the number of 256-row tile pairs:
// sum over documents of ceil(len / 256).
PRB_API int prb_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_seqlens,
                          int num_docs, int total_q, int heads_q, int heads_kv, int head_dim, long long ld_q,
                          long long ld_k, long long ld_v, long long ld_out, float scale, int window, int max_pairs,
                          int* status, void* stream_) {
  using namespace prb;
  if (head_dim != kFaD || heads_q % heads_kv) return -2;
  if (total_q <= 0 || num_docs <= 0) return 0;
  if ((ld_q % 8) || (ld_k % 8) || (ld_v % 8) || (ld_out % 8)) return -4;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_q, (uint64_t)heads_q * kFaD,
                        (uint64_t)ld_q, kFaBM, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_q, (uint64_t)heads_kv * kFaD,
                    (uint64_t)ld_k, kFaBN, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_q, (uint64_t)heads_kv * kFaD,
                    (uint64_t)ld_v, kFaBN, 64, true);
  if (rc) return rc;
  FaParams p;
  p.cu_seqlens = cu_seqlens; p.num_docs = num_docs; p.total_q = total_q;
  p.heads_q = heads_q; p.heads_kv = heads_kv;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ld_out = ld_out; p.lse = lse;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window; p.status = status;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFaSmem) != cudaSuccess)
      return -10;
    configured = true;
  }
  dim3 grid(max_pairs, heads_q);
  flash_fwd_kernel<<<grid, kFaThreads, kFaSmem, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
