// Flash attention backward for sm_100a (varlen, causal, optional sliding window, GQA,
// head_dim 128), as two atomics-free kernels over 128 x 128 (query x key) blocks. All products
// run on tcgen05 with N = 128 (an N = 64 product runs at half the tensor rate), accumulators
// live in TMEM, operands arrive by TMA (no multicast).
//
//   flash_bwd_dkdv_kernel   one CTA = 128 keys of one KV head in one document; walks over the
//                           query heads of the group and the query blocks that see those keys
//       S  = Q K^T, dP = dO V^T                                (front MMA thread)
//       P  = exp2(S c - lse), dS = P (dP - delta) scale        (8 softmax warps, registers)
//       dV += P^T dO, dK += dS^T Q                             (back MMA thread; TMEM, written once)
//   flash_bwd_dq_kernel     one CTA = 128 query rows of one head; walks over its key blocks
//       S, dP, P, dS as above (S double buffered), dQ += dS K  (TMEM, written once as bf16)
//
// Recomputing S / dP in both kernels costs two extra products per block but removes the fp32
// dQ reductions through L2, which were the bottleneck of a single-kernel version.
// TMEM: dkdv  S 0 | dP 128 | dV 256 | dK 384;   dq  S0 0 | S1 128 | dP 256 | dQ 384.
// Shared memory (7 tiles of 32 KB): dkdv  K V Q0 Q1 dO P dS;   dq  Q dO K0 K1 K2 V dS.
//
// Warps: 0 = TMA producer, 1 = front MMA issuer + TMEM owner, 2 = back MMA issuer,
// 3..10 = softmax (two warps per TMEM lane quarter; the pair splits the 128 columns).
// All waits are bounded and report through the status word.
//
// Takes the place of the flash-attn backward used by the reference
// (src/prime_rl/trainer/models/layers/attn.py:101-115).
#include "common.cuh"
#include "tma_host.cuh"

namespace prb {

constexpr int kBwD = 128;
constexpr int kBwB = 128;        // block edge (query rows and keys)
constexpr int kBwThreads = 352;
constexpr int kBwTile = kBwB * kBwD * 2;       // 32 KB: two 16 KB slabs of [128 rows][64 columns]
constexpr int kBwSmem = 7 * kBwTile + 1024 + 512;

struct FaBwdParams {
  const int* cu_seqlens;
  int num_docs, total_q, heads_q, heads_kv;
  int q_off, q_rows;       // q / dO / lse / delta / dq hold the global rows [q_off, q_off + q_rows) only
  int k_off, k_rows;       // k / v / dk / dv hold the global rows [k_off, k_off + k_rows) only (ring step); lse is the
                           // log-sum-exp over ALL keys, so the products over this key range are the exact partial gradients
  const float* lse;        // [heads_q, T] natural log
  const float* delta;      // [heads_q, T] rowsum(dO * O)
  __nv_bfloat16* dq;       // [T, heads_q, D] contiguous
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

// ---- softmax-warp helpers. A thread owns row r of the block (TMEM lane) and the 64 columns
// [64 w, 64 w + 64); a tile in shared memory is two slabs of [128 rows][64 columns] with the
// 128-byte swizzle, so the thread's 64 bf16 are exactly one swizzled row of slab w.

// P = exp2(S c - lse2) for the thread's 64 columns; column c is kept iff lim_lo < c <= lim_hi.
// Most blocks lie below the diagonal and inside the window: the warp then skips the compares.
__device__ __forceinline__ void bw_load_p(uint32_t s_taddr, float (&pf)[64], int lim_hi, int lim_lo, float scale_log2,
                                          float neg_lse2) {
  uint32_t sv[2][32];
  tmem_ld_32x32(s_taddr, sv[0]);
  tmem_ld_32x32(s_taddr + 32, sv[1]);
  const bool need_mask = __any_sync(0xffffffffu, (lim_hi < 63) | (lim_lo >= 0));
  tmem_ld_wait();
  if (need_mask) {
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      const float ex = bw_ex2(fmaf(__uint_as_float(sv[c >> 5][c & 31]), scale_log2, neg_lse2));
      pf[c] = ((c <= lim_hi) & (c > lim_lo)) ? ex : 0.f;
    }
  } else {
#pragma unroll
    for (int c = 0; c < 64; ++c) pf[c] = bw_ex2(fmaf(__uint_as_float(sv[c >> 5][c & 31]), scale_log2, neg_lse2));
  }
}

// dS = P (dP - delta), in place. The softmax scale is applied once, when dK / dQ leave TMEM.
__device__ __forceinline__ void bw_load_ds(uint32_t dp_taddr, float (&pf)[64], float neg_delta) {
  uint32_t dv[2][32];
  tmem_ld_32x32(dp_taddr, dv[0]);
  tmem_ld_32x32(dp_taddr + 32, dv[1]);
  tmem_ld_wait();
#pragma unroll
  for (int c = 0; c < 64; ++c) pf[c] *= __uint_as_float(dv[c >> 5][c & 31]) + neg_delta;
}

__device__ __forceinline__ void bw_store_row(uint8_t* row_ptr, int r, const float (&pf)[64]) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 val;
    val.x = pack_bf16(pf[8 * c + 0], pf[8 * c + 1]);
    val.y = pack_bf16(pf[8 * c + 2], pf[8 * c + 3]);
    val.z = pack_bf16(pf[8 * c + 4], pf[8 * c + 5]);
    val.w = pack_bf16(pf[8 * c + 6], pf[8 * c + 7]);
    *reinterpret_cast<uint4*>(row_ptr + ((c ^ (r & 7)) << 4)) = val;
  }
}

// One accumulating product of a 128 x 128 x 128 block: 8 k-steps.
//   kmajor operands: [128][64-column slabs], k-step = 32 bytes inside a slab, slab = 16 KB
//   mn-major operands: k-step = 16 rows = 2048 bytes, the two 64-wide atoms are 16 KB apart
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void bw_mma_block(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, bool accumulate) {
  constexpr uint32_t idesc = umma_idesc(1, 128, 128, A_MN, B_MN);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint64_t a = A_MN ? umma_smem_desc(a_addr + kk * 2048, 16384, 1024)
                            : umma_smem_desc(a_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 0, 1024);
    const uint64_t b = B_MN ? umma_smem_desc(b_addr + kk * 2048, 16384, 1024)
                            : umma_smem_desc(b_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 0, 1024);
    umma_f16(d_tmem, a, b, idesc, (accumulate || kk != 0) ? 1u : 0u);
  }
}

__device__ __forceinline__ void bw_load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int col, int row) {
  tma_load_2d(dst, tm, bar, col, row);
  tma_load_2d(dst + kBwTile / 2, tm, bar, col + 64, row);
}

// ============================================================================ dK, dV
__global__ void __launch_bounds__(kBwThreads, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                      const FaBwdParams p) {
  constexpr int kTmS = 0, kTmDP = 128, kTmDV = 256, kTmDK = 384;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = smem;
  uint8_t* v_s = k_s + kBwTile;
  uint8_t* q_s = v_s + kBwTile;            // 2 stages
  uint8_t* do_s = q_s + 2 * kBwTile;       // 1 stage
  uint8_t* p_s = do_s + kBwTile;
  uint8_t* ds_s = p_s + kBwTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_s + kBwTile);
  uint64_t* kv_full = bars;
  uint64_t* q_full = kv_full + 1;          // [2]
  uint64_t* q_empty = q_full + 2;          // [2]
  uint64_t* do_full = q_empty + 2;
  uint64_t* do_empty = do_full + 1;        // count 2: dP (front) and dV (back) both read dO
  uint64_t* s_full = do_empty + 1;
  uint64_t* s_free = s_full + 1;           // count 8
  uint64_t* dp_full = s_free + 1;
  uint64_t* dp_free = dp_full + 1;         // count 8
  uint64_t* p_ready = dp_free + 1;         // count 8
  uint64_t* p_free = p_ready + 1;
  uint64_t* ds_ready = p_free + 1;         // count 8
  uint64_t* ds_free = ds_ready + 1;
  uint64_t* final_done = ds_free + 1;
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
      const int nb = (len + kBwB - 1) / kBwB;
      if (blk < acc + nb) {
        s_work[0] = s0; s_work[1] = len; s_work[2] = (blk - acc) * kBwB; found = 1;
        break;
      }
      acc += nb;
    }
    s_work[3] = found;
  }
  __syncthreads();
  if (!s_work[3]) return;
  const int doc_start = s_work[0], doc_len = s_work[1], kv0 = s_work[2];
  // keys held by this call, as columns of the document: [kcol_lo, kcol_hi)
  const int kcol_lo = p.k_off - doc_start, kcol_hi = kcol_lo + p.k_rows;
  if (kv0 + kBwB <= kcol_lo || kv0 >= kcol_hi) return;           // none of this block's keys is held: nothing to write
  int i_begin = kv0 / kBwB;
  int i_end = (doc_len + kBwB - 1) / kBwB;
  if (p.window > 0) i_end = min(i_end, (kv0 + kBwB - 1 + p.window - 1) / kBwB + 1);
  // context parallelism: only the query blocks that intersect the held row slice
  if (p.q_off > doc_start) i_begin = max(i_begin, (p.q_off - doc_start) / kBwB);
  i_end = min(i_end, (p.q_off + p.q_rows - doc_start + kBwB - 1) / kBwB);
  const int iters_per_head = i_end - i_begin;
  const int num_iters = iters_per_head * group;
  if (iters_per_head <= 0) {
    // no query of this rank sees these keys: their gradient contribution is zero
    for (int idx = threadIdx.x; idx < kBwB * (kBwD / 8); idx += blockDim.x) {
      const int key = kv0 + idx / (kBwD / 8), c = (idx % (kBwD / 8)) * 8;
      if (key < doc_len && key >= kcol_lo && key < kcol_hi) {
        const long long tok = doc_start + key - p.k_off;
        *reinterpret_cast<uint4*>(p.dk + tok * p.ld_dk + static_cast<long long>(kv_head) * kBwD + c) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(p.dv + tok * p.ld_dv + static_cast<long long>(kv_head) * kBwD + c) = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    mbar_init(do_full, 1);
    mbar_init(do_empty, 2);
    mbar_init(s_full, 1);
    mbar_init(s_free, 8);
    mbar_init(dp_full, 1);
    mbar_init(dp_free, 8);
    mbar_init(p_ready, 8);
    mbar_init(p_free, 1);
    mbar_init(ds_ready, 8);
    mbar_init(ds_free, 1);
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
      mbar_expect_tx(kv_full, 2 * kBwTile);
      bw_load_tile(k_s, &tmK, kv_full, kv_head * kBwD, doc_start + kv0 - p.k_off);   // rows outside read as zero
      bw_load_tile(v_s, &tmV, kv_full, kv_head * kBwD, doc_start + kv0 - p.k_off);
      bool ok = true;
      for (int n = 0; n < num_iters && ok; ++n) {
        const int st = n & 1;
        const int g = n / iters_per_head;
        const int i = i_begin + (n - g * iters_per_head);
        const int head = kv_head * group + g;
        if (!mbar_wait(&q_empty[st], ((n >> 1) & 1) ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
        mbar_expect_tx(&q_full[st], kBwTile);
        bw_load_tile(q_s + st * kBwTile, &tmQ, &q_full[st], head * kBwD, doc_start + i * kBwB - p.q_off);
        if (!mbar_wait(do_empty, (n & 1) ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
        mbar_expect_tx(do_full, kBwTile);
        bw_load_tile(do_s, &tmDO, do_full, head * kBwD, doc_start + i * kBwB - p.q_off);
      }
      if (!ok) __nanosleep(200000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ front MMA issuer: S, dP
    if (lane == 0) {
      const uint32_t k_a = smem_u32(k_s), v_a = smem_u32(v_s), q_a = smem_u32(q_s), do_a = smem_u32(do_s);
      bool ok = mbar_wait(kv_full, 0, p.status, kTimeoutFullBarrier);
      for (int n = 0; n < num_iters && ok; ++n) {
        const int st = n & 1;
        if (!mbar_wait(&q_full[st], (n >> 1) & 1, p.status, kTimeoutFullBarrier)) break;
        // S is free again once the softmax warps hold block n - 1 in registers
        if (n > 0 && !mbar_wait(s_free, (n - 1) & 1, p.status, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        bw_mma_block<false, false>(tmem_base + kTmS, q_a + st * kBwTile, k_a, false);
        umma_commit(s_full);
        if (!mbar_wait(do_full, n & 1, p.status, kTimeoutFullBarrier)) break;
        if (n > 0 && !mbar_wait(dp_free, (n - 1) & 1, p.status, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        bw_mma_block<false, false>(tmem_base + kTmDP, do_a, v_a, false);
        umma_commit(dp_full);
        umma_commit(do_empty);
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ back MMA issuer: dV, dK
    if (lane == 0) {
      const uint32_t q_a = smem_u32(q_s), do_a = smem_u32(do_s), p_a = smem_u32(p_s), ds_a = smem_u32(ds_s);
      bool ok = true;
      for (int n = 0; n < num_iters && ok; ++n) {
        const int st = n & 1;
        if (!mbar_wait(do_full, n & 1, p.status, kTimeoutFullBarrier)) { ok = false; break; }
        if (!mbar_wait(p_ready, n & 1, p.status, kTimeoutPeerFlag)) { ok = false; break; }
        tc_fence_after();
        // dV[key][d] += sum_row P[row][key] dO[row][d]: both operands are read "transposed" (MN-major)
        bw_mma_block<true, true>(tmem_base + kTmDV, p_a, do_a, n > 0);
        umma_commit(p_free);
        umma_commit(do_empty);
        if (!mbar_wait(ds_ready, n & 1, p.status, kTimeoutPeerFlag)) { ok = false; break; }
        tc_fence_after();
        bw_mma_block<true, true>(tmem_base + kTmDK, ds_a, q_a + st * kBwTile, n > 0);
        umma_commit(ds_free);
        umma_commit(&q_empty[st]);
      }
      if (ok) umma_commit(final_done);
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue warps
    const int w = (warp - 3) >> 2;          // column half handled by this warp (0 or 1)
    const int qtr = warp & 3;
    const int r = qtr * 32 + lane;          // row of the query block / TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    uint8_t* p_row = p_s + w * (kBwTile / 2) + r * 128;
    uint8_t* ds_row = ds_s + w * (kBwTile / 2) + r * 128;
    const int col0 = kv0 + 64 * w;          // first key (in document) of this thread's columns
    bool ok = true;
    for (int n = 0; n < num_iters && ok; ++n) {
      const int g = n / iters_per_head;
      const int i = i_begin + (n - g * iters_per_head);
      const int head = kv_head * group + g;
      const int row = i * kBwB + r;                       // row in document
      const int grow = doc_start + row - p.q_off;         // row inside the held slice
      const bool row_ok = row < doc_len && grow >= 0 && grow < p.q_rows;
      const long long stat_idx = static_cast<long long>(head) * p.q_rows + grow;
      const float neg_lse2 = row_ok ? -p.lse[stat_idx] * 1.4426950408889634f : 0.f;
      const float neg_delta = row_ok ? -p.delta[stat_idx] : 0.f;
      const int causal_hi = row_ok ? row - col0 : -1;
      const int lim_hi = min(causal_hi, kcol_hi - 1 - col0);
      const int lim_lo = max((p.window > 0) ? causal_hi - p.window : -1, kcol_lo - 1 - col0);

      ok = mbar_wait_poll(s_full, n & 1, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float pf[64];
      bw_load_p(tmem_base + lane_off + kTmS + 64 * w, pf, lim_hi, lim_lo, p.scale_log2, neg_lse2);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      if (n > 0) {
        // P and dS of block n - 1 are still being read by dV / dK. Both products come from one
        // issuing thread and complete in order, so the later one (dK -> ds_free) covers both
        // buffers; by now it is almost always done, and the dS store below needs no wait of its own
        ok = mbar_wait_poll(ds_free, (n - 1) & 1, p.status, kTimeoutTmemFull);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      bw_store_row(p_row, r, pf);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);

      ok = mbar_wait_poll(dp_full, n & 1, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      bw_load_ds(tmem_base + lane_off + kTmDP + 64 * w, pf, neg_delta);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dp_free);
      bw_store_row(ds_row, r, pf);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    // ---------------------------------------------------------- epilogue: dV, dK (lane = key)
    if (ok) {
      ok = mbar_wait(final_done, 0, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const int key = kv0 + r;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = (which ? p.dk : p.dv) +
                             static_cast<long long>(doc_start + key - p.k_off) * (which ? p.ld_dk : p.ld_dv) +
                             static_cast<long long>(kv_head) * kBwD + 64 * w;
        const uint32_t tm = tmem_base + lane_off + (which ? kTmDK : kTmDV) + 64 * w;
        const float mul = which ? p.scale : 1.f;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t gv[32];
          tmem_ld_32x32(tm + 32 * c, gv);
          tmem_ld_wait();
          if (key < doc_len && key >= kcol_lo && key < kcol_hi) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(gv[8 * e + 0]) * mul, __uint_as_float(gv[8 * e + 1]) * mul);
              o.y = pack_bf16(__uint_as_float(gv[8 * e + 2]) * mul, __uint_as_float(gv[8 * e + 3]) * mul);
              o.z = pack_bf16(__uint_as_float(gv[8 * e + 4]) * mul, __uint_as_float(gv[8 * e + 5]) * mul);
              o.w = pack_bf16(__uint_as_float(gv[8 * e + 6]) * mul, __uint_as_float(gv[8 * e + 7]) * mul);
              *reinterpret_cast<uint4*>(dst + 32 * c + 8 * e) = o;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ============================================================================ dQ
__global__ void __launch_bounds__(kBwThreads, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const FaBwdParams p) {
  constexpr int kTmS = 0, kTmDP = 256, kTmDQ = 384;   // S buffers at 0 and 128
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* do_s = q_s + kBwTile;
  uint8_t* k_s = do_s + kBwTile;           // 3 stages: K of block n is held until dQ of block n is done
  uint8_t* v_s = k_s + 3 * kBwTile;        // 1 stage: V is released right after dP
  uint8_t* ds_s = v_s + kBwTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_s + kBwTile);
  uint64_t* qdo_full = bars;
  uint64_t* k_full = qdo_full + 1;         // [3]
  uint64_t* k_empty = k_full + 3;          // [3], count 2: S (front) and dQ (back) both read K
  uint64_t* v_full = k_empty + 3;
  uint64_t* v_empty = v_full + 1;
  uint64_t* s_full = v_empty + 1;          // [2]
  uint64_t* s_free = s_full + 2;           // [2], count 8
  uint64_t* dp_full = s_free + 2;
  uint64_t* dp_free = dp_full + 1;         // count 8
  uint64_t* ds_ready = dp_free + 1;        // count 8
  uint64_t* ds_free = ds_ready + 1;
  uint64_t* final_done = ds_free + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(final_done + 1);
  int* s_work = reinterpret_cast<int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kv_head = head / (p.heads_q / p.heads_kv);

  // ------------------------------------------------------------ locate the query block
  if (threadIdx.x == 0) {
    int blk = gridDim.x - 1 - blockIdx.x, acc = 0, found = 0;   // late (long) rows first
    for (int d = 0; d < p.num_docs; ++d) {
      const int s0 = p.cu_seqlens[d], len = p.cu_seqlens[d + 1] - s0;
      const int nb = (len + kBwB - 1) / kBwB;
      if (blk < acc + nb) {
        s_work[0] = s0; s_work[1] = len; s_work[2] = (blk - acc) * kBwB; found = 1;
        break;
      }
      acc += nb;
    }
    s_work[3] = found;
  }
  __syncthreads();
  if (!s_work[3]) return;
  const int doc_start = s_work[0], doc_len = s_work[1], q0 = s_work[2];
  if (doc_start + q0 + kBwB <= p.q_off || doc_start + q0 >= p.q_off + p.q_rows) return;   // rows not held here
  const int kcol_lo = p.k_off - doc_start, kcol_hi = kcol_lo + p.k_rows;      // keys held by this call (document columns)
  int j_begin = (p.window > 0) ? max(0, q0 - p.window + 1) / kBwB : 0;
  int j_end = q0 / kBwB + 1;                          // up to and including the diagonal block
  j_begin = max(j_begin, max(kcol_lo, 0) / kBwB);
  j_end = min(j_end, (kcol_hi > 0) ? (kcol_hi + kBwB - 1) / kBwB : 0);
  const int num_iters = j_end - j_begin;
  if (num_iters <= 0) {
    // no held key is visible to these rows: their partial dQ is zero
    for (int idx = threadIdx.x; idx < kBwB * (kBwD / 8); idx += blockDim.x) {
      const int row = q0 + idx / (kBwD / 8), c = (idx % (kBwD / 8)) * 8;
      const int grow = doc_start + row - p.q_off;
      if (row < doc_len && grow >= 0 && grow < p.q_rows)
        *reinterpret_cast<uint4*>(p.dq + (static_cast<long long>(grow) * p.heads_q + head) * kBwD + c) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 2); }
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 8); }
    mbar_init(dp_full, 1);
    mbar_init(dp_free, 8);
    mbar_init(ds_ready, 8);
    mbar_init(ds_free, 1);
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
      mbar_expect_tx(qdo_full, 2 * kBwTile);
      bw_load_tile(q_s, &tmQ, qdo_full, head * kBwD, doc_start + q0 - p.q_off);
      bw_load_tile(do_s, &tmDO, qdo_full, head * kBwD, doc_start + q0 - p.q_off);
      bool ok = true;
      int ks = 0;
      uint32_t kph = 0;
      for (int n = 0; n < num_iters && ok; ++n) {
        const int krow = doc_start + (j_begin + n) * kBwB - p.k_off;        // rows outside read as zero
        if (!mbar_wait(&k_empty[ks], kph ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
        mbar_expect_tx(&k_full[ks], kBwTile);
        bw_load_tile(k_s + ks * kBwTile, &tmK, &k_full[ks], kv_head * kBwD, krow);
        if (++ks == 3) { ks = 0; kph ^= 1; }
        if (!mbar_wait(v_empty, (n & 1) ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
        mbar_expect_tx(v_full, kBwTile);
        bw_load_tile(v_s, &tmV, v_full, kv_head * kBwD, krow);
      }
      if (!ok) __nanosleep(200000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ front MMA issuer: S, dP
    if (lane == 0) {
      const uint32_t k_a = smem_u32(k_s), v_a = smem_u32(v_s), q_a = smem_u32(q_s), do_a = smem_u32(do_s);
      bool ok = mbar_wait(qdo_full, 0, p.status, kTimeoutFullBarrier);
      int ks = 0;
      uint32_t kph = 0;
      for (int n = 0; n < num_iters && ok; ++n) {
        const int st = n & 1;                 // S buffer
        const uint32_t ph = (n >> 1) & 1;
        if (!mbar_wait(&k_full[ks], kph, p.status, kTimeoutFullBarrier)) break;
        // S buffer st was last used by block n - 2
        if (n >= 2 && !mbar_wait(&s_free[st], ph ^ 1, p.status, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        bw_mma_block<false, false>(tmem_base + kTmS + st * 128, q_a, k_a + ks * kBwTile, false);
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[ks]);
        if (++ks == 3) { ks = 0; kph ^= 1; }
        if (!mbar_wait(v_full, n & 1, p.status, kTimeoutFullBarrier)) break;
        if (n > 0 && !mbar_wait(dp_free, (n - 1) & 1, p.status, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        bw_mma_block<false, false>(tmem_base + kTmDP, do_a, v_a, false);
        umma_commit(dp_full);
        umma_commit(v_empty);
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ back MMA issuer: dQ
    if (lane == 0) {
      const uint32_t k_a = smem_u32(k_s), ds_a = smem_u32(ds_s);
      bool ok = true;
      int ks = 0;
      for (int n = 0; n < num_iters && ok; ++n) {
        // dS of block n is published only after S of block n was read, so K stage ks is loaded
        if (!mbar_wait(ds_ready, n & 1, p.status, kTimeoutPeerFlag)) { ok = false; break; }
        tc_fence_after();
        // dQ[row][d] += sum_key dS[row][key] K[key][d]: K is read MN-major
        bw_mma_block<false, true>(tmem_base + kTmDQ, ds_a, k_a + ks * kBwTile, n > 0);
        umma_commit(ds_free);
        umma_commit(&k_empty[ks]);
        if (++ks == 3) ks = 0;
      }
      if (ok) umma_commit(final_done);
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue warps
    const int w = (warp - 3) >> 2;
    const int qtr = warp & 3;
    const int r = qtr * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    uint8_t* ds_row = ds_s + w * (kBwTile / 2) + r * 128;
    const int row = q0 + r;
    const int grow = doc_start + row - p.q_off;           // row inside the held slice
    const bool row_ok = row < doc_len && grow >= 0 && grow < p.q_rows;
    const long long stat_idx = static_cast<long long>(head) * p.q_rows + grow;
    const float neg_lse2 = row_ok ? -p.lse[stat_idx] * 1.4426950408889634f : 0.f;
    const float neg_delta = row_ok ? -p.delta[stat_idx] : 0.f;
    bool ok = true;
    for (int n = 0; n < num_iters && ok; ++n) {
      const int st = n & 1;
      const int col0 = (j_begin + n) * kBwB + 64 * w;
      const int causal_hi = row_ok ? row - col0 : -1;
      const int lim_hi = min(causal_hi, kcol_hi - 1 - col0);
      const int lim_lo = max((p.window > 0) ? causal_hi - p.window : -1, kcol_lo - 1 - col0);
      ok = mbar_wait_poll(&s_full[st], (n >> 1) & 1, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float pf[64];
      bw_load_p(tmem_base + lane_off + kTmS + st * 128 + 64 * w, pf, lim_hi, lim_lo, p.scale_log2, neg_lse2);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[st]);

      ok = mbar_wait_poll(dp_full, n & 1, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      bw_load_ds(tmem_base + lane_off + kTmDP + 64 * w, pf, neg_delta);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dp_free);
      if (n > 0) {                                        // dQ of block n - 1 still reads dS
        ok = mbar_wait_poll(ds_free, (n - 1) & 1, p.status, kTimeoutTmemFull);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      bw_store_row(ds_row, r, pf);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    // ---------------------------------------------------------- epilogue: dQ (lane = row)
    if (ok) {
      ok = mbar_wait(final_done, 0, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dst = p.dq + (static_cast<long long>(grow) * p.heads_q + head) * kBwD + 64 * w;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t gv[32];
        tmem_ld_32x32(tmem_base + lane_off + kTmDQ + 64 * w + 32 * c, gv);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(gv[8 * e + 0]) * p.scale, __uint_as_float(gv[8 * e + 1]) * p.scale);
            o.y = pack_bf16(__uint_as_float(gv[8 * e + 2]) * p.scale, __uint_as_float(gv[8 * e + 3]) * p.scale);
            o.z = pack_bf16(__uint_as_float(gv[8 * e + 4]) * p.scale, __uint_as_float(gv[8 * e + 5]) * p.scale);
            o.w = pack_bf16(__uint_as_float(gv[8 * e + 6]) * p.scale, __uint_as_float(gv[8 * e + 7]) * p.scale);
            *reinterpret_cast<uint4*>(dst + 32 * c + 8 * e) = o;
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

}  // namespace prb

// q, k, v as in prb_flash_fwd; o / d_o: bf16 [T, heads_q, 128] (pitches ld_o / ld_do); lse: fp32
// [heads_q, T]. Scratch supplied by the caller: delta fp32 [heads_q, T]. Outputs dq (contiguous
// [T, heads_q, 128]), dk, dv (pitches ld_dk / ld_dv). max_blocks = sum over documents of
// ceil(len / 128).
// Context-parallel form: q / o / d_o / lse / delta / dq hold only the global rows
// [q_off, q_off + q_rows); k / v / dk / dv and cu_seqlens describe the complete sequence.
//
// Block form (`prb_flash_bwd_block`): in addition k / v / dk / dv hold only the global rows [k_off, k_off + k_rows).
// With o and lse the FINAL output and log-sum-exp of the rows (over all keys of all blocks), dq is the rows' partial
// gradient from these keys and dk / dv are these keys' partial gradients from these rows; the caller sums the
// partials. Every row of dq and every row of dk / dv is written (zeros where nothing is visible).
PRB_API int prb_flash_bwd_block(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                const float* lse, float* delta, void* dq, void* dk, void* dv, const int* cu_seqlens,
                                int num_docs, int total_q, int q_off, int q_rows, int k_off, int k_rows, int heads_q,
                                int heads_kv, int head_dim, long long ld_q, long long ld_k, long long ld_v,
                                long long ld_o, long long ld_do, long long ld_dk, long long ld_dv, float scale,
                                int window, int max_blocks, int* status, void* stream_) {
  using namespace prb;
  if (q_off < 0 || q_rows <= 0 || q_off + q_rows > total_q) return -3;
  if (k_off < 0 || k_rows <= 0 || k_off + k_rows > total_q) return -3;
  if (head_dim != kBwD || heads_q % heads_kv) return -2;
  if (total_q <= 0 || num_docs <= 0) return 0;
  if ((ld_q % 8) || (ld_k % 8) || (ld_v % 8) || (ld_do % 8) || (ld_dk % 8) || (ld_dv % 8)) return -4;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  CUtensorMap tmQ, tmK, tmV, tmDO;
  int rc = make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)q_rows, (uint64_t)heads_q * kBwD,
                        (uint64_t)ld_q, kBwB, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmDO, d_o, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)q_rows, (uint64_t)heads_q * kBwD,
                    (uint64_t)ld_do, kBwB, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)k_rows, (uint64_t)heads_kv * kBwD,
                    (uint64_t)ld_k, kBwB, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)k_rows, (uint64_t)heads_kv * kBwD,
                    (uint64_t)ld_v, kBwB, 64, true);
  if (rc) return rc;
  const long long items = static_cast<long long>(q_rows) * heads_q;
  flash_bwd_delta_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, stream>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, q_rows, heads_q, ld_o, ld_do);
  FaBwdParams p;
  p.cu_seqlens = cu_seqlens; p.num_docs = num_docs; p.total_q = total_q; p.heads_q = heads_q; p.heads_kv = heads_kv;
  p.q_off = q_off; p.q_rows = q_rows;
  p.k_off = k_off; p.k_rows = k_rows;
  p.lse = lse; p.delta = delta;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk); p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.ld_dk = ld_dk; p.ld_dv = ld_dv;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.window = window; p.status = status;
  static prb::DeviceOnce configured;
  if (configured.pending()) {
    if (cudaFuncSetAttribute(flash_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwSmem) != cudaSuccess ||
        cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwSmem) != cudaSuccess)
      return -10;
    configured.mark();
  }
  flash_bwd_dkdv_kernel<<<dim3(max_blocks, heads_kv), kBwThreads, kBwSmem, stream>>>(tmQ, tmK, tmV, tmDO, p);
  flash_bwd_dq_kernel<<<dim3(max_blocks, heads_q), kBwThreads, kBwSmem, stream>>>(tmQ, tmK, tmV, tmDO, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_flash_bwd_slice(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                const float* lse, float* delta, void* dq, void* dk, void* dv, const int* cu_seqlens,
                                int num_docs, int total_q, int q_off, int q_rows, int heads_q, int heads_kv,
                                int head_dim, long long ld_q, long long ld_k, long long ld_v, long long ld_o,
                                long long ld_do, long long ld_dk, long long ld_dv, float scale, int window,
                                int max_blocks, int* status, void* stream_) {
  return prb_flash_bwd_block(q, k, v, o, d_o, lse, delta, dq, dk, dv, cu_seqlens, num_docs, total_q, q_off, q_rows, 0,
                             total_q, heads_q, heads_kv, head_dim, ld_q, ld_k, ld_v, ld_o, ld_do, ld_dk, ld_dv, scale,
                             window, max_blocks, status, stream_);
}

// dq_acc is unused (kept in the signature for existing callers; may be null).
PRB_API int prb_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                          const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                          const int* cu_seqlens, int num_docs, int total_q, int heads_q, int heads_kv, int head_dim,
                          long long ld_q, long long ld_k, long long ld_v, long long ld_o, long long ld_do,
                          long long ld_dk, long long ld_dv, float scale, int window, int max_blocks, int* status,
                          void* stream_) {
  (void)dq_acc;
  return prb_flash_bwd_slice(q, k, v, o, d_o, lse, delta, dq, dk, dv, cu_seqlens, num_docs, total_q, 0, total_q, heads_q,
                             heads_kv, head_dim, ld_q, ld_k, ld_v, ld_o, ld_do, ld_dk, ld_dv, scale, window, max_blocks,
                             status, stream_);
}
