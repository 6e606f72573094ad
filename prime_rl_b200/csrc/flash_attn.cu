// Flash attention forward for sm_100a: varlen (packed documents), causal, optional sliding
// window, GQA, head_dim 128, bf16 in / bf16 out + fp32 log-sum-exp.
//
// One CTA owns 256 query rows of one head inside one document, as two 128-row tiles that
// run independently and share the K / V stream and the tensor core. Per 128-key block and tile:
//     S = Q K^T           tcgen05.mma  M128 x N128 x K128 (Q, K from shared memory, S in TMEM);
//                         N = 128 because an N = 64 product runs at half the tensor rate
//     softmax             4 warps, one thread per row, in two 64-key halves: S read with
//                         tcgen05.ld, running max / sum in registers, P written as bf16 into a
//                         128B-swizzled shared tile, O (TMEM) rescaled in place only when the
//                         running max moved by more than 2^8. The S buffer is handed back to
//                         the tensor core as soon as its second half is in registers, so the
//                         next Q K^T overlaps the exponentials of this block.
//     O += P V            tcgen05.mma  M128 x N128 x K64 per half (P from shared memory, V MN-major)
// K (128-key stages) and V (64-key stages) arrive by TMA (no multicast) through separate rings.
// TMEM per tile (256 columns): S (128) | O (128).
//
// Warp roles: 0 = TMA producer, 1 / 2 = MMA issuer of tile 0 / 1 (one thread each; a single
// issuer would serialise the two tiles' barrier round trips), 3..6 = softmax of tile 0,
// 7..10 = softmax of tile 1. All waits are bounded and report through the status word.
//
// Replaces flash_attn_varlen_func in the reference (src/prime_rl/trainer/models/layers/attn.py:101-115).
#include "common.cuh"
#include "tma_host.cuh"

namespace prb {

constexpr int kFaD = 128;        // head dim
constexpr int kFaBM = 128;       // rows per tile
constexpr int kFaBN = 128;       // keys per Q K^T block
constexpr int kFaHN = 64;        // keys per softmax / P V half
constexpr int kFaKStages = 2;
constexpr int kFaVStages = 3;
constexpr int kFaThreads = 352;

constexpr int kQBytes = kFaBM * kFaD * 2;          // 32 KB per tile (two 16 KB slabs of 64 columns)
constexpr int kKBytes = kFaBN * kFaD * 2;          // 32 KB per stage (two 16 KB slabs of 64 columns)
constexpr int kVBytes = kFaHN * kFaD * 2;          // 16 KB per stage (two 8 KB slabs)
constexpr int kPBytes = kFaBM * kFaHN * 2;         // 16 KB per tile
constexpr int kFaSmem = 2 * kQBytes + kFaKStages * kKBytes + kFaVStages * kVBytes + 2 * kPBytes + 1024 + 512;

struct FaParams {
  const int* cu_seqlens;  // [num_docs + 1]
  int num_docs;
  int total_q;            // T (rows of K / V)
  int q_off, q_rows;      // the query / output tensors hold global rows [q_off, q_off + q_rows) only
  int k_off, k_rows;      // the K / V tensors hold global rows [k_off, k_off + k_rows) only; keys outside do not exist
                          // for this call (ring step of context parallelism: the caller merges the partial results)
  int heads_q, heads_kv;
  __nv_bfloat16* out;     // [T, heads_q, D]
  long long ld_out;       // elements per token
  float* lse;             // [heads_q, T]
  float scale_log2;       // softmax scale * log2(e)
  int window;             // <= 0: none; else a query attends keys with q - k < window
  const float* sinks;     // optional [heads_q]: a per-head logit that only joins the softmax denominator
  int* status;
  // context-parallel gather (flash_fwd_kernel<true> only): K and V of the whole sequence live in one
  // buffer per rank ([K rows | V rows at v_off]) of which rank r has written the rows of its own
  // chunk [r * chunk_rows, (r + 1) * chunk_rows). One extra warp per CTA pulls the chunks of the
  // lower ranks from their owners (`peer[r]` = rank r's buffer) into the local buffer in 16 KB pieces
  // that CTAs claim from a shared counter; `ready[c]` counts the finished pieces of chunk c.
  const uint8_t* peer[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  uint8_t* kv_local = nullptr;
  unsigned* claim = nullptr;
  unsigned* ready = nullptr;
  int cp_rank = 0;
  int chunk_rows = 0;
  long long row_bytes = 0, v_off = 0;
};

constexpr int kFaPiece = 16384;

// Pieces of the chunks 0 .. cp_rank-1 (K region first, then V region of every chunk), claimed
// dynamically: a CTA that is not resident yet owes nothing, so waiting CTAs cannot starve the copy.
__device__ void fa_gather_warp(const FaParams& p, int lane) {
  const long long chunk_bytes = static_cast<long long>(p.chunk_rows) * p.row_bytes;
  const unsigned ppk = static_cast<unsigned>((chunk_bytes + kFaPiece - 1) / kFaPiece);
  const unsigned total = static_cast<unsigned>(p.cp_rank) * 2u * ppk;
  for (;;) {
    unsigned id = 0;
    if (lane == 0) id = atomicAdd(p.claim, 1u);
    id = __shfl_sync(0xffffffffu, id, 0);
    if (id >= total) break;
    const unsigned chunk = id / (2u * ppk), w = id % (2u * ppk);
    const unsigned piece = w % ppk;
    const long long off = (w >= ppk ? p.v_off : 0) + static_cast<long long>(chunk) * chunk_bytes +
                          static_cast<long long>(piece) * kFaPiece;
    const long long len = min(static_cast<long long>(kFaPiece), chunk_bytes - static_cast<long long>(piece) * kFaPiece);
    const int4* src = reinterpret_cast<const int4*>(p.peer[chunk] + off);
    int4* dst = reinterpret_cast<int4*>(p.kv_local + off);
    const int n16 = static_cast<int>(len >> 4);
    for (int i = lane; i < n16; i += 32 * 8) {
      int4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (i + u * 32 < n16) v[u] = __ldcg(src + i + u * 32);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (i + u * 32 < n16) dst[i + u * 32] = v[u];
    }
    __threadfence();
    __syncwarp();
    if (lane == 0) atomicAdd(p.ready + chunk, 1u);
  }
}

// Producer side: rows [row0, row1] are about to be loaded by TMA; wait (bounded) for the chunks of
// lower ranks they touch. `done` caches the chunks already seen complete.
__device__ bool fa_wait_rows(const FaParams& p, int row0, int row1, unsigned& done) {
  const long long chunk_bytes = static_cast<long long>(p.chunk_rows) * p.row_bytes;
  const unsigned want = 2u * static_cast<unsigned>((chunk_bytes + kFaPiece - 1) / kFaPiece);
  const int c1 = min(row1 / p.chunk_rows, p.cp_rank - 1);
  for (int c = row0 / p.chunk_rows; c <= c1; ++c) {
    if ((done >> c) & 1u) continue;
    const unsigned* flag = p.ready + c;
    bool ok = false;
    for (long long spin = 0; spin < (1LL << 24); ++spin) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v >= want) { ok = true; break; }
      __nanosleep(64);
    }
    if (!ok) {
      atomicCAS(p.status, 0, static_cast<int>(kTimeoutPeerFlag));
      return false;
    }
    asm volatile("fence.proxy.async;" ::: "memory");
    done |= 1u << c;
  }
  return true;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  // not volatile: a pure function, so the compiler may batch the MUFU ops of a row
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool GATHER>
__global__ void __launch_bounds__(kFaThreads + (GATHER ? 32 : 0), 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + 2 * kQBytes;
  uint8_t* v_s = k_s + kFaKStages * kKBytes;
  uint8_t* p_s = v_s + kFaVStages * kVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 2 * kPBytes);
  uint64_t* q_full = bars;                      // 1
  uint64_t* k_full = q_full + 1;                // K stages
  uint64_t* k_empty = k_full + kFaKStages;      // count 2: both MMA threads release a stage
  uint64_t* v_full = k_empty + kFaKStages;      // V stages
  uint64_t* v_empty = v_full + kFaVStages;      // count 2
  uint64_t* s_full = v_empty + kFaVStages;      // 2 (per tile)
  uint64_t* s_free = s_full + 2;                // 2, count 4 (softmax warps)
  uint64_t* p_ready = s_free + 2;               // 2, count 4
  uint64_t* o_ready = p_ready + 2;              // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_ready + 2);
  int* s_work = reinterpret_cast<int*>(tmem_slot + 1);  // doc_start, doc_len, row0 (in doc), found

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kv_head = head / (p.heads_q / p.heads_kv);

  // ------------------------------------------------------------ locate this CTA's work
  if (threadIdx.x == 0) {
    const int pair = gridDim.x - 1 - blockIdx.x;  // heavy (late) tiles first
    int found = 0, acc = 0;
    for (int d = 0; d < p.num_docs; ++d) {
      const int s0 = p.cu_seqlens[d], len = p.cu_seqlens[d + 1] - s0;
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
  // context parallelism: this rank holds only a slice of the query rows (keys are complete)
  const int g0 = doc_start + row0;                       // first global row of this CTA
  if (g0 + 2 * kFaBM <= p.q_off || g0 >= p.q_off + p.q_rows) return;

  // rows [q0, q1) of the document for each tile and the 128-key blocks [blk0, nblk) they need
  const int q0_0 = row0, q0_1 = row0 + kFaBM;
  const bool out_0 = (g0 + kFaBM <= p.q_off) || (g0 >= p.q_off + p.q_rows);               // tile 0 not held here
  const bool out_1 = (g0 + 2 * kFaBM <= p.q_off) || (g0 + kFaBM >= p.q_off + p.q_rows);
  const int q1_0 = out_0 ? q0_0 : min(q0_0 + kFaBM, doc_len), q1_1 = out_1 ? q0_1 : min(q0_1 + kFaBM, doc_len);
  // keys held by this call, as columns of the document: [kcol_lo, kcol_hi)
  const int kcol_lo = p.k_off - doc_start, kcol_hi = kcol_lo + p.k_rows;
  int nblk_0 = (q1_0 > q0_0) ? (q1_0 + kFaBN - 1) / kFaBN : 0;
  int nblk_1 = (q1_1 > q0_1) ? (q1_1 + kFaBN - 1) / kFaBN : 0;
  int blk0_0 = (p.window > 0 && nblk_0 > 0) ? max(0, q0_0 - p.window + 1) / kFaBN : 0;
  int blk0_1 = (p.window > 0 && nblk_1 > 0) ? max(0, q0_1 - p.window + 1) / kFaBN : 0;
  if (kcol_lo > 0 || kcol_hi < doc_len) {
    const int b_lo = max(kcol_lo, 0) / kFaBN, b_hi = (kcol_hi > 0) ? (kcol_hi + kFaBN - 1) / kFaBN : 0;
    blk0_0 = max(blk0_0, b_lo); nblk_0 = min(nblk_0, b_hi);
    blk0_1 = max(blk0_1, b_lo); nblk_1 = min(nblk_1, b_hi);
    if (nblk_0 <= blk0_0) nblk_0 = blk0_0 = 0;      // no key of this call is visible to the tile
    if (nblk_1 <= blk0_1) nblk_1 = blk0_1 = 0;
  }
  // union of the two ranges: the K / V stream of this CTA (tile 0 always has rows)
  const int j_begin = (nblk_1 > 0) ? (nblk_0 > 0 ? min(blk0_0, blk0_1) : blk0_1) : blk0_0;
  const int j_end = max(nblk_0, nblk_1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kFaKStages; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 2); }
    for (int i = 0; i < kFaVStages; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 2); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);
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
                      g0 + t * kFaBM - p.q_off);   // rows outside the held slice are zero-filled
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0;
      bool ok = true;
      unsigned chunks_done = 0;
      for (int j = j_begin; j < j_end && ok; ++j) {
        const int krow = doc_start + j * kFaBN - p.k_off;     // may start before row 0: those rows read as zero
        if constexpr (GATHER) {
          if (!fa_wait_rows(p, krow, krow + kFaBN - 1, chunks_done)) { ok = false; break; }
        }
        if (!mbar_wait(&k_empty[ks], kph ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
        mbar_expect_tx(&k_full[ks], kKBytes);
        tma_load_2d(k_s + ks * kKBytes, &tmK, &k_full[ks], kv_head * kFaD, krow);
        tma_load_2d(k_s + ks * kKBytes + kKBytes / 2, &tmK, &k_full[ks], kv_head * kFaD + 64, krow);
        if (++ks == kFaKStages) { ks = 0; kph ^= 1; }
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait(&v_empty[vs], vph ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
          mbar_expect_tx(&v_full[vs], kVBytes);
          tma_load_2d(v_s + vs * kVBytes, &tmV, &v_full[vs], kv_head * kFaD, krow + h * kFaHN);
          tma_load_2d(v_s + vs * kVBytes + kVBytes / 2, &tmV, &v_full[vs], kv_head * kFaD + 64, krow + h * kFaHN);
          if (++vs == kFaVStages) { vs = 0; vph ^= 1; }
        }
      }
      if (!ok) __nanosleep(200000);
    }
  } else if (warp <= 2) {
    // ------------------------------------------------------------ MMA issuer of tile (warp - 1)
    if (lane == 0) {
      const int t = warp - 1;
      const int my_blk0 = t ? blk0_1 : blk0_0, my_nblk = t ? nblk_1 : nblk_0;
      constexpr uint32_t idesc_qk = umma_idesc(1, kFaBM, kFaBN, false, false);
      constexpr uint32_t idesc_pv = umma_idesc(1, kFaBM, kFaD, false, true);
      const uint32_t q_addr = smem_u32(q_s) + t * kQBytes, k_addr = smem_u32(k_s), v_addr = smem_u32(v_s);
      const uint32_t p_addr = smem_u32(p_s) + t * kPBytes;
      const uint32_t s_tm = tmem_base + t * 256, o_tm = s_tm + 128;
      bool ok = mbar_wait(q_full, 0, p.status, kTimeoutFullBarrier);
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0;
      uint32_t n_qk = 0, n_pv = 0;   // products issued so far (phase sources)

      // K block j sits in stage ks: S = Q K^T if this tile needs the block, then release the stage.
      // Every stage is released by both issuers, so a tile that skips a block still arrives
      // (after the stage filled: an earlier arrival could land in the previous phase).
      auto handle_k = [&](int j) {
        if (!mbar_wait(&k_full[ks], kph, p.status, kTimeoutFullBarrier)) { ok = false; return; }
        if (j >= my_blk0 && j < my_nblk) {
          // the softmax warps hand S back once block n_qk - 1 is in their registers
          if (n_qk > 0 && !mbar_wait(&s_free[t], (n_qk - 1) & 1, p.status, kTimeoutTmemEmpty)) { ok = false; return; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t a = umma_smem_desc(q_addr + (kk >> 2) * (kQBytes / 2) + (kk & 3) * 32, 0, 1024);
            const uint64_t b = umma_smem_desc(k_addr + ks * kKBytes + (kk >> 2) * (kKBytes / 2) + (kk & 3) * 32, 0, 1024);
            umma_f16(s_tm, a, b, idesc_qk, kk != 0);
          }
          umma_commit(&s_full[t]);
          umma_commit(&k_empty[ks]);
          ++n_qk;
        } else {
          mbar_arrive(&k_empty[ks]);
        }
        if (++ks == kFaKStages) { ks = 0; kph ^= 1; }
      };
      // one 64-key half of V sits in stage vs: O += P V once the softmax warps published P
      auto handle_v = [&](int j) {
        if (!mbar_wait(&v_full[vs], vph, p.status, kTimeoutFullBarrier)) { ok = false; return; }
        if (j >= my_blk0 && j < my_nblk) {
          if (!mbar_wait(&p_ready[t], n_pv & 1, p.status, kTimeoutPeerFlag)) { ok = false; return; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t a = umma_smem_desc(p_addr + kk * 32, 0, 1024);
            const uint64_t b = umma_smem_desc(v_addr + vs * kVBytes + kk * 2048, kVBytes / 2, 1024);
            umma_f16(o_tm, a, b, idesc_pv, (n_pv | kk) != 0);
          }
          umma_commit(&o_ready[t]);
          umma_commit(&v_empty[vs]);
          ++n_pv;
        } else {
          mbar_arrive(&v_empty[vs]);
        }
        if (++vs == kFaVStages) { vs = 0; vph ^= 1; }
      };

      if (ok && j_begin < j_end) handle_k(j_begin);
      for (int j = j_begin; j < j_end && ok; ++j) {
        handle_v(j);
        // the next Q K^T goes in between the two halves: S is free again as soon as the softmax
        // warps have loaded the second half, long before they publish its P
        if (ok && j + 1 < j_end) handle_k(j + 1);
        if (ok) handle_v(j);
      }
    }
  } else if (GATHER && warp == kFaThreads / 32) {
    // ------------------------------------------------------------ gather warp (context parallelism)
    fa_gather_warp(p, lane);
  } else {
    // ------------------------------------------------------------ softmax warps
    const int t = (warp - 3) >> 2;          // tile
    const int qtr = warp & 3;               // TMEM lane quarter this warp may access
    const int r = qtr * 32 + lane;          // row in tile
    // scalars, not arrays indexed by t: a runtime index would put them in local memory
    const int my_q0 = t ? q0_1 : q0_0, my_q1 = t ? q1_1 : q1_0;
    const int my_blk0 = t ? blk0_1 : blk0_0, my_nblk = t ? nblk_1 : nblk_0;
    const int row = my_q0 + r;              // row in document
    const int grow = doc_start + row - p.q_off;          // row inside the held slice
    const bool row_ok = row < my_q1 && grow >= 0 && grow < p.q_rows;
    const uint32_t lane_off = static_cast<uint32_t>(qtr * 32) << 16;
    const uint32_t s_tm = tmem_base + t * 256 + lane_off;
    const uint32_t o_tm = s_tm + 128;
    uint8_t* p_row = p_s + t * kPBytes + r * 128;
    float m = -INFINITY, l = 0.f;
    uint32_t n = 0, it = 0;                 // blocks / halves done
    bool ok = true;
    for (int j = my_blk0; j < my_nblk && ok; ++j, ++n) {
      ok = mbar_wait_poll(&s_full[t], n & 1, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int h = 0; h < 2; ++h, ++it) {
        uint32_t sv[2][32];
        tmem_ld_32x32(s_tm + h * kFaHN, sv[0]);
        tmem_ld_32x32(s_tm + h * kFaHN + 32, sv[1]);
        tmem_ld_wait();
        if (h == 1) {
          // all of S is in registers: the tensor core may overwrite it with the next block
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_free[t]);
        }
        const int col0 = j * kFaBN + h * kFaHN;
        const bool need_mask = (col0 + kFaHN - 1 > my_q0) || (p.window > 0 && my_q1 - 1 - col0 >= p.window) ||
                               (col0 < kcol_lo) || (col0 + kFaHN > kcol_hi);
        // raw scores; masked entries become -inf. The running reference `m` (log2 domain) only
        // moves when the block maximum exceeds it by more than 8: P then stays below 2^8, and
        // most blocks need no rescale of O at all.
        float s[64];
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains instead of one
        // two straight-line variants: a per-element `if (need_mask)` is compiled to 64 branches
        if (need_mask) {
          const int causal_hi = row - col0;
          const int lim_hi = min(causal_hi, kcol_hi - 1 - col0);                                   // keep c <= lim_hi
          const int lim_lo = max((p.window > 0) ? causal_hi - p.window : -1, kcol_lo - 1 - col0);  // keep c >  lim_lo
#pragma unroll
          for (int c = 0; c < 64; ++c) {
            const float x = __uint_as_float(sv[c >> 5][c & 31]);
            s[c] = ((c <= lim_hi) & (c > lim_lo)) ? x : -INFINITY;
            mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 64; ++c) {
            s[c] = __uint_as_float(sv[c >> 5][c & 31]);
            mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
          }
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float m_blk = mx * p.scale_log2;          // scale > 0, so max commutes with it
        float alpha = 1.f;
        if (m_blk > m + 8.f) {                          // also true on the first unmasked block (m = -inf)
          alpha = ex2(m - m_blk);                       // m = -inf -> 0
          m = m_blk;
        }
        // rows without any valid key so far keep m = -inf: use 0 so that no NaN appears
        const float neg_m = (m == -INFINITY) ? 0.f : -m;
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const float p0 = ex2(fmaf(s[c], p.scale_log2, neg_m)), p1 = ex2(fmaf(s[c + 1], p.scale_log2, neg_m));
          sum4[(c >> 1) & 3] += p0 + p1;
          pk[c >> 1] = pack_bf16(p0, p1);
        }
        l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        if (it > 0) {
          // O holds the halves before this one and P is still being read by the last P V:
          // wait for it, then rescale O in place if some row of this warp moved its reference
          ok = mbar_wait_poll(&o_ready[t], (it - 1) & 1, p.status, kTimeoutTmemFull);
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
    }
    // ---------------------------------------------------------- epilogue: O / l, LSE
    if (ok && it > 0) {
      ok = mbar_wait(&o_ready[t], (it - 1) & 1, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        // attention sink: one more column exp(sink - max) in the row sum, no value attached (the output
        // shrinks, the log-sum-exp the backward pass works from grows)
        if (p.sinks != nullptr) l += exp2f(p.sinks[head] * 1.4426950408889634f - m);
        const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
        __nv_bfloat16* dst = p.out + static_cast<long long>(grow) * p.ld_out +
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
          p.lse[static_cast<long long>(head) * p.q_rows + grow] =
              (l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
    } else if (ok && it == 0 && row_ok) {
      // no key block of this call is visible to the tile: an empty partial result (weight zero in the merge)
      __nv_bfloat16* dst = p.out + static_cast<long long>(grow) * p.ld_out + static_cast<long long>(head) * kFaD;
#pragma unroll
      for (int i = 0; i < 16; ++i) *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(0, 0, 0, 0);
      p.lse[static_cast<long long>(head) * p.q_rows + grow] = -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// Combines a partial attention result over one key range into the running result of the rows: one warp per
// (token, head). acc / lse_acc: fp32 [T, H, 128] / [H, T]; part / lse_part: bf16 [T, H, 128] / fp32 [H, T].
//   lse = log(exp(lse_acc) + exp(lse_part)), acc = acc exp(lse_acc - lse) + part exp(lse_part - lse)
// A partial result with lse = -inf (no visible key) leaves the row unchanged.
__global__ void __launch_bounds__(256)
attn_merge_kernel(float* __restrict__ acc, float* __restrict__ lse_acc, const __nv_bfloat16* __restrict__ part,
                  const float* __restrict__ lse_part, long long T, int heads) {
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (item >= T * heads) return;
  const long long t = item / heads;
  const int h = static_cast<int>(item - t * heads);
  const long long si = static_cast<long long>(h) * T + t;
  const float la = lse_acc[si], lp = lse_part[si];
  if (lp == -INFINITY) return;
  const float mx = fmaxf(la, lp);
  const float wa = __expf(la - mx), wp = __expf(lp - mx);       // la = -inf -> 0
  const float inv = 1.f / (wa + wp);
  float4* a = reinterpret_cast<float4*>(acc + (t * heads + h) * kFaD) + lane;
  const uint2 pv = *(reinterpret_cast<const uint2*>(part + (t * heads + h) * kFaD) + lane);
  const float2 p0 = unpack_bf16(pv.x), p1 = unpack_bf16(pv.y);
  float4 v = *a;
  const float ca = wa * inv, cp = wp * inv;
  v.x = v.x * ca + p0.x * cp; v.y = v.y * ca + p0.y * cp;
  v.z = v.z * ca + p1.x * cp; v.w = v.w * ca + p1.y * cp;
  *a = v;
  __syncwarp();
  if (lane == 0) lse_acc[si] = mx + __logf(wa + wp);
}

}  // namespace prb

// q: bf16 [T, heads_q, 128] (token pitch ld_q elements), k / v: bf16 [T, heads_kv, 128] (pitches
// ld_k / ld_v; views into a packed qkv projection are fine), out: bf16 [T, heads_q, 128],
// lse: fp32 [heads_q, T] (natural log). max_pairs bounds the number of 256-row tile pairs:
// sum over documents of ceil(len / 256).
// Context-parallel form: q / out / lse hold only the global rows [q_off, q_off + q_rows) (lse is
// [heads_q, q_rows]); k / v and cu_seqlens describe the complete sequence of total_q tokens.
//
// Block form (`prb_flash_fwd_block`): in addition k / v hold only the global rows [k_off, k_off + k_rows); keys
// outside that range do not take part, so out / lse are a partial result over those keys (rows that see none of
// them get out = 0 and lse = -inf). Partial results over disjoint key ranges combine with
// lse = logaddexp(lse_a, lse_b), out = out_a exp(lse_a - lse) + out_b exp(lse_b - lse). No sinks in this form.
PRB_API int prb_flash_fwd_block(const void* q, const void* k, const void* v, void* out, float* lse,
                                const int* cu_seqlens, int num_docs, int total_q, int q_off, int q_rows, int k_off,
                                int k_rows, int heads_q, int heads_kv, int head_dim, long long ld_q, long long ld_k,
                                long long ld_v, long long ld_out, float scale, int window, int max_pairs,
                                const float* sinks, int* status, void* stream_) {
  using namespace prb;
  if (q_off < 0 || q_rows <= 0 || q_off + q_rows > total_q) return -3;
  if (k_off < 0 || k_rows <= 0 || k_off + k_rows > total_q) return -3;
  if (sinks != nullptr && (k_off != 0 || k_rows != total_q)) return -5;
  if (head_dim != kFaD || heads_q % heads_kv) return -2;
  if (total_q <= 0 || num_docs <= 0) return 0;
  if ((ld_q % 8) || (ld_k % 8) || (ld_v % 8) || (ld_out % 8)) return -4;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)q_rows, (uint64_t)heads_q * kFaD,
                        (uint64_t)ld_q, kFaBM, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)k_rows, (uint64_t)heads_kv * kFaD,
                    (uint64_t)ld_k, kFaBN, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)k_rows, (uint64_t)heads_kv * kFaD,
                    (uint64_t)ld_v, kFaHN, 64, true);
  if (rc) return rc;
  FaParams p;
  p.cu_seqlens = cu_seqlens; p.num_docs = num_docs; p.total_q = total_q;
  p.q_off = q_off; p.q_rows = q_rows;
  p.k_off = k_off; p.k_rows = k_rows;
  p.heads_q = heads_q; p.heads_kv = heads_kv;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ld_out = ld_out; p.lse = lse;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window; p.status = status; p.sinks = sinks;
  static prb::DeviceOnce configured;
  if (configured.pending()) {
    if (cudaFuncSetAttribute(flash_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFaSmem) != cudaSuccess)
      return -10;
    configured.mark();
  }
  dim3 grid(max_pairs, heads_q);
  flash_fwd_kernel<false><<<grid, kFaThreads, kFaSmem, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Context-parallel forward with the K / V exchange inside the kernel. `kv_local` is this rank's
// buffer [K: total_q rows | V: total_q rows at v_off_bytes], rows of heads_kv * 128 bf16; this rank
// has written the rows [cp_rank * chunk_rows, (cp_rank + 1) * chunk_rows) of both halves, every peer
// its own chunk of its own buffer (`peer_kv[r]`). `counters`: cp_size + 1 unsigned ints (piece claim
// counter, then one arrival counter per chunk); they are zeroed here, stream-ordered. The caller
// orders the launch after all ranks have written their chunk and keeps the chunk unchanged until
// all ranks have finished. Queries: the local rows (global rows [cp_rank * chunk_rows, ...)).
PRB_API int prb_flash_fwd_gather(const void* q, void* kv_local, void* const* peer_kv, long long v_off_bytes, void* out,
                                 float* lse, const int* cu_seqlens, int num_docs, int total_q, int heads_q, int heads_kv,
                                 long long ld_q, long long ld_out, float scale, int window, int max_pairs, int cp_rank,
                                 int cp_size, int chunk_rows, unsigned* counters, int* status, void* stream_) {
  using namespace prb;
  if (cp_size < 1 || cp_size > 8 || cp_rank < 0 || cp_rank >= cp_size || chunk_rows <= 0 ||
      static_cast<long long>(chunk_rows) * cp_size != total_q || heads_q % heads_kv)
    return -3;
  if ((ld_q % 8) || (ld_out % 8) || (v_off_bytes % 16) || (reinterpret_cast<uintptr_t>(kv_local) & 15)) return -4;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const long long ldkv = static_cast<long long>(heads_kv) * kFaD;
  const int q_off = cp_rank * chunk_rows, q_rows = chunk_rows;
  const uint8_t* kbase = reinterpret_cast<const uint8_t*>(kv_local);
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)q_rows, (uint64_t)heads_q * kFaD,
                        (uint64_t)ld_q, kFaBM, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, kbase, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_q, (uint64_t)ldkv, (uint64_t)ldkv,
                    kFaBN, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, kbase + v_off_bytes, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_q, (uint64_t)ldkv,
                    (uint64_t)ldkv, kFaHN, 64, true);
  if (rc) return rc;
  FaParams p;
  p.cu_seqlens = cu_seqlens; p.num_docs = num_docs; p.total_q = total_q;
  p.q_off = q_off; p.q_rows = q_rows;
  p.k_off = 0; p.k_rows = total_q;
  p.heads_q = heads_q; p.heads_kv = heads_kv;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.ld_out = ld_out; p.lse = lse;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window; p.status = status; p.sinks = nullptr;
  for (int r = 0; r < cp_size; ++r) p.peer[r] = reinterpret_cast<const uint8_t*>(peer_kv[r]);
  p.kv_local = reinterpret_cast<uint8_t*>(kv_local);
  p.claim = counters; p.ready = counters + 1;
  p.cp_rank = cp_rank; p.chunk_rows = chunk_rows;
  p.row_bytes = ldkv * 2; p.v_off = v_off_bytes;
  if (cudaMemsetAsync(counters, 0, sizeof(unsigned) * (cp_size + 1), stream) != cudaSuccess) return -12;
  static prb::DeviceOnce configured;
  if (configured.pending()) {
    if (cudaFuncSetAttribute(flash_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFaSmem) != cudaSuccess)
      return -10;
    configured.mark();
  }
  dim3 grid(max_pairs, heads_q);
  flash_fwd_kernel<true><<<grid, kFaThreads + 32, kFaSmem, stream>>>(tmQ, tmK, tmV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_flash_fwd_slice(const void* q, const void* k, const void* v, void* out, float* lse,
                                const int* cu_seqlens, int num_docs, int total_q, int q_off, int q_rows, int heads_q,
                                int heads_kv, int head_dim, long long ld_q, long long ld_k, long long ld_v,
                                long long ld_out, float scale, int window, int max_pairs, const float* sinks,
                                int* status, void* stream_) {
  return prb_flash_fwd_block(q, k, v, out, lse, cu_seqlens, num_docs, total_q, q_off, q_rows, 0, total_q, heads_q,
                             heads_kv, head_dim, ld_q, ld_k, ld_v, ld_out, scale, window, max_pairs, sinks, status,
                             stream_);
}

PRB_API int prb_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_seqlens,
                          int num_docs, int total_q, int heads_q, int heads_kv, int head_dim, long long ld_q,
                          long long ld_k, long long ld_v, long long ld_out, float scale, int window, int max_pairs,
                          int* status, void* stream_) {
  return prb_flash_fwd_slice(q, k, v, out, lse, cu_seqlens, num_docs, total_q, 0, total_q, heads_q, heads_kv, head_dim,
                             ld_q, ld_k, ld_v, ld_out, scale, window, max_pairs, nullptr, status, stream_);
}

// acc fp32 [T, heads, 128] and lse_acc fp32 [heads, T] are updated in place with the partial result (part bf16
// [T, heads, 128] contiguous, lse_part fp32 [heads, T]); start from acc = 0, lse_acc = -inf.
PRB_API int prb_attn_merge(float* acc, float* lse_acc, const void* part, const float* lse_part, long long T, int heads,
                           void* stream_) {
  if (T <= 0 || heads <= 0) return 0;
  const long long items = T * heads;
  prb::attn_merge_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      acc, lse_acc, reinterpret_cast<const __nv_bfloat16*>(part), lse_part, T, heads);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
