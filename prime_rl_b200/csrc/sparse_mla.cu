// Sparse multi-head-latent attention forward for sm_100a (DSA: every query attends to the top-k
// rows of one shared latent KV stream that an indexer selected for it).
//
//   q    bf16 [T, H, 576]   absorbed queries: 512 latent channels + 64 rotary channels, H <= 128
//   kv   bf16 [S, 576]      latent KV stream (one "head"); values are its first 512 channels
//   idx  int32 [T, topk]    selected rows per query; anything outside [0, S) is an empty slot
//   out  bf16 [T, H, 512],  lse fp32 [T, H] (natural log; -inf for a query without any slot)
//
// One CTA handles one query token and one 256-channel half of the output (grid = 2 x T): all H
// heads are the M = 128 rows of the tcgen05 tiles, so a selected KV row is gathered once per CTA
// and shared by every head. Per block of 64 selected rows:
//
//   gather warps   cp.async 16-byte units of the 64 rows into shared memory in the 128-byte
//                  swizzled K-major layout that TMA would have produced (empty slots are
//                  zero-filled), so that the same tile is the B operand of both products
//   MMA thread     S = Q K^T (9 x 4 tcgen05.mma, K = 576) into TMEM; after the softmax warps
//                  have replaced S by P: O += P V, with P read from TMEM (A operand) and V the
//                  MN-major view of the tile's channels [256 half, 256 half + 256)
//   softmax warps  one thread per head row: online softmax in the exp2 domain with a lazy
//                  rescale of O (only when the running maximum grew by more than 8), P packed
//                  to bf16 into TMEM
//
// The accumulators of 128 heads x 512 channels would fill all 512 TMEM columns by themselves,
// which is why the output channels are split over two CTAs (each repeats Q K^T). Q (147 KB) and
// one KV tile (74 KB) fill the shared memory of the SM, so there is no second tile: the stages of a
// block run one after another (measured per block of 64 rows at 1.9 GHz: gather 1.4 k cycles,
// Q K^T 2.4 k, softmax 1.4 k, P V 0.5 k). Refilling the five k-blocks that only Q K^T reads while
// softmax and P V still run was tried and measured slower (6.13 ms against 5.91 ms at T = 4096).
// Every wait is bounded and reports through the status word.
//
// Takes the place of the reference's TileLang kernel
// (src/prime_rl/trainer/models/kernels/sparse_mla_fwd.py:23-186).
#include "common.cuh"
#include "tma_host.cuh"

namespace prb {

constexpr int kMlaD = 576;          // score channels
constexpr int kMlaDv = 512;         // value channels
constexpr int kMlaHalf = 256;       // output channels per CTA
constexpr int kMlaBN = 64;          // selected rows per block
constexpr int kMlaKB = kMlaD / 64;  // 9 k-blocks of 64 channels
constexpr int kMlaQBytes = 128 * kMlaD * 2;        // 147456
constexpr int kMlaKvBytes = kMlaBN * kMlaD * 2;    // 73728
constexpr int kMlaSmem = kMlaQBytes + kMlaKvBytes + 1024 /*align*/ + 512 /*barriers, mask, indices*/;
constexpr int kMlaThreads = 352;    // warp 0 MMA + Q load, warps 1-4 softmax, warps 5-10 gather
constexpr int kMlaGather = 192;     // gather threads: 24 segments of 128 bytes per pass
constexpr uint32_t kMlaColS = 0, kMlaColP = 64, kMlaColO = 128;

__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

struct MlaParams {
  const __nv_bfloat16* kv;
  const int* idx;
  __nv_bfloat16* out;
  float* lse;
  int T, H, S, topk;
  float scale_log2;   // softmax scale * log2(e)
  int* status;
};

__global__ void __launch_bounds__(kMlaThreads, 1)
sparse_mla_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const MlaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + kMlaQBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kMlaQBytes + kMlaKvBytes);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 2;
  uint64_t* s_full = bars + 3;
  uint64_t* p_ready = bars + 4;
  uint64_t* o_done = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  uint32_t* valid_mask = tmem_slot + 1;   // [2 buffers][2 words]: bit r = row r of the block is a real slot
  int* fail_flag = reinterpret_cast<int*>(valid_mask + 4);      // set when a gather thread's wait ran out
  int* blk_idx = reinterpret_cast<int*>(smem + kMlaQBytes + kMlaKvBytes + 256);   // [2 buffers][64] row indices

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = blockIdx.x, t = blockIdx.y;
  const int nblocks = p.topk / kMlaBN;

  if (threadIdx.x == 0) {
    *fail_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(kv_full, kMlaGather);
    mbar_init(kv_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ------------------------------------------------------------ Q load + MMA issuer
    if (lane == 0) {
      mbar_expect_tx(q_full, kMlaQBytes);
      for (int c = 0; c < kMlaKB; ++c) tma_load_2d(q_s + c * 16384, &tmQ, q_full, c * 64, t * p.H);
      bool ok = mbar_wait(q_full, 0, p.status, kTimeoutFullBarrier);
      constexpr uint32_t idesc_qk = umma_idesc(1, 128, kMlaBN, false, false);
      constexpr uint32_t idesc_pv = umma_idesc(1, 128, kMlaHalf, false, true);
      const uint32_t q_addr = smem_u32(q_s), kv_addr = smem_u32(kv_s);
      for (int j = 0; ok && j < nblocks; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait_poll(kv_full, ph, p.status, kTimeoutFullBarrier)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < kMlaKB; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base + kMlaColS, umma_smem_desc(q_addr + c * 16384 + k * 32, 0, 1024),
                     umma_smem_desc(kv_addr + c * 8192 + k * 32, 0, 1024), idesc_qk, (c | k) != 0);
        }
        umma_commit(s_full);
        if (!mbar_wait_poll(p_ready, ph, p.status, kTimeoutTmemFull)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kMlaBN / 16; ++k)
          umma_f16_ts(tmem_base + kMlaColO, tmem_base + kMlaColP + k * 8,
                      umma_smem_desc(kv_addr + (half * 4) * 8192 + k * 2048, 8192, 1024), idesc_pv, (j | k) != 0);
        umma_commit(kv_empty);
        if (j == nblocks - 1) umma_commit(o_done);
      }
      if (!ok) __nanosleep(200000);   // let copies that are still in flight land before exit
    }
  } else if (warp <= 4) {
    // ------------------------------------------------------------ softmax (one thread per head row)
    const int q4 = warp & 3;                        // TMEM lane quarter this warp may access
    const int row = q4 * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblocks; ++j) {
      const uint32_t ph = j & 1;
      ok = mbar_wait_poll(s_full, ph, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t v0[32], v1[32];
      tmem_ld_32x32(tmem_base + kMlaColS + lane_off, v0);
      tmem_ld_32x32(tmem_base + kMlaColS + 32 + lane_off, v1);
      tmem_ld_wait();
      const uint32_t mk0 = valid_mask[(j & 1) * 2], mk1 = valid_mask[(j & 1) * 2 + 1];
      if ((mk0 & mk1) != 0xffffffffu) {             // rare: a block with empty slots (warp-uniform branch)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (!((mk0 >> i) & 1u)) v0[i] = 0xff800000u;   // -inf
          if (!((mk1 >> i) & 1u)) v1[i] = 0xff800000u;
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(v0[i]), __uint_as_float(v1[i])));
      mx *= p.scale_log2;                           // the scale is positive: max commutes with it
      // lazy rescale: keep the reference maximum while the new one is within 2^8 of it
      if (mx > m_ref + 8.f) {
        if (m_ref != -INFINITY) {
          const float alpha = exp2f(m_ref - mx);
          l *= alpha;
          for (int c = 0; c < kMlaHalf / 32; ++c) {
            uint32_t ov[32];
            tmem_ld_32x32(tmem_base + kMlaColO + c * 32 + lane_off, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st_32x32(tmem_base + kMlaColO + c * 32 + lane_off, ov);
          }
          tmem_st_wait();
        }
        m_ref = mx;
      }
      uint32_t pk[32];
      float sum = 0.f;
      if (m_ref == -INFINITY) {                     // every slot so far was empty
#pragma unroll
        for (int i = 0; i < 32; ++i) pk[i] = 0u;
      } else {
        const float neg = -m_ref, sc = p.scale_log2;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a0 = ex2_approx(fmaf(__uint_as_float(v0[2 * i]), sc, neg));
          const float b0 = ex2_approx(fmaf(__uint_as_float(v0[2 * i + 1]), sc, neg));
          const float a1 = ex2_approx(fmaf(__uint_as_float(v1[2 * i]), sc, neg));
          const float b1 = ex2_approx(fmaf(__uint_as_float(v1[2 * i + 1]), sc, neg));
          sum += (a0 + b0) + (a1 + b1);
          pk[i] = pack_bf16(a0, b0);
          pk[16 + i] = pack_bf16(a1, b1);
        }
      }
      l += sum;
      tmem_st_32x32(tmem_base + kMlaColP + lane_off, pk);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok) {
      ok = mbar_wait(o_done, 0, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool live = row < p.H;
      __nv_bfloat16* dst = p.out + (static_cast<long long>(t) * p.H + row) * kMlaDv + half * kMlaHalf;
      for (int c = 0; c < kMlaHalf / 32; ++c) {
        uint32_t ov[32];
        tmem_ld_32x32(tmem_base + kMlaColO + c * 32 + lane_off, ov);
        tmem_ld_wait();
        if (live) {
          uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(ov[8 * i + 0]) * inv, __uint_as_float(ov[8 * i + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv);
            d4[i] = w;
          }
        }
      }
      if (live && half == 0)
        p.lse[static_cast<long long>(t) * p.H + row] = l > 0.f ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  } else {
    // ------------------------------------------------------------ gather (128 threads)
    const int g = threadIdx.x - 160;               // 0..191
    const int unit = g & 7, seg0 = g >> 3;         // 24 segments of 128 bytes per pass
    constexpr int kSegs = kMlaGather / 8;
    constexpr int kPasses = kMlaBN * kMlaKB / kSegs;   // 24 passes x 24 segments = 64 rows x 9 k-blocks
    const uint32_t kv_addr = smem_u32(kv_s);
    const int* my_idx = p.idx + static_cast<long long>(t) * p.topk;
    const uint8_t* kv_bytes = reinterpret_cast<const uint8_t*>(p.kv);
    int next_id = (g < kMlaBN) ? my_idx[g] : 0;    // threads 0..63 carry one row index of the coming block
    uint32_t dst[kPasses];
#pragma unroll
    for (int pass = 0; pass < kPasses; ++pass) {
      const int seg = pass * kSegs + seg0, r = seg / kMlaKB, c = seg - r * kMlaKB;
      dst[pass] = kv_addr + c * 8192 + r * 128 + ((unit ^ (r & 7)) << 4);
    }
    for (int j = 0; j < nblocks; ++j) {
      // everything that does not touch the KV tile happens before the wait for its release
      int* bidx = blk_idx + (j & 1) * kMlaBN;
      if (g < kMlaBN) {
        const bool live = next_id >= 0 && next_id < p.S;
        bidx[g] = live ? next_id : -1;
        const uint32_t bits = __ballot_sync(0xffffffffu, live);
        if ((g & 31) == 0) valid_mask[(j & 1) * 2 + (g >> 5)] = bits;
        if (j + 1 < nblocks) next_id = my_idx[(j + 1) * kMlaBN + g];     // in flight while this block is copied
      }
      asm volatile("bar.sync 2, 192;" ::: "memory");
      uint32_t src[kPasses];                        // offset into kv in 16-byte units, or ~0 for an empty slot
#pragma unroll
      for (int pass = 0; pass < kPasses; ++pass) {
        const int seg = pass * kSegs + seg0, r = seg / kMlaKB, c = seg - r * kMlaKB;
        const int id = bidx[r];
        src[pass] = id >= 0 ? static_cast<uint32_t>(id) * (kMlaD / 8) + c * 8 + unit : 0xffffffffu;
      }
      if (j > 0 && !mbar_wait_poll(kv_empty, (j - 1) & 1, p.status, kTimeoutEmptyBarrier)) atomicExch(fail_flag, 1);
      asm volatile("bar.sync 2, 192;" ::: "memory");
      if (*reinterpret_cast<volatile int*>(fail_flag) != 0) break;   // the same verdict for all gather threads
#pragma unroll
      for (int pass = 0; pass < kPasses; ++pass)
        cp_async_16(dst[pass], kv_bytes + (src[pass] != 0xffffffffu ? static_cast<size_t>(src[pass]) << 4 : 0),
                    src[pass] != 0xffffffffu ? 16u : 0u);
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      fence_async_smem();                           // generic-proxy writes -> visible to the tensor core
      mbar_arrive(kv_full);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

}  // namespace prb

// q [T*H, 576] bf16 contiguous, kv [S, 576] bf16 contiguous, idx [T, topk] int32 (topk a multiple of
// 64), out [T, H, 512] bf16, lse [T, H] fp32. Returns 0 when the launch was issued.
PRB_API int prb_sparse_mla_fwd(const void* q, const void* kv, const int* idx, void* out, float* lse, int T, int H, int S,
                               int topk, float scale, int* status, void* stream_) {
  using namespace prb;
  if (T <= 0) return 0;
  if (H <= 0 || H > 128 || S <= 0 || topk <= 0 || (topk % kMlaBN) != 0) return -3;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(kv) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -4;
  CUtensorMap tmQ;
  int rc = make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)T * H, (uint64_t)kMlaD, (uint64_t)kMlaD,
                        128, 64, true);
  if (rc) return rc;
  static prb::DeviceOnce configured;
  if (configured.pending()) {
    if (cudaFuncSetAttribute(sparse_mla_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem) != cudaSuccess)
      return -10;
    configured.mark();
  }
  MlaParams p;
  p.kv = reinterpret_cast<const __nv_bfloat16*>(kv);
  p.idx = idx;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.T = T; p.H = H; p.S = S; p.topk = topk;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  dim3 grid(2, T);
  sparse_mla_fwd_kernel<<<grid, kMlaThreads, kMlaSmem, reinterpret_cast<cudaStream_t>(stream_)>>>(tmQ, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
