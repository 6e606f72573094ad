// Block-scaled fp8 (e4m3) GEMM for sm_100a, dense and grouped (MoE):
//
//   C[m, n] = sum_kb  sa[m, kb] * sb[n / 128, kb] * sum_{k in block kb} Aq[m, k] * Bq[n, k]
//
// Aq [M, K] e4m3 with one fp32 scale per row and 128-wide K block (1 x 128), Bq [N, K] e4m3 with
// one fp32 scale per 128 x 128 block (the layout of DeepSeek-style fp8 checkpoints and of the
// in-flight quantiser of the weight push). The reference gets this from DeepGEMM
// (src/prime_rl/trainer/models/layers/fp8_utils.py, vLLM's fp8 linear in the engine).
//
// One K block (128 e4m3 = one 128-byte swizzled row per tile row) is four tcgen05.mma
// kind::f8f6f4 instructions (K = 32 each) into a TMEM accumulator that is NOT carried across
// K blocks: the epilogue warps read each block's partial sum from TMEM and add it, times the
// block's scale product, to fp32 accumulators in registers (four TMEM buffers, so the next blocks are
// on the tensor core while block kb is being promoted). BN = 128 = one weight scale block, so
// the scale of a tile and K block is one scalar per row. A K block is a few hundred cycles of tensor-core work,
// so the waits between the MMA issuer and the promotion warps poll (test_wait) instead of suspending.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer + TMEM owner, 2..9 = promotion / epilogue: warp w reads TMEM
// lanes 32 (w % 4) .. + 31 (the quarter a warp may address) and columns 64 ((w - 2) / 4) .. + 63, so the
// promotion of one K block is spread over eight warps and costs each of them two tcgen05.ld and 64 FMAs.
// Grouped mode as in gemm.cu: 128-row blocks owned by block_expert[blk] (-1 = unused).
#include "common.cuh"
#include "tma_host.cuh"
#include <cuda_fp8.h>

namespace prb {

constexpr int kF8BM = 128, kF8BN = 128, kF8BK = 128;      // BK in elements = bytes
constexpr int kF8Stages = 6;
constexpr int kF8AccBufs = 4;                  // TMEM accumulators in flight (4 x 128 columns = all of TMEM)
constexpr int kF8EpiWarps = 8;                 // two warps per TMEM lane quarter, 64 accumulator columns each
constexpr int kF8Threads = 64 + 32 * kF8EpiWarps;
constexpr int kF8StageBytes = (kF8BM + kF8BN) * kF8BK;    // 32 KB
constexpr int kF8Smem = kF8Stages * kF8StageBytes + 1024 + 256;

struct Fp8Params {
  int M, N, K;
  const float* sa;          // [M, KB]
  const float* sb;          // [E, ceil(N/128), KB]
  __nv_bfloat16* C;
  long long ldc;
  const int* block_expert;  // nullptr = dense
  int b_rows_per_expert;    // N rows of B per expert
  const int* row_valid;     // optional [M]: rows with a negative entry are padding and are not stored
  int* status;
};

struct Fp8Tile {
  int tile, num_tiles, tiles_m, tiles_n;
  __device__ Fp8Tile(const Fp8Params& p)
      : tile(blockIdx.x - gridDim.x), tiles_m((p.M + kF8BM - 1) / kF8BM), tiles_n((p.N + kF8BN - 1) / kF8BN) {
    num_tiles = tiles_m * tiles_n;
  }
  // n-major inside a group of 8 M blocks so that neighbouring CTAs share B tiles in L2
  __device__ bool next(const Fp8Params& p, int& m_blk, int& n_blk, int& expert) {
    for (;;) {
      tile += gridDim.x;
      if (tile >= num_tiles) return false;
      constexpr int kGroup = 8;
      const int per_group = kGroup * tiles_n;
      const int g = tile / per_group, first_m = g * kGroup;
      const int gsize = min(tiles_m - first_m, kGroup);
      const int r = tile - g * per_group;
      m_blk = first_m + (r % gsize);
      n_blk = r / gsize;
      expert = 0;
      if (p.block_expert == nullptr) return true;
      expert = p.block_expert[m_blk];
      if (expert >= 0) return true;
    }
  }
};

__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kF8Stages * kF8StageBytes);
  uint64_t* empty = full + kF8Stages;
  uint64_t* tfull = empty + kF8Stages;     // [4] partial sum of a K block is in TMEM buffer b
  uint64_t* tempty = tfull + kF8AccBufs;   // [4] count 8: the epilogue warps have read buffer b
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + kF8AccBufs);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = (p.K + kF8BK - 1) / kF8BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kF8Stages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < kF8AccBufs; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], kF8EpiWarps); }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, kF8AccBufs * kF8BN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  int m_blk = 0, n_blk = 0, expert = 0;

  if (warp == 0) {
    if (lane == 0) {
      Fp8Tile sched(p);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && sched.next(p, m_blk, n_blk, expert)) {
        const int brow = expert * p.b_rows_per_expert + n_blk * kF8BN;
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
          mbar_expect_tx(&full[s], kF8StageBytes);
          uint8_t* a_dst = smem + s * kF8StageBytes;
          tma_load_2d(a_dst, &tmA, &full[s], kb * kF8BK, m_blk * kF8BM);
          tma_load_2d(a_dst + kF8BM * kF8BK, &tmB, &full[s], kb * kF8BK, brow);
          if (++s == kF8Stages) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) __nanosleep(200000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // kind::f8f6f4: a / b format 0 = e4m3, fp32 accumulator, both operands K-major
      constexpr uint32_t idesc = umma_idesc(0, kF8BM, kF8BN, false, false);
      Fp8Tile sched(p);
      int s = 0;
      uint32_t ph = 0, u = 0;               // u: K blocks issued so far (TMEM buffer = u % kF8AccBufs)
      bool ok = true;
      while (ok && sched.next(p, m_blk, n_blk, expert)) {
        for (int kb = 0; kb < KB; ++kb, ++u) {
          const uint32_t buf = u % kF8AccBufs;
          if (!mbar_wait_poll(&tempty[buf], ((u / kF8AccBufs) & 1) ^ 1, p.status, kTimeoutTmemEmpty)) { ok = false; break; }
          if (!mbar_wait_poll(&full[s], ph, p.status, kTimeoutFullBarrier)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * kF8StageBytes), b_addr = a_addr + kF8BM * kF8BK;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f8(tmem_base + buf * kF8BN, umma_smem_desc(a_addr + k * 32, 0, 1024),
                    umma_smem_desc(b_addr + k * 32, 0, 1024), idesc, k != 0);
          umma_commit(&empty[s]);
          umma_commit(&tfull[buf]);
          if (++s == kF8Stages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else {
    const int q = warp & 3;                    // TMEM lane quarter of this warp
    const int half = (warp - 2) >> 2;          // which 64 of the tile's 128 columns
    constexpr int kCols = kF8BN / 2;
    Fp8Tile sched(p);
    uint32_t u = 0;
    const int n_tiles_scale = (p.N + kF8BN - 1) / kF8BN;
    bool ok = true;
    while (ok && sched.next(p, m_blk, n_blk, expert)) {
      const int row = m_blk * kF8BM + q * 32 + lane;
      const bool row_ok = row < p.M && (p.row_valid == nullptr || p.row_valid[row] >= 0);
      const float* sa_row = p.sa + static_cast<long long>(row < p.M ? row : 0) * KB;
      const float* sb_row = p.sb + (static_cast<long long>(expert) * n_tiles_scale + n_blk) * KB;
      float acc[kCols];
#pragma unroll
      for (int c = 0; c < kCols; ++c) acc[c] = 0.f;
      // the scale product of the next K block is fetched while this one is promoted: two dependent global
      // loads at the head of every iteration would otherwise be the longest step of the loop
      float sc_next = sa_row[0] * sb_row[0];
      for (int kb = 0; kb < KB; ++kb, ++u) {
        const uint32_t buf = u % kF8AccBufs;
        const float sc = sc_next;
        if (kb + 1 < KB) sc_next = sa_row[kb + 1] * sb_row[kb + 1];
        ok = mbar_wait_poll(&tfull[buf], (u / kF8AccBufs) & 1, p.status, kTimeoutTmemFull);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // both TMEM loads of this warp's 64 columns are in flight before the single wait
        uint32_t v0[32], v1[32];
        const uint32_t taddr = tmem_base + buf * kF8BN + half * kCols + (static_cast<uint32_t>(q * 32) << 16);
        tmem_ld_32x32(taddr, v0);
        tmem_ld_32x32(taddr + 32, v1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[buf]);       // the values are in registers: the buffer may be reused
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          acc[j] = fmaf(__uint_as_float(v0[j]), sc, acc[j]);
          acc[32 + j] = fmaf(__uint_as_float(v1[j]), sc, acc[32 + j]);
        }
      }
      if (!ok) break;
      if (row_ok) {
        const int col_base = n_blk * kF8BN + half * kCols;
        __nv_bfloat16* dst = p.C + static_cast<long long>(row) * p.ldc + col_base;
        const bool vec = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
#pragma unroll
        for (int c = 0; c < kCols; c += 8) {
          const int col = col_base + c;
          if (vec && col + 8 <= p.N) {
            uint4 o;
            o.x = pack_bf16(acc[c], acc[c + 1]); o.y = pack_bf16(acc[c + 2], acc[c + 3]);
            o.z = pack_bf16(acc[c + 4], acc[c + 5]); o.w = pack_bf16(acc[c + 6], acc[c + 7]);
            *reinterpret_cast<uint4*>(dst + c) = o;
          } else {
            for (int j = 0; j < 8 && col + j < p.N; ++j) dst[c + j] = __float2bfloat16(acc[c + j]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kF8AccBufs * kF8BN);
}


// Activation quantiser: x bf16 [M, K] -> e4m3 [M, K] + fp32 scales [M, ceil(K / 128)] (scale =
// amax / 448 per row and 128-wide block). One warp per (row, block): lane = 4 elements.
__global__ void __launch_bounds__(256)
act_quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q,
                     float* __restrict__ scales, int M, int K, const int* __restrict__ row_valid) {
  const int KB = (K + 127) / 128;
  const long long item = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (item >= static_cast<long long>(M) * KB) return;
  const int row = static_cast<int>(item / KB), kb = static_cast<int>(item - static_cast<long long>(row) * KB);
  if (row_valid != nullptr && row_valid[row] < 0) return;      // padding row: neither read nor written
  const int lane = threadIdx.x & 31;
  const int c = kb * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (c + 4 <= K && (ldx % 4 == 0)) {
    const uint2 u = *reinterpret_cast<const uint2*>(x + static_cast<long long>(row) * ldx + c);
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    for (int j = 0; j < 4; ++j)
      if (c + j < K) v[j] = __bfloat162float(x[static_cast<long long>(row) * ldx + c + j]);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_max(amax);
  const float sc = fmaxf(amax, 1e-12f) / 448.f, inv = 1.f / sc;
  if (lane == 0) scales[static_cast<long long>(row) * KB + kb] = sc;
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3);
  const uint32_t packed = lo | (hi << 16);
  if (c + 4 <= K && (K % 4 == 0)) {
    *reinterpret_cast<uint32_t*>(q + static_cast<long long>(row) * K + c) = packed;
  } else {
    for (int j = 0; j < 4; ++j)
      if (c + j < K) q[static_cast<long long>(row) * K + c + j] = static_cast<uint8_t>((packed >> (8 * j)) & 0xff);
  }
}

}  // namespace prb

// Aq e4m3 [M, K] (pitch K), sa fp32 [M, ceil(K/128)]; Bq e4m3 [E * N, K] (E = 1 when dense),
// sb fp32 [E, ceil(N/128), ceil(K/128)]; C bf16 [M, N] (pitch ldc). K must be a multiple of 16.
// row_valid (optional, [M] int32): rows with a negative entry are not stored (padding rows of a grouped call).
PRB_API int prb_gemm_fp8(const void* Aq, const float* sa, const void* Bq, const float* sb, void* C, int M, int N, int K,
                         long long ldc, const int* block_expert, int num_experts, const int* row_valid, int* status,
                         void* stream_) {
  using namespace prb;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 16) || (reinterpret_cast<uintptr_t>(Aq) & 15) || (reinterpret_cast<uintptr_t>(Bq) & 15)) return -4;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const bool grouped = block_expert != nullptr;
  const uint64_t E = grouped ? (uint64_t)num_experts : 1;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, Aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)M, (uint64_t)K, (uint64_t)K, kF8BM, kF8BK,
                        true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, Bq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, E * (uint64_t)N, (uint64_t)K, (uint64_t)K, kF8BN, kF8BK,
                    true);
  if (rc) return rc;
  Fp8Params p;
  p.M = M; p.N = N; p.K = K; p.sa = sa; p.sb = sb;
  p.C = reinterpret_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.block_expert = block_expert; p.b_rows_per_expert = grouped ? N : 0; p.row_valid = row_valid; p.status = status;
  static prb::DeviceOnce configured;
  if (configured.pending()) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kF8Smem) != cudaSuccess)
      return -10;
    configured.mark();
  }
  const int tiles = ((M + kF8BM - 1) / kF8BM) * ((N + kF8BN - 1) / kF8BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_fp8_kernel<<<grid, kF8Threads, kF8Smem, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// row_valid (optional, [M] int32): rows with a negative entry are skipped.
PRB_API int prb_act_quant_fp8(const void* x, long long ldx, void* q, float* scales, int M, int K, const int* row_valid,
                              void* stream) {
  if (M <= 0 || K <= 0) return 0;
  const long long items = static_cast<long long>(M) * ((K + 127) / 128);
  prb::act_quant_fp8_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<uint8_t*>(q), scales, M, K, row_valid);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
