// bf16 GEMM for sm_100a: persistent, warp-specialised, TMA -> shared memory (128B swizzle)
// -> tcgen05.mma (cta_group::1, M=128) -> TMEM accumulators (double buffered) -> epilogue.
//
//   C[M,N] = alpha * A . B + beta * C      (fp32 accumulate, C bf16 or fp32)
//
// Operand layouts (both given as row-major 2-D tensors):
//   A K-major : A[M,K]      A MN-major: A[K,M]   (i.e. A^T is what is stored)
//   B K-major : B[N,K]      B MN-major: B[K,N]
// so that  x @ W^T (nn.Linear forward) = (A K-major, B K-major),
//          dY @ W  (dgrad)             = (A K-major, B MN-major),
//          dY^T @ X (wgrad)            = (A MN-major, B MN-major).
//
// Grouped (MoE) mode: rows of A / C are 128-row blocks that each belong to one expert
// (`block_expert[blk]`, -1 = unused block; unused blocks come after all used ones); B is the stacked per-expert weight viewed as a
// 2-D tensor with `b_rows_per_expert` rows per expert. No host synchronisation is needed:
// the grid covers the static upper bound of blocks and unused blocks are skipped.
//
// Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 =
// epilogue (one TMEM lane quarter each). All waits are bounded (see common.cuh).
//
// Replaces nn.Linear / cuBLAS and torch._grouped_mm in the reference
// (src/prime_rl/trainer/models/layers/grouped_gemm.py:21-31, layers/moe.py:124-164).
#include "common.cuh"
#include "tma_host.cuh"
#include <type_traits>

namespace prb {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;

struct GemmParams {
  int M, N, K;
  long long rows_total;  // rows of C (M, or num_experts * M when K-grouped)
  void* C;
  long long ldc;
  int out_fp32;
  float alpha, beta;
  const int* block_expert;  // nullptr = dense
  int b_rows_per_expert;
  int* status;
  // optional extra reduction segment (fused low-rank term): after the K blocks of (A, B) the
  // same accumulator takes k2_blocks more blocks from a second operand pair (A2 [M, K2],
  // B2 laid out like B with b2_rows_per_expert rows per expert); K2 need not be a multiple of
  // 64, TMA zero-fills A2 past K2
  int k2_blocks = 0;
  int b2_rows_per_expert = 0;
  // optional: rows r of C with row_valid[r] < 0 are not stored (padding rows of a grouped inference GEMM)
  const int* row_valid = nullptr;
  // reduce-scatter epilogue: row r of C is added into peer_c[r / rows_per_rank] (fp32, pitch ldc)
  float* peer_c[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int rows_per_rank = 0;
  // all-gather prologue: B [N, K] lives in a buffer that every rank holds in full but of which
  // only the rows [r * ag_rows, (r + 1) * ag_rows) are valid on rank r. Gather warps copy the
  // other ranks' rows (ag_src[r] = rank r's buffer base) into the local buffer in pieces and
  // count finished pieces per N block in ag_ready; the producer loads a remote N block once
  // its count reaches ag_target (counters only grow: target = call number * pieces per block).
  const uint8_t* ag_src[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  uint8_t* ag_dst = nullptr;
  unsigned* ag_ready = nullptr;
  unsigned ag_target = 0;
  int ag_rank = 0, ag_ranks = 1, ag_rows = 0;
  long long ag_row_bytes = 0;
  // grouped mode fed by a peer-memory dispatch: rows of M block b are complete once blk_arrive[b] (bumped by the
  // senders with release-adds at system scope) has reached blk_rows[b]; the producer waits per block (bounded)
  const unsigned* blk_arrive = nullptr;
  const int* blk_rows = nullptr;
  // split-K (decode-sized dense GEMMs): the K blocks of one output tile are dealt to sk_splits CTAs, split ks
  // stores its fp32 partial tile to rows [ks * M, (ks + 1) * M) of a workspace (C points there) and a second
  // kernel adds the partials in split order
  int sk_splits = 1;
  const int* expert_offset;  // K-grouped mode
  int num_experts;
  // fused LM head (logprob / entropy) extras
  int num_splits;
  const int* labels;
  const float* inv_temp;
  float* part_m;
  float* part_s;
  float* part_t;
  float* target_logit;
  const float* grad_logprob;
  const float* lse;
};

// Width in columns of one vocabulary split (the unit `end_item` indexes partials by).
__device__ __forceinline__ int sched_split_width(const GemmParams& p, int bn) {
  if (p.num_splits <= 0) return 1 << 30;
  const int tiles_n = (p.N + bn - 1) / bn;
  return ((tiles_n + p.num_splits - 1) / p.num_splits) * bn;
}

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = kBM * kBK * 2;
  static constexpr int B_BYTES = BN * kBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int ACC_COLS = 2 * BN;  // two accumulator buffers; 512 / 256 / 128 columns
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

// ---------------------------------------------------------------- tile schedulers
// A scheduler enumerates the (m_blk, n_blk) tiles of one CTA; all three warp roles run the
// same enumeration so that their pipelines stay in step.
struct SchedDense {
  static constexpr int kGatherWarps = 0;
  int tile, num_tiles, tiles_m, tiles_n;
  int group_first = 0;                 // first M block of the raster group of the current tile
  __device__ SchedDense(const GemmParams& p, int bn)
      : tile(blockIdx.x - gridDim.x), tiles_m((p.M + kBM - 1) / kBM), tiles_n((p.N + bn - 1) / bn) {
    num_tiles = tiles_m * tiles_n;
  }
  // Grouped raster: 8 consecutive M blocks share their B tiles in L2.
  __device__ bool next(const GemmParams& p, int& m_blk, int& n_blk, int& brow, bool& last_of_item, int& kb0,
                       int& nkb, long long& c_row0) {
    kb0 = 0;
    nkb = (p.K + kBK - 1) / kBK;
    c_row0 = 0;
    tile += gridDim.x;
    if (tile >= num_tiles) return false;
    constexpr int kGroup = 8;
    const int per_group = kGroup * tiles_n;
    const int g = tile / per_group;
    const int first_m = g * kGroup;
    group_first = first_m;
    const int gsize = min(tiles_m - first_m, kGroup);
    const int r = tile - g * per_group;
    m_blk = first_m + (r % gsize);
    n_blk = r / gsize;
    brow = 0;
    last_of_item = true;
    return true;
  }
};

struct SchedGrouped : SchedDense {
  __device__ SchedGrouped(const GemmParams& p, int bn) : SchedDense(p, bn) {}
  __device__ bool next(const GemmParams& p, int& m_blk, int& n_blk, int& brow, bool& last_of_item, int& kb0,
                       int& nkb, long long& c_row0) {
    while (SchedDense::next(p, m_blk, n_blk, brow, last_of_item, kb0, nkb, c_row0)) {
      const int e = p.block_expert[m_blk];
      if (e >= 0) {
        brow = e * p.b_rows_per_expert;
        return true;
      }
      // used blocks are a prefix of the row space (the grid covers a static upper bound): when the first block of
      // a raster group is unused, so is everything after it
      if (m_blk == group_first) return false;
    }
    return false;
  }
};

// Split-K: tile = (m_blk, n_blk, k split); split ks writes to rows ks * M .. of the workspace (c_row0). Every
// split owns at least one K block (the host sees to it).
struct SchedSplitK {
  static constexpr int kGatherWarps = 0;
  int tile, num_tiles, tiles_m, tiles_n, nkb_total, per;
  __device__ SchedSplitK(const GemmParams& p, int bn)
      : tile(blockIdx.x - gridDim.x), tiles_m((p.M + kBM - 1) / kBM), tiles_n((p.N + bn - 1) / bn),
        nkb_total((p.K + kBK - 1) / kBK) {
    per = (nkb_total + p.sk_splits - 1) / p.sk_splits;
    num_tiles = tiles_m * tiles_n * p.sk_splits;
  }
  __device__ bool next(const GemmParams& p, int& m_blk, int& n_blk, int& brow, bool& last_of_item, int& kb0,
                       int& nkb, long long& c_row0) {
    tile += gridDim.x;
    if (tile >= num_tiles) return false;
    const int mn = tile / p.sk_splits;
    const int ks = tile - mn * p.sk_splits;
    m_blk = mn % tiles_m;
    n_blk = mn / tiles_m;
    kb0 = ks * per;
    nkb = min(per, nkb_total - kb0);
    c_row0 = static_cast<long long>(ks) * p.M;
    brow = 0;
    last_of_item = true;
    return true;
  }
};

// Split order for the fused LM head: an item is (split, m_blk) and covers the N tiles
// [split * per_split, (split + 1) * per_split); consecutive tiles of a CTA stay on one
// M block so that per-row running statistics can live in registers. Items are numbered
// split-major so that the CTAs in flight stream the same slice of the vocabulary.
struct SchedSplit {
  static constexpr int kGatherWarps = 0;
  int item, j, tiles_m, tiles_n, per_split, num_items;
  __device__ SchedSplit(const GemmParams& p, int bn)
      : item(blockIdx.x - gridDim.x), j(0x7fffffff), tiles_m((p.M + kBM - 1) / kBM),
        tiles_n((p.N + bn - 1) / bn) {
    per_split = (tiles_n + p.num_splits - 1) / p.num_splits;
    num_items = tiles_m * p.num_splits;
  }
  __device__ bool next(const GemmParams& p, int& m_blk, int& n_blk, int& brow, bool& last_of_item, int& kb0,
                       int& nkb, long long& c_row0) {
    kb0 = 0;
    nkb = (p.K + kBK - 1) / kBK;
    c_row0 = 0;
    for (;;) {
      if (j >= per_split) {
        item += gridDim.x;
        j = 0;
        if (item >= num_items) return false;
      }
      const int split = item / tiles_m;
      m_blk = item - split * tiles_m;
      n_blk = split * per_split + j;
      ++j;
      if (n_blk < tiles_n) {
        brow = 0;
        last_of_item = (j >= per_split) || (n_blk + 1 >= tiles_n);
        if (last_of_item) j = per_split;
        return true;
      }
      j = per_split;  // rest of this split is empty
    }
  }
};

// K-grouped (per-expert weight gradient): tile = (expert, m_blk, n_blk); the reduction runs
// over the expert's 128-aligned row range [expert_offset[e], expert_offset[e+1]) of the
// MN-major operands and the result goes to rows [e*M, (e+1)*M) of the stacked output.
// Experts without rows produce nkb = 0: producer and MMA skip the tile, the epilogue
// writes zeros.
struct SchedKGrouped {
  static constexpr int kGatherWarps = 0;
  int tile, num_tiles, tiles_m, tiles_n;
  __device__ SchedKGrouped(const GemmParams& p, int bn)
      : tile(blockIdx.x - gridDim.x), tiles_m((p.M + kBM - 1) / kBM), tiles_n((p.N + bn - 1) / bn) {
    num_tiles = tiles_m * tiles_n * p.num_experts;
  }
  __device__ bool next(const GemmParams& p, int& m_blk, int& n_blk, int& brow, bool& last_of_item, int& kb0,
                       int& nkb, long long& c_row0) {
    tile += gridDim.x;
    if (tile >= num_tiles) return false;
    const int per_e = tiles_m * tiles_n;
    const int e = tile / per_e;
    const int r = tile - e * per_e;
    m_blk = r % tiles_m;
    n_blk = r / tiles_m;
    brow = 0;
    last_of_item = true;
    const int r0 = p.expert_offset[e], r1 = p.expert_offset[e + 1];
    kb0 = r0 / kBK;
    nkb = (r1 - r0) / kBK;
    c_row0 = static_cast<long long>(e) * p.M;
    return true;
  }
};

// All-gather order: N-major (all M blocks of one N block are consecutive, so the CTAs in flight
// share one B tile) and rotated so that the N blocks of this rank's own rows come first, then
// those of rank+1, rank+2, ...; the gather warps fetch remote rows in the same order.
constexpr int kAgPieceBytes = 16384;
struct SchedAllGather {
  static constexpr int kGatherWarps = 2;
  int tile, num_tiles, tiles_m, tiles_n, first_n;
  __device__ SchedAllGather(const GemmParams& p, int bn)
      : tile(blockIdx.x - gridDim.x), tiles_m((p.M + kBM - 1) / kBM), tiles_n((p.N + bn - 1) / bn) {
    num_tiles = tiles_m * tiles_n;
    first_n = p.ag_rank * (p.ag_rows / bn);
  }
  __device__ bool next(const GemmParams& p, int& m_blk, int& n_blk, int& brow, bool& last_of_item, int& kb0,
                       int& nkb, long long& c_row0) {
    kb0 = 0;
    nkb = (p.K + kBK - 1) / kBK;
    c_row0 = 0;
    tile += gridDim.x;
    if (tile >= num_tiles) return false;
    const int n_idx = tile / tiles_m;
    m_blk = tile - n_idx * tiles_m;
    n_blk = n_idx + first_n;
    if (n_blk >= tiles_n) n_blk -= tiles_n;
    brow = 0;
    last_of_item = true;
    return true;
  }
};

// Gather warps of one CTA: pieces of kAgPieceBytes, numbered in schedule order over the remote
// N blocks, are dealt round-robin to the CTAs. `bn` rows of `ag_row_bytes` make one N block.
__device__ void ag_gather(const GemmParams& p, int bn, int tid, int nthreads) {
  const int blocks_per_rank = p.ag_rows / bn;
  const int tiles_n = p.ag_ranks * blocks_per_rank;
  const long long block_bytes = static_cast<long long>(bn) * p.ag_row_bytes;
  const int ppb = static_cast<int>((block_bytes + kAgPieceBytes - 1) / kAgPieceBytes);
  const long long remote_pieces = static_cast<long long>(tiles_n - blocks_per_rank) * ppb;
  for (long long g = blockIdx.x; g < remote_pieces; g += gridDim.x) {
    const int n_idx = blocks_per_rank + static_cast<int>(g / ppb);
    const int piece = static_cast<int>(g % ppb);
    int n_blk = n_idx + p.ag_rank * blocks_per_rank;
    if (n_blk >= tiles_n) n_blk -= tiles_n;
    const int owner = n_blk / blocks_per_rank;
    const long long off = static_cast<long long>(n_blk) * block_bytes + static_cast<long long>(piece) * kAgPieceBytes;
    const long long len = min(static_cast<long long>(kAgPieceBytes), block_bytes - static_cast<long long>(piece) * kAgPieceBytes);
    const int4* src = reinterpret_cast<const int4*>(p.ag_src[owner] + off);
    int4* dst = reinterpret_cast<int4*>(p.ag_dst + off);
    const int n16 = static_cast<int>(len >> 4);
    for (int i = tid; i < n16; i += nthreads * 4) {
      int4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u * nthreads < n16) v[u] = __ldcg(src + i + u * nthreads);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u * nthreads < n16) dst[i + u * nthreads] = v[u];
    }
    __threadfence();
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    if (tid == 0) atomicAdd(p.ag_ready + n_blk, 1u);
  }
}

// Producer side: wait (bounded) until every piece of N block n_blk has landed.
__device__ bool ag_wait_block(const GemmParams& p, int bn, int n_blk) {
  const int blocks_per_rank = p.ag_rows / bn;
  if (n_blk / blocks_per_rank == p.ag_rank) return true;
  const long long block_bytes = static_cast<long long>(bn) * p.ag_row_bytes;
  const unsigned ppb = static_cast<unsigned>((block_bytes + kAgPieceBytes - 1) / kAgPieceBytes);
  const unsigned want = p.ag_target * ppb;
  const unsigned* flag = p.ag_ready + n_blk;
  for (long long spin = 0; spin < (1LL << 24); ++spin) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= want) {
      asm volatile("fence.proxy.async;" ::: "memory");
      return true;
    }
    __nanosleep(64);
  }
  if (p.status) atomicCAS(p.status, 0, kTimeoutPeerFlag);
  return false;
}

// Producer side of a GEMM whose A rows are being written by other GPUs: wait (bounded) until every row of M block
// m_blk has landed, then order the async-proxy reads (TMA) after the generic-proxy writes.
__device__ bool blk_wait(const GemmParams& p, int m_blk) {
  const unsigned want = static_cast<unsigned>(p.blk_rows[m_blk]);
  const unsigned* flag = p.blk_arrive + m_blk;
  const long long t0 = clock64();
  for (unsigned spin = 0;; ++spin) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= want) {
      asm volatile("fence.proxy.async;" ::: "memory");
      return true;
    }
    if ((spin & 0xff) == 0xff) {
      if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) return false;
      if (clock64() - t0 > 4000000000LL) break;   // about 2 s
    }
    __nanosleep(64);
  }
  if (p.status) atomicCAS(p.status, 0, kTimeoutPeerFlag);
  return false;
}

// ---------------------------------------------------------------- epilogues
// An epilogue consumes 32-column chunks of one accumulator row per thread.
struct EpiStore {
  __device__ EpiStore(const GemmParams&) {}
  __device__ void begin_item(const GemmParams&, long long) {}
  __device__ void end_item(const GemmParams&, long long, int) {}
  __device__ void chunk(const GemmParams& p, long long row, int col0, uint32_t (&v)[32]) {
    if (row >= p.rows_total || col0 >= p.N) return;
    const bool base_ok = (reinterpret_cast<uintptr_t>(p.C) & 15) == 0;
    if (p.out_fp32) {
      float* dst = reinterpret_cast<float*>(p.C) + row * p.ldc + col0;
      if (col0 + 32 <= p.N && (p.ldc % 4 == 0) && base_ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 o;
          o.x = p.alpha * __uint_as_float(v[4 * j + 0]);
          o.y = p.alpha * __uint_as_float(v[4 * j + 1]);
          o.z = p.alpha * __uint_as_float(v[4 * j + 2]);
          o.w = p.alpha * __uint_as_float(v[4 * j + 3]);
          if (p.beta != 0.f) {
            const float4 old = *reinterpret_cast<const float4*>(dst + 4 * j);
            o.x += p.beta * old.x; o.y += p.beta * old.y; o.z += p.beta * old.z; o.w += p.beta * old.w;
          }
          *reinterpret_cast<float4*>(dst + 4 * j) = o;
        }
      } else {
        for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
          float o = p.alpha * __uint_as_float(v[j]);
          if (p.beta != 0.f) o += p.beta * dst[j];
          dst[j] = o;
        }
      }
    } else {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
      if (col0 + 32 <= p.N && (p.ldc % 8 == 0) && base_ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float f[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) f[t] = p.alpha * __uint_as_float(v[8 * j + t]);
          if (p.beta != 0.f) {
            const uint4 old = *reinterpret_cast<const uint4*>(dst + 8 * j);
            const float2 o0 = unpack_bf16(old.x), o1 = unpack_bf16(old.y), o2 = unpack_bf16(old.z),
                         o3 = unpack_bf16(old.w);
            f[0] += p.beta * o0.x; f[1] += p.beta * o0.y; f[2] += p.beta * o1.x; f[3] += p.beta * o1.y;
            f[4] += p.beta * o2.x; f[5] += p.beta * o2.y; f[6] += p.beta * o3.x; f[7] += p.beta * o3.y;
          }
          uint4 o;
          o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
          o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
          *reinterpret_cast<uint4*>(dst + 8 * j) = o;
        }
      } else {
        for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
          float o = p.alpha * __uint_as_float(v[j]);
          if (p.beta != 0.f) o += p.beta * __bfloat162float(dst[j]);
          dst[j] = __float2bfloat16(o);
        }
      }
    }
  }
};

// fp32 accumulation into C (weight gradients: C += alpha * A.B) without reading C: every epilogue warp stages its
// 32 x 32 fp32 chunk in shared memory (128-byte swizzle, two buffers per warp) and hands it to the TMA unit as a
// reduce-add, which the L2 applies. Against the load / add / store form of EpiStore this halves the bytes the
// SM moves and makes them full 128-byte lines. The work happens in the kernel body (it needs the warp and the
// tensor map); tmA2 carries the map of C. Needs beta = 1, fp32 C, N and ldc multiples of 4.
struct EpiTmaReduce {
  static constexpr bool kTmaReduce = true;
  __device__ EpiTmaReduce(const GemmParams&) {}
  __device__ void begin_item(const GemmParams&, long long) {}
  __device__ void end_item(const GemmParams&, long long, int) {}
  __device__ void chunk(const GemmParams&, long long, int, uint32_t (&)[32]) {}
};
constexpr int kRedStageBytes = 4 * 2 * 4096;      // 4 epilogue warps x 2 buffers x (32 rows x 128 bytes)
template <class E, class = void>
struct epi_is_tma_reduce : std::false_type {};
template <class E>
struct epi_is_tma_reduce<E, std::void_t<decltype(E::kTmaReduce)>> : std::true_type {};

// GEMM -> reduce-scatter in one kernel: the fp32 tile leaves TMEM as vector reductions into the
// row owner's shard (peer memory over NVLink, or this GPU's own shard), so the transfer of a
// tile overlaps the tensor-core work of the next one and no partial result is materialised.
// The shards must be zero (or hold the running sum) before any rank starts.
struct EpiPeerReduce {
  __device__ EpiPeerReduce(const GemmParams&) {}
  __device__ void begin_item(const GemmParams&, long long) {}
  __device__ void end_item(const GemmParams&, long long, int) {}
  __device__ void chunk(const GemmParams& p, long long row, int col0, uint32_t (&v)[32]) {
    if (row >= p.rows_total || col0 >= p.N) return;
    const int owner = static_cast<int>(row / p.rows_per_rank);
    float* dst = p.peer_c[owner] + (row - static_cast<long long>(owner) * p.rows_per_rank) * p.ldc + col0;
    if (col0 + 32 <= p.N && (p.ldc % 4 == 0)) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * j),
                     "f"(p.alpha * __uint_as_float(v[4 * j + 0])), "f"(p.alpha * __uint_as_float(v[4 * j + 1])),
                     "f"(p.alpha * __uint_as_float(v[4 * j + 2])), "f"(p.alpha * __uint_as_float(v[4 * j + 3]))
                     : "memory");
    } else {
      for (int j = 0; j < 32 && col0 + j < p.N; ++j)
        asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(dst + j), "f"(p.alpha * __uint_as_float(v[j]))
                     : "memory");
    }
  }
};

// Fused LM head, forward: per row running (max, sum exp, sum exp * z) over the vocabulary
// slice of this item plus the target logit; z = logit * inv_temp[row].
struct EpiLogprobStats {
  float m, s, t, it;
  int label;
  __device__ EpiLogprobStats(const GemmParams&) : m(-INFINITY), s(0.f), t(0.f), it(1.f), label(-1) {}
  __device__ void begin_item(const GemmParams& p, long long row) {
    m = -INFINITY; s = 0.f; t = 0.f;
    const bool ok = row < p.M;
    it = (ok && p.inv_temp) ? p.inv_temp[row] : 1.f;
    label = ok ? p.labels[row] : -1;
  }
  __device__ void chunk(const GemmParams& p, long long row, int col0, uint32_t (&v)[32]) {
    if (col0 >= p.N) return;
    float z[32];
    float cm = -INFINITY;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      z[j] = (col0 + j < p.N) ? __uint_as_float(v[j]) * it : -INFINITY;
      cm = fmaxf(cm, z[j]);
    }
    if (label >= col0 && label < col0 + 32 && row < p.M) {
      float zl = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) zl = (col0 + j == label) ? z[j] : zl;
      p.target_logit[row] = zl;
    }
    const float mn = fmaxf(m, cm);
    const float corr = __expf(m - mn);  // m = -inf on the first chunk -> 0
    float ls = 0.f, lt = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float e = __expf(z[j] - mn);  // -inf -> 0
      ls += e;
      lt += (col0 + j < p.N) ? e * z[j] : 0.f;
    }
    s = s * corr + ls;
    t = t * corr + lt;
    m = mn;
  }
  __device__ void end_item(const GemmParams& p, long long row, int split) {
    if (row >= p.M) return;
    const long long o = static_cast<long long>(split) * p.M + row;
    p.part_m[o] = m;
    p.part_s[o] = s;
    p.part_t[o] = t;
  }
};

// Fused LM head, backward: dlogits = g[row] * inv_temp[row] * (onehot(label) - softmax(z)),
// written as bf16 [M, N] (C). softmax is rebuilt from the saved log-sum-exp.
struct EpiDLogits {
  float it, g, lse;
  int label;
  __device__ EpiDLogits(const GemmParams&) : it(1.f), g(0.f), lse(0.f), label(-1) {}
  __device__ void begin_item(const GemmParams& p, long long row) {
    const bool ok = row < p.M;
    it = (ok && p.inv_temp) ? p.inv_temp[row] : 1.f;
    lse = ok ? p.lse[row] : 0.f;
    label = ok ? p.labels[row] : -1;
    // an ignored label makes the log-probability a constant 0: no gradient for that row
    g = (ok && label >= 0 && label < p.N) ? p.grad_logprob[row] : 0.f;
  }
  __device__ void end_item(const GemmParams&, long long, int) {}
  __device__ void chunk(const GemmParams& p, long long row, int col0, uint32_t (&v)[32]) {
    if (row >= p.M || col0 >= p.N) return;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col0;
    float d[32];
    const float gs = g * it;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float z = __uint_as_float(v[j]) * it;
      const float pr = __expf(z - lse);
      d[j] = gs * (((col0 + j) == label ? 1.f : 0.f) - pr);
    }
    if (col0 + 32 <= p.N && (p.ldc % 8 == 0)) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 o;
        o.x = pack_bf16(d[8 * j + 0], d[8 * j + 1]); o.y = pack_bf16(d[8 * j + 2], d[8 * j + 3]);
        o.z = pack_bf16(d[8 * j + 4], d[8 * j + 5]); o.w = pack_bf16(d[8 * j + 6], d[8 * j + 7]);
        *reinterpret_cast<uint4*>(dst + 8 * j) = o;
      }
    } else {
      for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = __float2bfloat16(d[j]);
    }
  }
};

template <int BN, bool A_MN, bool B_MN, class Sched, class Epi>
__global__ void __launch_bounds__(kGemmThreads + 32 * Sched::kGatherWarps, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                 const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (p.k2_blocks > 0) {
      tma_prefetch_desc(&tmA2);
      tma_prefetch_desc(&tmB2);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::ACC_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  int m_blk = 0, n_blk = 0, brow = 0, kb0 = 0, nkb = 0;
  long long c_row0 = 0;
  bool last = true;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      Sched sched(p, BN);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && sched.next(p, m_blk, n_blk, brow, last, kb0, nkb, c_row0)) {
        const int nk_total = nkb > 0 ? nkb + p.k2_blocks : 0;
        for (int it = 0; it < nk_total; ++it) {
          const bool ext = it >= nkb;                 // block of the extra (A2, B2) segment
          const int kb = ext ? it - nkb : kb0 + it;
          const CUtensorMap* ma = ext ? &tmA2 : &tmA;
          const CUtensorMap* mb = ext ? &tmB2 : &tmB;
          const int brow_k = (ext && p.b_rows_per_expert > 0) ? (brow / p.b_rows_per_expert) * p.b2_rows_per_expert
                                                              : brow;
          if (!mbar_wait(&empty[s], ph ^ 1, p.status, kTimeoutEmptyBarrier)) {
            ok = false;
            break;
          }
          if constexpr (Sched::kGatherWarps > 0) {
            if (it == 0 && !ag_wait_block(p, BN, n_blk)) {
              ok = false;
              break;
            }
          }
          if constexpr (std::is_same<Sched, SchedGrouped>::value) {
            if (it == 0 && p.blk_arrive != nullptr && !blk_wait(p, m_blk)) {
              ok = false;
              break;
            }
          }
          mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
          uint8_t* a_dst = smem + s * Cfg::STAGE_BYTES;
          uint8_t* b_dst = a_dst + Cfg::A_BYTES;
          if (!A_MN) {
            tma_load_2d(a_dst, ma, &full[s], kb * kBK, m_blk * kBM);
          } else {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)
              tma_load_2d(a_dst + j * 8192, ma, &full[s], m_blk * kBM + 64 * j, kb * kBK);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, mb, &full[s], kb * kBK, brow_k + n_blk * BN);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * 8192, mb, &full[s], n_blk * BN + 64 * j, brow_k + kb * kBK);
          }
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
      if (!ok) __nanosleep(200000);  // let copies that are still in flight land before exit
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(1, kBM, BN, A_MN, B_MN);
      Sched sched(p, BN);
      int s = 0, acc = 0;
      uint32_t ph = 0, acc_ph = 0;
      bool ok = true;
      while (ok && sched.next(p, m_blk, n_blk, brow, last, kb0, nkb, c_row0)) {
        if (nkb == 0) continue;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, p.status, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int nk_total = nkb + p.k2_blocks;
        for (int kb = 0; kb < nk_total; ++kb) {
          if (!mbar_wait(&full[s], ph, p.status, kTimeoutFullBarrier)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t adesc =
                A_MN ? umma_smem_desc(a_addr + k * 2048, 8192, 1024) : umma_smem_desc(a_addr + k * 32, 0, 1024);
            const uint64_t bdesc =
                B_MN ? umma_smem_desc(b_addr + k * 2048, 8192, 1024) : umma_smem_desc(b_addr + k * 32, 0, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0);
          }
          umma_commit(&empty[s]);
          if (++s == STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_ph ^= 1;
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------ gather warps (all-gather variant)
    if constexpr (Sched::kGatherWarps > 0)
      ag_gather(p, BN, threadIdx.x - kGemmThreads, 32 * Sched::kGatherWarps);
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lanes [32q, 32q+32) are the ones this warp may read
    Sched sched(p, BN);
    Epi epi(p);
    int acc = 0;
    uint32_t acc_ph = 0;
    bool first = true;
    [[maybe_unused]] uint32_t red_seq = 0;           // chunks this warp has handed to the TMA unit (EpiTmaReduce)
    while (sched.next(p, m_blk, n_blk, brow, last, kb0, nkb, c_row0)) {
      const int row_in_m = m_blk * kBM + q * 32 + lane;
      long long row = (row_in_m < p.M) ? c_row0 + row_in_m : (1LL << 40);  // out of range -> masked
      if (p.row_valid != nullptr && row < p.rows_total && p.row_valid[row] < 0) row = 1LL << 40;
      if constexpr (epi_is_tma_reduce<Epi>::value) {
        if (nkb == 0) continue;                      // C += 0
      }
      if (nkb == 0) {
        // nothing to reduce: the tile is all zeros
        uint32_t z[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) z[j] = 0u;
        for (int c = 0; c < BN / 32; ++c) epi.chunk(p, row, n_blk * BN + c * 32, z);
        continue;
      }
      if (first) epi.begin_item(p, row);
      bool ok = mbar_wait(&tfull[acc], acc_ph, p.status, kTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if constexpr (epi_is_tma_reduce<Epi>::value) {
        uint8_t* my_stage = smem + STAGES * Cfg::STAGE_BYTES + 1024 + q * 8192;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c, ++red_seq) {
          if (n_blk * BN + c * 32 >= p.N) break;
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
          tmem_ld_wait();
          uint8_t* sb = my_stage + (red_seq & 1) * 4096;
          if (red_seq >= 2) {                         // the reduce that last read this buffer (two chunks ago) is done
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(sb + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_float4(p.alpha * __uint_as_float(v[4 * j]), p.alpha * __uint_as_float(v[4 * j + 1]),
                            p.alpha * __uint_as_float(v[4 * j + 2]), p.alpha * __uint_as_float(v[4 * j + 3]));
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_reduce_add_2d(&tmA2, sb, n_blk * BN + c * 32, static_cast<int>(c_row0) + m_blk * kBM + q * 32);
            tma_store_commit();
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
        tmem_ld_wait();
        epi.chunk(p, row, n_blk * BN + c * 32, v);
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_ph ^= 1;
      if (last) epi.end_item(p, row, (n_blk * BN) / (sched_split_width(p, BN)));
      first = last;
    }
    if constexpr (epi_is_tma_reduce<Epi>::value) {
      if (lane == 0) tma_store_wait<0>();             // shared memory must outlive the reduces that read it
      __syncwarp();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::ACC_COLS);
}

template <int BN, bool A_MN, bool B_MN, bool GROUPED>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmA2,
                       const CUtensorMap& tmB2, const GemmParams& p, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  using Sched = typename std::conditional<GROUPED, SchedGrouped, SchedDense>::type;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, Sched, EpiStore>;
  static prb::DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return -10;
    configured.mark();
  }
  const int tiles = ((p.M + kBM - 1) / kBM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  if (grid <= 0) return 0;
  kern<<<grid, kGemmThreads, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, tmA2, tmB2, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Dense weight gradient C += alpha * A^T.B (both operands MN-major) into an fp32 accumulator through TMA
// reduce-adds (EpiTmaReduce); tmC rides in the tmA2 slot.
template <int BN>
static int launch_gemm_reduce(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                              const GemmParams& p, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  constexpr int kSmem = Cfg::SMEM_BYTES + 768 + kRedStageBytes;
  auto kern = gemm_bf16_kernel<BN, true, true, SchedDense, EpiTmaReduce>;
  static prb::DeviceOnce configured;
  if (configured.pending()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return -10;
    configured.mark();
  }
  const int tiles = ((p.M + kBM - 1) / kBM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  if (grid <= 0) return 0;
  kern<<<grid, kGemmThreads, kSmem, stream>>>(tmA, tmB, tmC, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

template <int BN, bool B_MN>
static int launch_gemm_splitk(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                              cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_kernel<BN, false, B_MN, SchedSplitK, EpiStore>;
  static prb::DeviceOnce configured;
  if (configured.pending()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return -10;
    configured.mark();
  }
  const int items = ((p.M + kBM - 1) / kBM) * ((p.N + BN - 1) / BN) * p.sk_splits;
  const int grid = items < sm_count() ? items : sm_count();
  kern<<<grid, kGemmThreads, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Adds the split-K partials in split order and applies the GEMM's alpha / beta / output type:
// C[m, n] = alpha * sum_s ws[s][m][n] + beta * C[m, n]. One float4 of a workspace row per thread and step.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, int splits, int M, int N, void* __restrict__ C, long long ldc,
                     int out_fp32, float alpha, float beta) {
  const int n4 = N / 4;
  const long long total = static_cast<long long>(M) * n4;
  const long long plane = static_cast<long long>(M) * N;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / n4;
    const int col = static_cast<int>(i - row * n4) * 4;
    const float* src = ws + row * N + col;
    float4 acc = __ldcg(reinterpret_cast<const float4*>(src));
    for (int s2 = 1; s2 < splits; ++s2) {
      const float4 t = __ldcg(reinterpret_cast<const float4*>(src + s2 * plane));
      acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    }
    float o[4] = {alpha * acc.x, alpha * acc.y, alpha * acc.z, alpha * acc.w};
    if (out_fp32) {
      float* dst = reinterpret_cast<float*>(C) + row * ldc + col;
#pragma unroll
      for (int j = 0; j < 4; ++j) dst[j] = (beta != 0.f) ? o[j] + beta * dst[j] : o[j];
    } else {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(C) + row * ldc + col;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        dst[j] = __float2bfloat16((beta != 0.f) ? o[j] + beta * __bfloat162float(dst[j]) : o[j]);
    }
  }
}

// Tile width and K split for a dense GEMM with few output tiles. Every CTA streams its operand slabs through
// its own SM's L2 port (about 80 GB/s), so: time = fixed + waves x slab bytes of one work item / that rate, plus,
// when split, the second kernel that adds the partials. Returns splits (1 = no split) and sets bn. N % 4 == 0
// is needed for a split (the partials are read as float4).
struct SplitKWorkspace {
  float* ws;
  long long ws_bytes;
  int force_splits;
};
static int choose_splitk(int M, int N, int K, int force_bn, const SplitKWorkspace& w, int& bn_out) {
  const int sms = sm_count();
  const int nkb = (K + kBK - 1) / kBK;
  const long long tiles_m = (M + kBM - 1) / kBM;
  double best = 1e30;
  int best_bn = bn_out, best_s = 1;
  const int bns[3] = {256, 128, 64};
  for (int bi = 0; bi < 3; ++bi) {
    const int bn = bns[bi];
    if (force_bn > 0 && bn != force_bn) continue;
    if (bn > 64 && bn / 2 >= N) continue;               // a tile twice as wide as the output
    const long long tiles = tiles_m * ((N + bn - 1) / bn);
    for (int s = 1; s <= 8; ++s) {
      if (w.force_splits > 0 && s != w.force_splits) continue;
      const int per = (nkb + s - 1) / s;
      if (s > 1 && (per < 2 || (nkb + per - 1) / per != s)) continue;     // no empty split
      if (s > 1 && ((N % 4) || static_cast<long long>(s) * M * N * 4 > w.ws_bytes)) continue;
      const long long waves = (tiles * s + sms - 1) / sms;
      double t = 3.0 + waves * per * (kBM + bn) * kBK * 2.0 / 80e3;
      if (s > 1) t += 6.0 + (s + 1.0) * M * N * 4.0 / 3e6;                // second launch + its traffic at 3 TB/s
      if (t < best) {
        best = t;
        best_bn = bn;
        best_s = s;
      }
    }
  }
  bn_out = best_bn;
  return best_s;
}

template <bool A_MN, bool B_MN, bool GROUPED>
static int dispatch_bn(int bn, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmA2,
                       const CUtensorMap& tmB2, const GemmParams& p, cudaStream_t stream) {
  switch (bn) {
    case 256: return launch_gemm<256, A_MN, B_MN, GROUPED>(tmA, tmB, tmA2, tmB2, p, stream);
    case 128: return launch_gemm<128, A_MN, B_MN, GROUPED>(tmA, tmB, tmA2, tmB2, p, stream);
    default: return launch_gemm<64, A_MN, B_MN, GROUPED>(tmA, tmB, tmA2, tmB2, p, stream);
  }
}

}  // namespace prb

// A, B, C are device pointers; lda/ldb/ldc are row pitches in elements of the stored 2-D
// tensors described at the top of this file. `block_expert` (device, int32) switches on
// grouped mode. `status` is a device int that receives a prb::StatusCode on a bounded-wait
// failure (and is left untouched otherwise). Returns 0 when the launch was issued.
static int gemm_bf16_impl(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, int a_mn, int b_mn, int out_fp32, float alpha, float beta,
                          const int* block_expert, int num_experts, int b_rows_per_expert, int force_bn,
                          const void* A2, const void* B2, int K2, long long lda2, long long ldb2,
                          int b2_rows_per_expert, int* status, void* stream_, const int* row_valid = nullptr,
                          const prb::SplitKWorkspace* sk = nullptr, const unsigned* blk_arrive = nullptr,
                          const int* blk_rows = nullptr) {
  using namespace prb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -3;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -4;  // TMA needs 16-byte aligned bases and row pitches
  const bool grouped = block_expert != nullptr;
  // Grouped MN-major B with a reduction length that is not a multiple of 64: the last K
  // slab of expert e also covers the first rows of expert e+1, but the matching columns of
  // A lie past K and are zero-filled by TMA, so they contribute nothing (B must be finite).
  int bn = force_bn > 0 ? force_bn : (N > 128 ? 256 : (N > 64 ? 128 : 64));
  // narrower tiles while the wide ones would leave SMs idle (decode-sized M): a 128 x 64 tile keeps the
  // tensor pipe half as busy per CTA, but an idle SM does nothing at all
  if (force_bn <= 0 && !grouped) {
    // the per-CTA traffic model of choose_splitk, one split only (a width that needs a second wave of CTAs is
    // worse than a wider tile that leaves some SMs idle)
    if ((long long)((M + 127) / 128) * ((N + 255) / 256) < sm_count()) {
      const SplitKWorkspace none{nullptr, 0, 1};
      choose_splitk(M, N, K, 0, none, bn);
    }
  } else if (force_bn <= 0 && bn == 256) {
    const long long t256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
    if (t256 < sm_count() && N % 256 != 0) bn = 128;
  }
  if (b_mn && bn < 64) bn = 64;
  int splits = 1;
  if (sk != nullptr && !grouped && !a_mn && A2 == nullptr && row_valid == nullptr &&
      (long long)((M + 127) / 128) * ((N + 255) / 256) * 2 <= sm_count())
    splits = choose_splitk(M, N, K, force_bn, *sk, bn);

  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn)
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda, kBM, kBK,
                      true);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda, kBK, 64,
                      true);
  if (rc) return rc;
  const uint64_t E = grouped ? (uint64_t)num_experts : 1;
  if (!b_mn)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, grouped ? E * b_rows_per_expert : (uint64_t)N,
                      (uint64_t)K, (uint64_t)ldb, bn, kBK, true);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, grouped ? E * b_rows_per_expert : (uint64_t)K,
                      (uint64_t)N, (uint64_t)ldb, kBK, 64, true);
  if (rc) return rc;
  CUtensorMap tmA2 = tmA, tmB2 = tmB;
  if (A2 != nullptr && K2 > 0) {
    // the extra segment shares the layout flags of the main operands; A2 is always [M, K2]
    if (a_mn) return -6;
    if ((lda2 % 8) || (ldb2 % 8) || (reinterpret_cast<uintptr_t>(A2) & 15) || (reinterpret_cast<uintptr_t>(B2) & 15))
      return -4;
    rc = make_tmap_2d(&tmA2, A2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K2, (uint64_t)lda2, kBM,
                      kBK, true);
    if (rc) return rc;
    if (!b_mn)
      rc = make_tmap_2d(&tmB2, B2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                        grouped ? E * b2_rows_per_expert : (uint64_t)N, (uint64_t)K2, (uint64_t)ldb2, bn, kBK, true);
    else
      rc = make_tmap_2d(&tmB2, B2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                        grouped ? E * b2_rows_per_expert : (uint64_t)K2, (uint64_t)N, (uint64_t)ldb2, kBK, 64, true);
    if (rc) return rc;
  }

  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.rows_total = M;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.k2_blocks = (A2 != nullptr && K2 > 0) ? (K2 + kBK - 1) / kBK : 0;
  p.b2_rows_per_expert = b2_rows_per_expert;
  p.row_valid = row_valid;
  p.blk_arrive = grouped ? blk_arrive : nullptr;
  p.blk_rows = blk_rows;
  p.expert_offset = nullptr; p.num_experts = 0;
  p.alpha = alpha; p.beta = beta;
  p.block_expert = block_expert;
  p.b_rows_per_expert = b_rows_per_expert;
  p.status = status;
  p.num_splits = 0;
  p.labels = nullptr; p.inv_temp = nullptr; p.part_m = p.part_s = p.part_t = p.target_logit = nullptr;
  p.grad_logprob = nullptr; p.lse = nullptr;
  if (splits > 1) {
    // the GEMM proper writes fp32 partials (alpha = 1, beta = 0) to the workspace, split ks to rows ks * M ..
    p.sk_splits = splits;
    p.C = sk->ws; p.ldc = N; p.out_fp32 = 1; p.alpha = 1.f; p.beta = 0.f;
    p.rows_total = static_cast<long long>(splits) * M;
    int rc2;
    switch (bn) {
      case 256: rc2 = b_mn ? launch_gemm_splitk<256, true>(tmA, tmB, p, stream) : launch_gemm_splitk<256, false>(tmA, tmB, p, stream); break;
      case 128: rc2 = b_mn ? launch_gemm_splitk<128, true>(tmA, tmB, p, stream) : launch_gemm_splitk<128, false>(tmA, tmB, p, stream); break;
      default: rc2 = b_mn ? launch_gemm_splitk<64, true>(tmA, tmB, p, stream) : launch_gemm_splitk<64, false>(tmA, tmB, p, stream); break;
    }
    if (rc2) return rc2;
    const long long items = static_cast<long long>(M) * (N / 4);
    long long blocks = (items + 255) / 256;
    if (blocks > 4LL * sm_count()) blocks = 4LL * sm_count();
    splitk_reduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(sk->ws, splits, M, N, C, ldc, out_fp32,
                                                                           alpha, beta);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }

  if (!grouped && a_mn && b_mn && out_fp32 && beta == 1.f && A2 == nullptr && row_valid == nullptr && (N % 4 == 0) &&
      (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0)) {
    // weight gradient accumulated in place: TMA reduce-adds instead of a read-modify-write by the epilogue warps
    CUtensorMap tmC;
    rc = make_tmap_2d(&tmC, C, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, 32, 32, true);
    if (rc) return rc;
    switch (bn) {
      case 256: return launch_gemm_reduce<256>(tmA, tmB, tmC, p, stream);
      case 128: return launch_gemm_reduce<128>(tmA, tmB, tmC, p, stream);
      default: return launch_gemm_reduce<64>(tmA, tmB, tmC, p, stream);
    }
  }

#define PRB_DISPATCH(AMN, BMN)                                                              \
  (grouped ? dispatch_bn<AMN, BMN, true>(bn, tmA, tmB, tmA2, tmB2, p, stream)                           \
           : dispatch_bn<AMN, BMN, false>(bn, tmA, tmB, tmA2, tmB2, p, stream))
  if (!a_mn && !b_mn) return PRB_DISPATCH(false, false);
  if (!a_mn && b_mn) return PRB_DISPATCH(false, true);
  if (a_mn && b_mn) return PRB_DISPATCH(true, true);
  return PRB_DISPATCH(true, false);
#undef PRB_DISPATCH
}

PRB_API int prb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, int a_mn, int b_mn, int out_fp32, float alpha, float beta,
                          const int* block_expert, int num_experts, int b_rows_per_expert, int force_bn,
                          int* status, void* stream_) {
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, alpha, beta, block_expert, num_experts,
                        b_rows_per_expert, force_bn, nullptr, nullptr, 0, 0, 0, 0, status, stream_);
}

// Grouped GEMM whose A rows arrive from other GPUs while it runs: M block b is loaded once blk_arrive[b] >=
// blk_rows[b] (uint32 / int32 per 128-row block; see csrc/ep_p2p.cu: ep_push_blocks_kernel).
PRB_API int prb_gemm_bf16_grouped_arrive(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                         long long ldb, long long ldc, int b_mn, int out_fp32,
                                         const int* block_expert, int num_experts, int b_rows_per_expert,
                                         const void* blk_arrive, const int* blk_rows, int* status, void* stream_) {
  if (block_expert == nullptr || blk_arrive == nullptr || blk_rows == nullptr) return -2;
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, 0, b_mn, out_fp32, 1.f, 0.f, block_expert, num_experts,
                        b_rows_per_expert, 0, nullptr, nullptr, 0, 0, 0, 0, status, stream_, nullptr, nullptr,
                        reinterpret_cast<const unsigned*>(blk_arrive), blk_rows);
}

// Dense GEMM with few rows (decode): may split the reduction over several CTAs per output tile, whose fp32
// partials a second kernel adds in split order (the result does not depend on timing). `ws` (ws_bytes, 16-byte
// aligned) is scratch that calls on one stream may share; force_splits > 0 pins the split count (1 = one kernel).
PRB_API int prb_gemm_bf16_splitk(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                 long long ldb, long long ldc, int b_mn, int out_fp32, float alpha, float beta,
                                 void* ws, long long ws_bytes, int force_bn, int force_splits, int* status,
                                 void* stream_) {
  prb::SplitKWorkspace w{reinterpret_cast<float*>(ws), ws_bytes, force_splits};
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, 0, b_mn, out_fp32, alpha, beta, nullptr, 0, 0, force_bn,
                        nullptr, nullptr, 0, 0, 0, 0, status, stream_, nullptr, &w);
}

// Same as prb_gemm_bf16, but rows r of C with row_valid[r] < 0 are computed and not stored: the padding rows that
// round every expert of a grouped inference GEMM up to 128 (their inputs may hold anything).
PRB_API int prb_gemm_bf16_rowmask(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                  long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32, float alpha,
                                  float beta, const int* block_expert, int num_experts, int b_rows_per_expert,
                                  int force_bn, const int* row_valid, int* status, void* stream_) {
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, alpha, beta, block_expert, num_experts,
                        b_rows_per_expert, force_bn, nullptr, nullptr, 0, 0, 0, 0, status, stream_, row_valid);
}

// C = alpha * (A B + A2 B2) + beta * C in one pass: the accumulator of every tile takes the
// K blocks of (A, B) and then those of (A2, B2). Used for y = x W^T + (x A^T) B^T of a LoRA
// linear (and its input gradient), where a separate rank-r product would re-read and re-write
// all of C. A2: bf16 [M, K2] row-major; B2 is laid out like B (K-major [N, K2] rows, or
// MN-major [K2, N]); grouped mode: b2_rows_per_expert rows of B2 per expert.
PRB_API int prb_gemm_bf16_ext(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                              long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32, float alpha,
                              float beta, const int* block_expert, int num_experts, int b_rows_per_expert,
                              int force_bn, const void* A2, const void* B2, int K2, long long lda2, long long ldb2,
                              int b2_rows_per_expert, int* status, void* stream_) {
  return gemm_bf16_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, alpha, beta, block_expert, num_experts,
                        b_rows_per_expert, force_bn, A2, B2, K2, lda2, ldb2, b2_rows_per_expert, status, stream_);
}

// C_shard[owner(row)] += alpha * (A B)[row] with fp32 reductions into the owners' shards
// (peer_c: R device pointers, own shard at index rank; rows_per_rank rows of pitch ldc each).
// Dense operands only; B K-major [N, K] or MN-major [K, N]; A K-major [M, K] or MN-major [K, M].
PRB_API int prb_gemm_bf16_reduce_scatter(const void* A, const void* B, int M, int N, int K, long long lda,
                                         long long ldb, int a_mn, int b_mn, float alpha, void* const* peer_c,
                                         int num_ranks, int rows_per_rank, long long ldc, int* status,
                                         void* stream_) {
  using namespace prb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || num_ranks < 1 || num_ranks > 8 || rows_per_rank <= 0 ||
      static_cast<long long>(rows_per_rank) * num_ranks < M)
    return -3;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -4;
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn)
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda, kBM, kBK,
                      true);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda, kBK, 64,
                      true);
  if (rc) return rc;
  if (!b_mn)
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 256, kBK,
                      true);
  else
    rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, kBK, 64,
                      true);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.rows_total = M;
  p.C = nullptr; p.ldc = ldc; p.out_fp32 = 1;
  p.expert_offset = nullptr; p.num_experts = 0;
  p.alpha = alpha; p.beta = 0.f;
  p.block_expert = nullptr; p.b_rows_per_expert = 0;
  p.status = status;
  p.num_splits = 0;
  p.labels = nullptr; p.inv_temp = nullptr; p.part_m = p.part_s = p.part_t = p.target_logit = nullptr;
  p.grad_logprob = nullptr; p.lse = nullptr;
  for (int i = 0; i < num_ranks; ++i) p.peer_c[i] = reinterpret_cast<float*>(peer_c[i]);
  p.rows_per_rank = rows_per_rank;
  using Cfg = GemmCfg<256>;
  const int tiles = ((M + kBM - 1) / kBM) * ((N + 255) / 256);
  const int grid = tiles < sm_count() ? tiles : sm_count();
#define PRB_RS_LAUNCH(AMN, BMN)                                                                              \
  {                                                                                                          \
    auto kern = gemm_bf16_kernel<256, AMN, BMN, SchedDense, EpiPeerReduce>;                                  \
    static prb::DeviceOnce configured;                                                                          \
    if (configured.pending()) {                                                                                       \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) \
        return -10;                                                                                          \
      configured.mark();                                                                                     \
    }                                                                                                        \
    kern<<<grid, kGemmThreads, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, tmA, tmB, p);                            \
  }
  if (!a_mn && !b_mn) PRB_RS_LAUNCH(false, false)
  else if (!a_mn && b_mn) PRB_RS_LAUNCH(false, true)
  else if (a_mn && b_mn) PRB_RS_LAUNCH(true, true)
  else PRB_RS_LAUNCH(true, false)
#undef PRB_RS_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// C = alpha * A W^T where W [N, K] (K-major, dense pitch K) is row-sharded over the ranks: the
// full-size buffer `w_local` holds this rank's rows [rank * rows_per_rank, ...) and receives the
// other ranks' rows from `peer_w[r]` (the same buffer on rank r) while the tiles that need only
// local rows are already running. `ready` holds one counter per 256-row N block (zero before the
// first call, never reset); `call_index` counts calls from 1. The caller orders this launch after
// every rank has published its rows and must not rewrite its rows until all ranks have finished.
PRB_API int prb_gemm_bf16_allgather(const void* A, void* w_local, void* const* peer_w, void* C, int M, int N, int K,
                                    long long lda, long long ldc, int a_mn, int out_fp32, float alpha, int rank,
                                    int num_ranks, int rows_per_rank, unsigned* ready, unsigned call_index,
                                    int* status, void* stream_) {
  using namespace prb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || num_ranks < 1 || num_ranks > 8 || rank < 0 || rank >= num_ranks || rows_per_rank <= 0 ||
      rows_per_rank % 256 != 0 || rows_per_rank * num_ranks != N || K % 8 != 0)
    return -3;
  if ((lda % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(w_local) & 15)) return -4;
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn)
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda, kBM, kBK,
                      true);
  else
    rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda, kBK, 64,
                      true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, w_local, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)N, (uint64_t)K, (uint64_t)K, 256, kBK,
                    true);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.rows_total = M;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.expert_offset = nullptr; p.num_experts = 0;
  p.alpha = alpha; p.beta = 0.f;
  p.block_expert = nullptr; p.b_rows_per_expert = 0;
  p.status = status;
  p.num_splits = 0;
  p.labels = nullptr; p.inv_temp = nullptr; p.part_m = p.part_s = p.part_t = p.target_logit = nullptr;
  p.grad_logprob = nullptr; p.lse = nullptr;
  for (int i = 0; i < num_ranks; ++i) p.ag_src[i] = reinterpret_cast<const uint8_t*>(peer_w[i]);
  p.ag_dst = reinterpret_cast<uint8_t*>(w_local);
  p.ag_ready = ready;
  p.ag_target = call_index;
  p.ag_rank = rank; p.ag_ranks = num_ranks; p.ag_rows = rows_per_rank;
  p.ag_row_bytes = static_cast<long long>(K) * 2;
  using Cfg = GemmCfg<256>;
  const int tiles = ((M + kBM - 1) / kBM) * (N / 256);
  // every CTA must be resident at once (producers wait on the gather warps of all CTAs)
  const int grid = tiles < sm_count() ? tiles : sm_count();
#define PRB_AG_LAUNCH(AMN)                                                                                   \
  {                                                                                                          \
    auto kern = gemm_bf16_kernel<256, AMN, false, SchedAllGather, EpiStore>;                                 \
    static prb::DeviceOnce configured;                                                                          \
    if (configured.pending()) {                                                                                       \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) \
        return -10;                                                                                          \
      configured.mark();                                                                                     \
    }                                                                                                        \
    kern<<<grid, kGemmThreads + 32 * SchedAllGather::kGatherWarps, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, tmA, tmB, p); \
  }
  if (!a_mn) PRB_AG_LAUNCH(false)
  else PRB_AG_LAUNCH(true)
#undef PRB_AG_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// ---------------------------------------------------------------- fused LM head
// Replaces _SequenceChunkedLogProbEntropyFn (trainer/models/layers/lm_head.py:114-266 of the
// reference): logits never reach global memory in the forward pass.
namespace prb {

// logprob = z_label - lse, entropy = lse - sum(p z), from the per-split partials.
__global__ void __launch_bounds__(256)
lmhead_combine_kernel(const float* __restrict__ part_m, const float* __restrict__ part_s,
                      const float* __restrict__ part_t, const float* __restrict__ target, const int* __restrict__ labels,
                      float* __restrict__ logprob, float* __restrict__ entropy, float* __restrict__ lse_out,
                      long long T, int splits, int V) {
  const long long r = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= T) return;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_m[static_cast<long long>(s) * T + r]);
  float S = 0.f, Tt = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float c = __expf(part_m[static_cast<long long>(s) * T + r] - M);
    S += part_s[static_cast<long long>(s) * T + r] * c;
    Tt += part_t[static_cast<long long>(s) * T + r] * c;
  }
  const float lse = M + logf(S);
  lse_out[r] = lse;
  const int lb = labels[r];
  logprob[r] = (lb >= 0 && lb < V) ? target[r] - lse : 0.f;
  entropy[r] = lse - Tt / S;
}

static int lmhead_maps(CUtensorMap* tmA, CUtensorMap* tmB, const void* h, const void* W, int T, int V, int H,
                       long long ldh, long long ldw) {
  if ((ldh % 8) || (ldw % 8) || (reinterpret_cast<uintptr_t>(h) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return -4;
  int rc = make_tmap_2d(tmA, h, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)T, (uint64_t)H, (uint64_t)ldh, kBM,
                        kBK, true);
  if (rc) return rc;
  return make_tmap_2d(tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)V, (uint64_t)H, (uint64_t)ldw, 256, kBK,
                      true);
}

}  // namespace prb

// Number of vocabulary splits the forward kernel will use for T rows and V columns; the
// caller sizes part_m / part_s / part_t as fp32 [splits, T].
PRB_API int prb_lmhead_num_splits(int T, int V) {
  const int tiles_m = (T + 127) / 128;
  const int tiles_n = (V + 255) / 256;
  int s = (2 * prb::sm_count() + tiles_m - 1) / tiles_m;
  if (s < 1) s = 1;
  if (s > tiles_n) s = tiles_n;
  // avoid empty trailing splits
  const int per = (tiles_n + s - 1) / s;
  s = (tiles_n + per - 1) / per;
  return s;
}

// h: bf16 [T, H]; W: bf16 [V, H]; labels: int32 [T] (outside [0, V) = ignored, logprob 0);
// inv_temp: fp32 [T] or null. Outputs fp32 [T]: logprob, entropy, lse. Scratch: part_*
// fp32 [splits, T] and target fp32 [T] (zeroed here).
PRB_API int prb_lmhead_fwd(const void* h, const void* W, const int* labels, const float* inv_temp, float* part_m,
                           float* part_s, float* part_t, float* target, float* logprob, float* entropy, float* lse,
                           int T, int V, int H, long long ldh, long long ldw, int splits, int* status,
                           void* stream_) {
  using namespace prb;
  if (T <= 0) return 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (splits < 1) return -12;
  {
    // a slice without vocabulary tiles writes no partial row, and the merge reads every row:
    // use only as many slices as own at least one tile (the scratch layout is indexed by slice)
    const int tiles_n = (V + 255) / 256;
    const int per = (tiles_n + splits - 1) / splits;
    splits = (tiles_n + per - 1) / per;
  }
  CUtensorMap tmA, tmB;
  int rc = lmhead_maps(&tmA, &tmB, h, W, T, V, H, ldh, ldw);
  if (rc) return rc;
  GemmParams p = {};
  p.M = T; p.N = V; p.K = H; p.rows_total = T;
  p.alpha = 1.f; p.status = status;
  p.num_splits = splits;
  p.labels = labels; p.inv_temp = inv_temp;
  p.part_m = part_m; p.part_s = part_s; p.part_t = part_t; p.target_logit = target;
  cudaMemsetAsync(target, 0, sizeof(float) * T, stream);
  using Cfg = GemmCfg<256>;
  auto kern = gemm_bf16_kernel<256, false, false, SchedSplit, EpiLogprobStats>;
  static prb::DeviceOnce configured;
  if (configured.pending()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return -10;
    configured.mark();
  }
  const int items = ((T + 127) / 128) * splits;
  const int grid = items < sm_count() ? items : sm_count();
  kern<<<grid, kGemmThreads, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, tmA, tmB, p);
  lmhead_combine_kernel<<<(T + 255) / 256, 256, 0, stream>>>(part_m, part_s, part_t, target, labels, logprob, entropy,
                                                            lse, T, splits, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// dlogits (bf16 [T, V], pitch ldd) = grad_logprob[row] * inv_temp[row] * (onehot - softmax).
PRB_API int prb_lmhead_bwd_dlogits(const void* h, const void* W, const int* labels, const float* inv_temp,
                                   const float* grad_logprob, const float* lse, void* dlogits, int T, int V, int H,
                                   long long ldh, long long ldw, long long ldd, int* status, void* stream_) {
  using namespace prb;
  if (T <= 0) return 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  CUtensorMap tmA, tmB;
  int rc = lmhead_maps(&tmA, &tmB, h, W, T, V, H, ldh, ldw);
  if (rc) return rc;
  GemmParams p = {};
  p.M = T; p.N = V; p.K = H; p.rows_total = T;
  p.C = dlogits; p.ldc = ldd;
  p.alpha = 1.f; p.status = status;
  p.labels = labels; p.inv_temp = inv_temp; p.grad_logprob = grad_logprob; p.lse = lse;
  using Cfg = GemmCfg<256>;
  auto kern = gemm_bf16_kernel<256, false, false, SchedDense, EpiDLogits>;
  static prb::DeviceOnce configured;
  if (configured.pending()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return -10;
    configured.mark();
  }
  const int tiles = ((T + 127) / 128) * ((V + 255) / 256);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kGemmThreads, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Per-expert weight gradient: C[e] (rows [e*M, (e+1)*M) of a [E*M, N] tensor) =
// alpha * A_e^T . B_e + beta * C[e], where A is [rows, M] and B is [rows, N] (both
// MN-major, bf16) and expert e owns rows [expert_offset[e], expert_offset[e+1]) — multiples
// of 128. Rows of A / B past the last expert are never read.
PRB_API int prb_gemm_bf16_kgrouped(const void* A, const void* B, void* C, int M, int N, long long total_rows,
                                   long long lda, long long ldb, long long ldc, int out_fp32, float alpha,
                                   float beta, const int* expert_offset, int num_experts, int* status,
                                   void* stream_) {
  using namespace prb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || num_experts <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -4;
  const int bn = N > 128 ? 256 : (N > 64 ? 128 : 64);
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_rows, (uint64_t)M,
                        (uint64_t)lda, kBK, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_rows, (uint64_t)N, (uint64_t)ldb,
                    kBK, 64, true);
  if (rc) return rc;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = 0; p.rows_total = static_cast<long long>(num_experts) * M;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.alpha = alpha; p.beta = beta;
  p.status = status;
  p.expert_offset = expert_offset; p.num_experts = num_experts;
  const long long tiles = static_cast<long long>(num_experts) * ((M + kBM - 1) / kBM) * ((N + bn - 1) / bn);
  const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  // pure accumulation into an fp32 buffer (the flat gradient accumulator): hand the tiles to the TMA unit as
  // reduce-adds instead of reading C back (see EpiTmaReduce)
  const bool tma_reduce = out_fp32 && beta == 1.f && (M % kBM == 0) && (N % 4 == 0) && (ldc % 4 == 0) &&
                          ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
  CUtensorMap tmC = tmA;
  if (tma_reduce) {
    rc = make_tmap_2d(&tmC, C, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)num_experts * (uint64_t)M, (uint64_t)N,
                      (uint64_t)ldc, 32, 32, true);
    if (rc) return rc;
  }
#define PRB_KG(BN_, EPI_, EXTRA_)                                                                         \
  {                                                                                                       \
    auto kern = gemm_bf16_kernel<BN_, true, true, SchedKGrouped, EPI_>;                                   \
    static prb::DeviceOnce configured;                                                                       \
    if (configured.pending()) {                                                                                    \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                         \
                               GemmCfg<BN_>::SMEM_BYTES + EXTRA_) != cudaSuccess)                         \
        return -10;                                                                                       \
      configured.mark();                                                                                  \
    }                                                                                                     \
    kern<<<grid, kGemmThreads, GemmCfg<BN_>::SMEM_BYTES + EXTRA_, stream>>>(tmA, tmB, tmC, tmB, p);       \
  }
  constexpr int kRedExtra = 768 + kRedStageBytes;
  if (tma_reduce) {
    if (bn == 256) PRB_KG(256, EpiTmaReduce, kRedExtra) else if (bn == 128) PRB_KG(128, EpiTmaReduce, kRedExtra)
    else PRB_KG(64, EpiTmaReduce, kRedExtra)
  } else {
    if (bn == 256) PRB_KG(256, EpiStore, 0) else if (bn == 128) PRB_KG(128, EpiStore, 0) else PRB_KG(64, EpiStore, 0)
  }
#undef PRB_KG
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
