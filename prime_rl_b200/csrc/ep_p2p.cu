// Expert-parallel token exchange over NVLink peer memory (one process per GPU, buffers mapped
// into every rank with CUDA IPC). Rows go straight from the sender's activations into their
// final position of the owner's expert-sorted, 128-row-aligned buffer (no staging copy, no
// host read of split sizes), and come back through peer loads fused with the top-k weighted
// sum. Synchronisation is by epoch flags in peer memory; every wait is bounded.
//
//   ep_hist_kernel     every rank stores its per-expert pair counts into all peers' tables
//   ep_plan_kernel     waits for the tables, then derives (a) where this rank's rows of each
//                      expert start inside the owner's buffer, (b) the local expert offsets /
//                      block map for the grouped GEMM
//   ep_push_kernel     one warp per (token, k) pair: 16-byte peer stores of the row (optionally
//                      scaled: the gradient of the combine), then a data flag on every peer
//   ep_recv_kernel     waits for all senders' data flags, zeroes the padding rows
//   ep_push_fp8_kernel / ep_recv_fp8_kernel   the same trip with an e4m3 payload: the sender
//                      quantises each 128-column group of a row (scale = amax / 448, fp32) on
//                      the way out, the owner expands its rows back to bf16 after the flags
//   ep_prepare_kernel / ep_push_blocks_kernel   the dispatch without a global wait: rows are pushed in the
//                      order of the owner's buffer (whole 128-row runs of one expert at a time, starting with
//                      the next rank's experts), every run ends with a release-add of its row count onto
//                      the arrival counter of the owner's 128-row block, and the owner's grouped GEMM waits
//                      per block (csrc/gemm.cu: blk_wait) instead of for everybody
//   ep_signal_kernel   "my buffer is complete" flag on every peer
//   ep_pull_kernel     waits for the owners' flags; out[t] = sum_k w[t,k] * peer_row(t,k) with
//                      peer loads (also: gradient of the dispatch with w = 1); optional
//                      dw[t,k] = <peer_row(t,k), g[t]>
//
// Takes the place of the all-to-all token dispatchers of the reference
// (src/prime_rl/trainer/distributed/token_dispatcher.py:247-301 and its DeepEP variant,
// deepep.py): those move rows with library collectives and permute them in separate kernels.
// No TMA multicast and no library kernel ever touches peer memory here: plain ld / st only.
#include <cuda_fp8.h>

#include "common.cuh"

namespace prb {

constexpr int kEpMaxRanks = 16;
constexpr long long kEpWaitCycles = 4000000000LL;   // about 2 s

struct EpPeers {
  void* buf[kEpMaxRanks];     // a symmetric buffer on every rank (index = rank)
};

// flags: int32 [kinds][R] on every rank; slot [kind][src] is written by rank src only.
__device__ __forceinline__ bool ep_wait_flag(const int* flag, int epoch, int* status) {
  const volatile int* f = flag;
  if (*f - epoch >= 0) return true;
  const long long t0 = clock64();
  unsigned spins = 0;
  while (*f - epoch < 0) {
    if ((++spins & 0xff) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (clock64() - t0 > kEpWaitCycles) {
        atomicCAS(status, 0, static_cast<int>(kTimeoutPeerFlag));
        return false;
      }
    }
  }
  return true;
}

// All threads of the CTA return the same verdict; thread i < R waits for source i.
__device__ __forceinline__ bool ep_wait_all(const int* flags_kind, int R, int epoch, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < R && !ep_wait_flag(flags_kind + threadIdx.x, epoch, status)) s_ok = 0;
  __syncthreads();
  __threadfence_system();   // acquire side: order the payload reads after the flag reads
  return s_ok != 0;
}

__global__ void __launch_bounds__(128)
ep_hist_kernel(const int* __restrict__ counts, EpPeers hist, EpPeers flags, int rank, int R, int E, int kind,
               int epoch) {
  for (int d = 0; d < R; ++d) {
    int* dst = reinterpret_cast<int*>(hist.buf[d]) + rank * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < R) {
    volatile int* f = reinterpret_cast<int*>(flags.buf[threadIdx.x]) + kind * R + rank;
    *f = epoch;
  }
}

// hist: local table [R][E]. send_base[e]: first row of this rank's pairs of expert e inside the
// owner's buffer. expert_offset [El + 1], block_expert [max_blocks], total_rows [1]: the local
// receive layout. Sets kBadArgument in *status when the local layout exceeds cap_rows.
__global__ void __launch_bounds__(128)
ep_plan_kernel(const int* __restrict__ hist, const int* __restrict__ flags_kind, int rank, int R, int E, int epoch,
               int cap_rows, int max_blocks, int* __restrict__ send_base, int* __restrict__ expert_offset,
               int* __restrict__ block_expert, int* __restrict__ total_rows, int* status) {
  __shared__ int s_off[1024 + 1];
  if (!ep_wait_all(flags_kind, R, epoch, status)) return;
  const int El = E / R;
  // every thread owns some global experts: totals and the part in front of this rank
  __shared__ int s_tot[1024], s_pre[1024];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, pre = 0;
    for (int s = 0; s < R; ++s) {
      const int c = hist[s * E + e];
      tot += c;
      if (s < rank) pre += c;
    }
    s_tot[e] = tot;
    s_pre[e] = pre;
  }
  __syncthreads();
  if (threadIdx.x < R) {   // thread d lays out destination d
    const int d = threadIdx.x;
    int off = 0;
    for (int le = 0; le < El; ++le) {
      const int e = d * El + le;
      send_base[e] = off + s_pre[e];
      if (d == rank) s_off[le] = off;
      off += (s_tot[e] + 127) / 128 * 128;
    }
    if (d == rank) {
      s_off[El] = off;
      total_rows[0] = off;
      if (off > cap_rows) atomicCAS(status, 0, static_cast<int>(kBadArgument));
    }
  }
  __syncthreads();
  for (int le = threadIdx.x; le <= El; le += blockDim.x) expert_offset[le] = s_off[le];
  for (int b = threadIdx.x; b < max_blocks; b += blockDim.x) {
    const int row = b * 128;
    int ex = -1;
    if (row < s_off[El]) {
      int lo = 0, hi = El;   // last le with s_off[le] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid;
      }
      ex = lo;
    }
    block_expert[b] = ex;
  }
}

// One warp per pair. pos_out[p] = row inside the owner's buffer (kept for the way back).
// When pos_in != nullptr the positions are given (second trip over the same routes).
__global__ void __launch_bounds__(256)
ep_push_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx, const int* __restrict__ slot,
               const int* __restrict__ local_off, const int* __restrict__ send_base, const int* __restrict__ pos_in,
               const float* __restrict__ scale, EpPeers dst, EpPeers flags, int* __restrict__ pos_out,
               unsigned* __restrict__ done_counter, int num_pairs, int k, int H, int El, int rank, int R, int kind,
               int epoch, int cap_rows, int* status) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  for (int p = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); p < num_pairs; p += gridDim.x * warps_per_cta) {
    const int e = topk_idx[p];
    const int d = e / El;
    const int pos = pos_in ? pos_in[p] : send_base[e] + slot[p] - local_off[e];
    if (pos_out && lane == 0) pos_out[p] = pos;
    if (pos < 0 || pos >= cap_rows) {   // never store outside the peer's buffer
      if (lane == 0) atomicCAS(status, 0, static_cast<int>(kBadArgument));
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(p / k) * H);
    uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.buf[d]) + static_cast<long long>(pos) * H);
    if (scale == nullptr) {
      for (int i = lane; i < H / 8; i += 32) out[i] = src[i];
    } else {
      const float s = scale[p];
      for (int i = lane; i < H / 8; i += 32) {
        uint4 v = src[i];
        float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), dd = unpack_bf16(v.w);
        v.x = pack_bf16(a.x * s, a.y * s); v.y = pack_bf16(b.x * s, b.y * s);
        v.z = pack_bf16(c.x * s, c.y * s); v.w = pack_bf16(dd.x * s, dd.y * s);
        out[i] = v;
      }
    }
  }
  // completion: the last CTA to finish raises the data flag on every peer
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(done_counter, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < R) {
      volatile int* f = reinterpret_cast<int*>(flags.buf[threadIdx.x]) + kind * R + rank;
      *f = epoch;
    }
    if (threadIdx.x == 0) *done_counter = 0;   // ready for the next launch on this stream
  }
}

// One CTA per local expert: wait for every sender, then zero the rows between the expert's
// real rows and its 128-aligned end (they take part in reductions over the row range).
__global__ void __launch_bounds__(256)
ep_recv_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ hist, const int* __restrict__ expert_offset,
               const int* __restrict__ flags_kind, int rank, int R, int E, int H, int epoch, int* status) {
  if (!ep_wait_all(flags_kind, R, epoch, status)) return;
  const int El = E / R;
  const int le = blockIdx.x;
  if (le >= El) return;
  int tot = 0;
  for (int s = 0; s < R; ++s) tot += hist[s * E + rank * El + le];
  const long long r0 = expert_offset[le] + tot, r1 = expert_offset[le + 1];
  uint4* p = reinterpret_cast<uint4*>(buf + r0 * H);
  const long long n = (r1 - r0) * (H / 8);
  for (long long i = threadIdx.x; i < n; i += blockDim.x) p[i] = make_uint4(0u, 0u, 0u, 0u);
}


// Owner side of the per-block dispatch: one CTA per local expert. (a) rows each of its 128-row blocks will
// receive (block_rows, what the GEMM producer compares the arrival counter with), (b) zeroes the padding rows
// behind the expert's last real row (nobody pushes there), (c) zeroes the arrival counters of the OTHER parity
// for the call after this one: no peer can be pushing for that call yet, because pushes start after the
// histogram exchange in which this rank takes part only after this kernel.
__global__ void __launch_bounds__(256)
ep_prepare_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ hist, const int* __restrict__ expert_offset,
                  int* __restrict__ block_rows, unsigned* __restrict__ zero_cnt, int max_blocks, int rank, int R, int E,
                  int H) {
  const int El = E / R;
  const int le = blockIdx.x;
  for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < max_blocks; b += gridDim.x * blockDim.x) zero_cnt[b] = 0u;
  int tot = 0;
  for (int s = 0; s < R; ++s) tot += hist[s * E + rank * El + le];
  const int r0 = expert_offset[le], r1 = expert_offset[le + 1];
  for (int b = r0 / 128 + threadIdx.x; b < r1 / 128; b += blockDim.x)
    block_rows[b] = max(0, min(128, tot - (b * 128 - r0)));
  if (le == El - 1)
    for (int b = r1 / 128 + threadIdx.x; b < max_blocks; b += blockDim.x) block_rows[b] = 0;
  uint4* p = reinterpret_cast<uint4*>(buf + static_cast<long long>(r0 + tot) * H);
  const long long n = static_cast<long long>(r1 - r0 - tot) * (H / 8);
  for (long long i = threadIdx.x; i < n; i += blockDim.x) p[i] = make_uint4(0u, 0u, 0u, 0u);
}

// Sender side: CTA i takes the local 128-row block (i + first) % blocks of the expert-sorted pair order
// (row_src / block_expert / local_off: the local routing plan), `first` = the first block of the next rank's
// experts, so that at any moment the ranks write to different owners. The block's real rows are consecutive
// rows of the owner's buffer; after the stores: system fence, CTA barrier, then one release-add per touched
// owner block.
__global__ void __launch_bounds__(256)
ep_push_blocks_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_src,
                      const int* __restrict__ local_block_expert, const int* __restrict__ local_off,
                      const int* __restrict__ local_total, const int* __restrict__ counts,
                      const int* __restrict__ send_base, EpPeers dst, EpPeers cnt, long long cnt_off,
                      int* __restrict__ pos_out, int k, int H, int El, int rank, int R, int cap_rows, int* status) {
  const int nblk = local_total[0] / 128;
  if (nblk <= 0) return;
  const int first = local_off[((rank + 1) % R) * El] / 128 % nblk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = blockIdx.x; i < nblk; i += gridDim.x) {
    int b = i + first;
    if (b >= nblk) b -= nblk;
    const int e = local_block_expert[b];
    if (e < 0) continue;
    const int d = e / El;
    const int r0 = b * 128;
    const int n = min(128, counts[e] - (r0 - local_off[e]));
    const int pos0 = send_base[e] + (r0 - local_off[e]);
    if (n <= 0) continue;
    if (pos0 < 0 || pos0 + n > cap_rows) {   // never store outside the peer's buffer
      if (threadIdx.x == 0) atomicCAS(status, 0, static_cast<int>(kBadArgument));
      continue;
    }
    __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(dst.buf[d]) + static_cast<long long>(pos0) * H;
    for (int j = warp; j < n; j += 8) {
      const int p = row_src[r0 + j];
      if (lane == 0) pos_out[p] = pos0 + j;
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(p / k) * H);
      uint4* out = reinterpret_cast<uint4*>(base + static_cast<long long>(j) * H);
      for (int c = lane; c < H / 8; c += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c + 32 * u < H / 8) v[u] = src[c + 32 * u];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c + 32 * u < H / 8) out[c + 32 * u] = v[u];
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned* c = reinterpret_cast<unsigned*>(reinterpret_cast<uint8_t*>(cnt.buf[d]) + cnt_off) + pos0 / 128;
      const unsigned head = static_cast<unsigned>(min(n, 128 - (pos0 & 127)));
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(c), "r"(head) : "memory");
      if (static_cast<unsigned>(n) > head)
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(c + 1), "r"(static_cast<unsigned>(n) - head) : "memory");
    }
  }
}

// fp8 payload: one warp per pair, one 128-column group per iteration (lane = 4 columns). The
// quantised row goes to qdst [cap_rows, H] (bytes) and its scales to sdst [cap_rows, H / 128].
__global__ void __launch_bounds__(256)
ep_push_fp8_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_idx, const int* __restrict__ slot,
                   const int* __restrict__ local_off, const int* __restrict__ send_base, const int* __restrict__ pos_in,
                   const float* __restrict__ scale, EpPeers qdst, EpPeers sdst, EpPeers flags, int* __restrict__ pos_out,
                   unsigned* __restrict__ done_counter, int num_pairs, int k, int H, int El, int rank, int R, int kind,
                   int epoch, int cap_rows, int* status) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int groups = H / 128;
  for (int p = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); p < num_pairs; p += gridDim.x * warps_per_cta) {
    const int e = topk_idx[p];
    const int d = e / El;
    const int pos = pos_in ? pos_in[p] : send_base[e] + slot[p] - local_off[e];
    if (pos_out && lane == 0) pos_out[p] = pos;
    if (pos < 0 || pos >= cap_rows) {
      if (lane == 0) atomicCAS(status, 0, static_cast<int>(kBadArgument));
      continue;
    }
    const float s = scale ? scale[p] : 1.f;
    const uint2* src = reinterpret_cast<const uint2*>(x + static_cast<long long>(p / k) * H);
    uint32_t* qout = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(qdst.buf[d]) + static_cast<long long>(pos) * H);
    float* sout = reinterpret_cast<float*>(sdst.buf[d]) + static_cast<long long>(pos) * groups;
    for (int g = 0; g < groups; ++g) {
      const uint2 u = src[g * 32 + lane];
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
      const float v0 = a.x * s, v1 = a.y * s, v2 = b.x * s, v3 = b.y * s;
      float amax = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
      amax = warp_max(amax);
      const float sc = fmaxf(amax, 1e-12f) / 448.f, inv = 1.f / sc;
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v0 * inv, v1 * inv), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v2 * inv, v3 * inv), __NV_SATFINITE, __NV_E4M3);
      qout[g * 32 + lane] = lo | (hi << 16);
      if (lane == 0) sout[g] = sc;
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(done_counter, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < R) {
      volatile int* f = reinterpret_cast<int*>(flags.buf[threadIdx.x]) + kind * R + rank;
      *f = epoch;
    }
    if (threadIdx.x == 0) *done_counter = 0;
  }
}

// blockIdx.x = local expert, blockIdx.y strides over its rows: real rows are expanded from the
// e4m3 staging buffer into the bf16 buffer the grouped GEMM reads, padding rows are zeroed.
__global__ void __launch_bounds__(256)
ep_recv_fp8_kernel(__nv_bfloat16* __restrict__ buf, const uint8_t* __restrict__ q, const float* __restrict__ scales,
                   const int* __restrict__ hist, const int* __restrict__ expert_offset,
                   const int* __restrict__ flags_kind, int rank, int R, int E, int H, int epoch, int* status) {
  if (!ep_wait_all(flags_kind, R, epoch, status)) return;
  const int El = E / R;
  const int le = blockIdx.x;
  if (le >= El) return;
  int tot = 0;
  for (int s = 0; s < R; ++s) tot += hist[s * E + rank * El + le];
  const long long r0 = expert_offset[le], r_real = r0 + tot, r1 = expert_offset[le + 1];
  const int groups = H / 128;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (long long r = r0 + blockIdx.y * warps + warp; r < r1; r += static_cast<long long>(gridDim.y) * warps) {
    uint2* out = reinterpret_cast<uint2*>(buf + r * H);
    if (r >= r_real) {
      for (int i = lane; i < H / 4; i += 32) out[i] = make_uint2(0u, 0u);
      continue;
    }
    const uint32_t* qr = reinterpret_cast<const uint32_t*>(q + r * H);
    for (int g = 0; g < groups; ++g) {
      const float sc = scales[r * groups + g];
      const uint32_t w = qr[g * 32 + lane];
      const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w & 0xffffu), __NV_E4M3);
      const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w >> 16), __NV_E4M3);
      const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
      const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
      out[g * 32 + lane] = make_uint2(pack_bf16(f01.x * sc, f01.y * sc), pack_bf16(f23.x * sc, f23.y * sc));
    }
  }
}

// Reduce-scatter of a flat fp32 gradient buffer that every rank holds in symmetric memory: this
// rank sums elements [off, off + n) of all R buffers with peer loads, scales the sum and writes its
// fp32 shard (the cast / scale of the bucket happens in the same pass). n and off are multiples of 4.
__global__ void __launch_bounds__(256)
rs_pull_kernel(EpPeers grads, long long off, long long n4, float scale, float4* __restrict__ out, int R) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < R; ++r) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.buf[r]) + off) + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    out[i] = make_float4(acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale);
  }
}

// All-gather by stores: this rank's updated slice (n16 16-byte units at unit offset off16 of the
// flat parameter buffer) is written into the same place of every other rank's buffer; blockIdx.y
// walks over the peers.
__global__ void __launch_bounds__(256)
ag_push_kernel(const uint4* __restrict__ src, EpPeers dst, long long off16, long long n16, int rank, int R) {
  int d = blockIdx.y;
  if (d >= rank) ++d;                      // R - 1 destinations: everybody but me
  if (d >= R) return;
  uint4* o = reinterpret_cast<uint4*>(dst.buf[d]) + off16;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    o[i] = src[i];
}

// Plain copy of 16-byte units from a peer's (or this rank's) memory into local memory with a bounded grid, so that
// it can run on a side stream next to a compute kernel (the ring form of context parallelism pulls the K / V block
// of the next step with it while the current block is in the tensor cores).
__global__ void __launch_bounds__(256)
peer_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __ldcg(src + i);
}

// Every rank holds R slots of n bf16 elements in symmetric memory (slot o = its contribution for owner o). The owner
// sums slot `rank` of all R buffers in rank order (fp32) and writes bf16: a reduce-scatter by peer loads with a
// fixed summation order. n is a multiple of 8.
__global__ void __launch_bounds__(256)
slot_pull_reduce_kernel(EpPeers bufs, long long slot_off16, long long n16, uint4* __restrict__ out, int R) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < R; ++r) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(bufs.buf[r]) + slot_off16 + i);
      const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), d = unpack_bf16(v.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    out[i] = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                        pack_bf16(acc[6], acc[7]));
  }
}

__global__ void __launch_bounds__(32)
ep_signal_kernel(EpPeers flags, int rank, int R, int kind, int epoch) {
  __threadfence_system();
  if (threadIdx.x < R) {
    volatile int* f = reinterpret_cast<int*>(flags.buf[threadIdx.x]) + kind * R + rank;
    *f = epoch;
  }
}

// Waits until every rank's flag of one kind has reached `epoch` (a stream-ordered barrier
// between kernels that touch peer memory).
__global__ void __launch_bounds__(32)
ep_wait_kernel(const int* __restrict__ flags_kind, int R, int epoch, int* status) {
  ep_wait_all(flags_kind, R, epoch, status);
}

// Equal-split all-to-all, send side: blockIdx.y = destination rank; block d of `src` (bytes16
// 16-byte units) goes to slot `rank` of rank d's receive buffer. The last CTA raises the data flag
// on every peer.
__global__ void __launch_bounds__(256)
a2a_push_kernel(const uint4* __restrict__ src, EpPeers dst, EpPeers flags, long long bytes16, long long slot16,
                long long buf_off16, unsigned* __restrict__ done_counter, int rank, int R, int kind, int epoch) {
  const int d = blockIdx.y;
  const uint4* s = src + static_cast<long long>(d) * bytes16;
  uint4* o = reinterpret_cast<uint4*>(dst.buf[d]) + buf_off16 + static_cast<long long>(rank) * slot16;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < bytes16;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    o[i] = s[i];
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(done_counter, 1u) == gridDim.x * gridDim.y - 1) ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < R) {
      volatile int* f = reinterpret_cast<int*>(flags.buf[threadIdx.x]) + kind * R + rank;
      *f = epoch;
    }
    if (threadIdx.x == 0) *done_counter = 0;
  }
}

// Receive side: wait for every sender's data flag, copy the R slots of this rank's own buffer into
// the (contiguous) output, then tell every peer that the buffer has been consumed.
__global__ void __launch_bounds__(256)
a2a_recv_kernel(const uint4* __restrict__ local, uint4* __restrict__ out, EpPeers flags, const int* __restrict__ my_flags,
                long long bytes16, long long slot16, unsigned* __restrict__ done_counter, int rank, int R, int kind_data,
                int kind_consumed, int epoch, int* status) {
  if (!ep_wait_all(my_flags + kind_data * R, R, epoch, status)) return;
  const int sblk = blockIdx.y;
  const uint4* s = local + static_cast<long long>(sblk) * slot16;
  uint4* o = out + static_cast<long long>(sblk) * bytes16;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < bytes16;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    o[i] = s[i];
  __syncthreads();
  __shared__ unsigned s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(done_counter, 1u) == gridDim.x * gridDim.y - 1) ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < R) {
      volatile int* f = reinterpret_cast<int*>(flags.buf[threadIdx.x]) + kind_consumed * R + rank;
      *f = epoch;
    }
    if (threadIdx.x == 0) *done_counter = 0;
  }
}

// One CTA per token: out[t] = sum_j w[t, j] * row(owner(t, j), pos[t, j]); w == nullptr -> 1.
// dw (optional): dw[t, j] = <row(t, j), g[t]>.
__global__ void __launch_bounds__(256)
ep_pull_kernel(EpPeers src, const int* __restrict__ topk_idx, const int* __restrict__ pos, const float* __restrict__ w,
               const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ out, float* __restrict__ dw,
               const int* __restrict__ flags_kind, int T, int k, int H, int El, int R, int epoch, int* status) {
  if (!ep_wait_all(flags_kind, R, epoch, status)) return;
  __shared__ float s_red[8];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    // thread i handles 8 consecutive features (H <= 2048 per pass of 256 threads)
    for (int c0 = 0; c0 < H; c0 += blockDim.x * 8) {
      const int c = c0 + threadIdx.x * 8;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        const int pr = t * k + j;
        const int d = topk_idx[pr] / El;
        const float wj = w ? w[pr] : 1.f;
        if (c < H) {
          const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src.buf[d]) +
                                                          static_cast<long long>(pos[pr]) * H + c);
          const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), dd = unpack_bf16(v.w);
          acc[0] += wj * a.x; acc[1] += wj * a.y; acc[2] += wj * b.x; acc[3] += wj * b.y;
          acc[4] += wj * cc.x; acc[5] += wj * cc.y; acc[6] += wj * dd.x; acc[7] += wj * dd.y;
        }
      }
      if (out && c < H) {
        uint4 o;
        o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
        o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H + c) = o;
      }
    }
    if (dw) {
      for (int j = 0; j < k; ++j) {
        const int pr = t * k + j;
        const int d = topk_idx[pr] / El;
        float part = 0.f;
        for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
          const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src.buf[d]) +
                                                          static_cast<long long>(pos[pr]) * H + c);
          const uint4 gv = *reinterpret_cast<const uint4*>(g + static_cast<long long>(t) * H + c);
          const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), dd = unpack_bf16(v.w);
          const float2 ga = unpack_bf16(gv.x), gb = unpack_bf16(gv.y), gc = unpack_bf16(gv.z), gd = unpack_bf16(gv.w);
          part += a.x * ga.x + a.y * ga.y + b.x * gb.x + b.y * gb.y + cc.x * gc.x + cc.y * gc.y + dd.x * gd.x +
                  dd.y * gd.y;
        }
        part = warp_sum(part);
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = part;
        __syncthreads();
        if (threadIdx.x == 0) {
          float s = 0.f;
          for (int i = 0; i < (blockDim.x >> 5); ++i) s += s_red[i];
          dw[pr] = s;
        }
        __syncthreads();
      }
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Tensor-parallel decode: all-reduce + residual add + RMSNorm in one kernel.
//
// Every rank has written its partial sums (bf16 [rows, cols]) into its own symmetric buffer with the
// GEMM that precedes this kernel on the stream. The kernel then
//   1. tells every peer "my partial of call e is complete" (CTA 0: release store into the peer's
//      flag slot [rank]) and waits, with a bound, until all peers have said the same,
//   2. reads the R partials of its rows with plain peer loads (always in rank order, so that all
//      ranks get bit-identical sums), adds the residual stream and writes the new residual,
//   3. normalises the row (RMSNorm with the weight of the NEXT norm layer) and writes that too.
// The call number e lives in device memory (state[0], advanced by the last CTA), so a CUDA graph can
// replay the launch with unchanged arguments. The caller alternates between two partial buffers:
// a rank only reaches the barrier of call e + 1 after its reads of call e have finished, so a
// buffer is never overwritten (by the GEMM of call e + 2) while a peer still reads it.
//
// Same role as the custom all-reduce + fused add-RMSNorm passes of the serving engine the reference
// drives (vLLM tensor parallelism, packages/prime-rl-configs/src/prime_rl/configs/inference.py:88-97).

__device__ __forceinline__ void ar_accumulate(float (&acc)[8], const uint4& u) {
  const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
}

// MAXVEC 16-byte vectors per thread, kArThreads threads per row (cols <= MAXVEC * kArThreads * 8). Hidden sizes up to
// 2048 run with 128 threads x 2 vectors: small CTAs, so that many rows are in flight per SM to hide the peer-load
// latency; wider rows use 256 threads x 4.
template <int MAXVEC, int kArThreads>
__global__ void __launch_bounds__(kArThreads)
ar_add_rmsnorm_kernel(EpPeers partial, EpPeers flags, int* __restrict__ state, const __nv_bfloat16* __restrict__ residual,
                      const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out_h,
                      __nv_bfloat16* __restrict__ out_x, int rows, int cols, float eps, int rank, int R, int* status) {
  const int e = *reinterpret_cast<volatile int*>(state) + 1;
  if (blockIdx.x == 0) {
    __threadfence_system();
    if (threadIdx.x < R) {
      volatile int* f = reinterpret_cast<int*>(flags.buf[threadIdx.x]) + rank;
      *f = e;
    }
  }
  const bool ok = ep_wait_all(reinterpret_cast<const int*>(flags.buf[rank]), R, e, status);
  __shared__ float s_part[kArThreads / 32];
  const int nvec = cols / 8;
  if (ok) {
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      const long long base = static_cast<long long>(row) * cols;
      float acc[MAXVEC][8];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < MAXVEC; ++i) {
        const int v = threadIdx.x + i * kArThreads;
        if (v >= nvec) break;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
        // all loads of a group of four ranks are issued before the first add; the adds keep the rank order,
        // so every rank computes bit-identical sums
        uint4 rv = make_uint4(0u, 0u, 0u, 0u);
        if (residual != nullptr) rv = *(reinterpret_cast<const uint4*>(residual + base) + v);
        for (int r0 = 0; r0 < R; r0 += 4) {
          uint4 pv[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (r0 + j < R)
              pv[j] = __ldcv(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(partial.buf[r0 + j]) + base) + v);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (r0 + j < R) ar_accumulate(acc[i], pv[j]);
        }
        if (residual != nullptr) ar_accumulate(acc[i], rv);
        // the residual stream is stored in bf16: normalise what the next layer will read
        uint4 o;
        o.x = pack_bf16(acc[i][0], acc[i][1]); o.y = pack_bf16(acc[i][2], acc[i][3]);
        o.z = pack_bf16(acc[i][4], acc[i][5]); o.w = pack_bf16(acc[i][6], acc[i][7]);
        *(reinterpret_cast<uint4*>(out_h + base) + v) = o;
        const float2 a = unpack_bf16(o.x), b = unpack_bf16(o.y), c = unpack_bf16(o.z), d = unpack_bf16(o.w);
        acc[i][0] = a.x; acc[i][1] = a.y; acc[i][2] = b.x; acc[i][3] = b.y;
        acc[i][4] = c.x; acc[i][5] = c.y; acc[i][6] = d.x; acc[i][7] = d.y;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(acc[i][j], acc[i][j], ss);
      }
      if (out_x != nullptr) {
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int k = 0; k < kArThreads / 32; ++k) tot += s_part[k];
        __syncthreads();
        const float rstd = rsqrtf(tot / static_cast<float>(cols) + eps);
#pragma unroll
        for (int i = 0; i < MAXVEC; ++i) {
          const int v = threadIdx.x + i * kArThreads;
          if (v >= nvec) break;
          const uint4 wu = *(reinterpret_cast<const uint4*>(w) + v);
          const float2 a = unpack_bf16(wu.x), b = unpack_bf16(wu.y), c = unpack_bf16(wu.z), d = unpack_bf16(wu.w);
          uint4 o;
          o.x = pack_bf16(acc[i][0] * rstd * a.x, acc[i][1] * rstd * a.y);
          o.y = pack_bf16(acc[i][2] * rstd * b.x, acc[i][3] * rstd * b.y);
          o.z = pack_bf16(acc[i][4] * rstd * c.x, acc[i][5] * rstd * c.y);
          o.w = pack_bf16(acc[i][6] * rstd * d.x, acc[i][7] * rstd * d.y);
          *(reinterpret_cast<uint4*>(out_x + base) + v) = o;
        }
      }
    }
  }
  // the last CTA to finish advances the call number for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(state + 1, 1);
    if (prev == static_cast<int>(gridDim.x) - 1) {
      state[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(state) = e;
    }
  }
}

}  // namespace prb

// ---------------------------------------------------------------- symmetric memory (CUDA IPC)
PRB_API int prb_symm_alloc(long long bytes, void** out) {
  return cudaMalloc(out, static_cast<size_t>(bytes)) == cudaSuccess ? 0 : -1;
}
PRB_API int prb_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }
PRB_API int prb_symm_memset(void* p, int v, long long bytes, void* stream) {
  return cudaMemsetAsync(p, v, static_cast<size_t>(bytes), reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : -1;
}
// handle: 64 bytes
PRB_API int prb_symm_export(void* p, void* handle) {
  return cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle), p) == cudaSuccess ? 0 : -1;
}
PRB_API int prb_symm_import(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : -1;
}
PRB_API int prb_symm_unmap(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }

// ---------------------------------------------------------------- launches
// `peers` arrays hold R device pointers (own pointer at index rank).
static prb::EpPeers ep_peers(void* const* p, int R) {
  prb::EpPeers o;
  for (int i = 0; i < prb::kEpMaxRanks; ++i) o.buf[i] = i < R ? p[i] : nullptr;
  return o;
}

PRB_API int prb_ep_hist(const int* counts, void* const* hist_peers, void* const* flag_peers, int rank, int R, int E,
                        int kind, int epoch, void* stream) {
  if (R > prb::kEpMaxRanks || E > 1024 || E % R) return -2;
  prb::ep_hist_kernel<<<1, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(counts, ep_peers(hist_peers, R),
                                                                           ep_peers(flag_peers, R), rank, R, E, kind, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_ep_plan(const int* hist, const int* flags, int rank, int R, int E, int kind, int epoch, int cap_rows,
                        int max_blocks, int* send_base, int* expert_offset, int* block_expert, int* total_rows,
                        int* status, void* stream) {
  if (R > prb::kEpMaxRanks || E > 1024 || E % R) return -2;
  prb::ep_plan_kernel<<<1, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      hist, flags + kind * R, rank, R, E, epoch, cap_rows, max_blocks, send_base, expert_offset, block_expert, total_rows,
      status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_ep_push(const void* x, const int* topk_idx, const int* slot, const int* local_off,
                        const int* send_base, const int* pos_in, const float* scale, void* const* dst_peers,
                        void* const* flag_peers, int* pos_out, unsigned* done_counter, int num_pairs, int k, int H,
                        int E, int rank, int R, int kind, int epoch, int cap_rows, int* status, void* stream) {
  if (R > prb::kEpMaxRanks || (H % 8) || E % R) return -2;
  if (num_pairs <= 0) {
    prb::ep_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(ep_peers(flag_peers, R), rank, R, kind, epoch);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }
  int grid = (num_pairs + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  prb::ep_push_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), topk_idx, slot, local_off, send_base, pos_in, scale,
      ep_peers(dst_peers, R), ep_peers(flag_peers, R), pos_out, done_counter, num_pairs, k, H, E / R, rank, R, kind, epoch,
      cap_rows, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Per-block dispatch (see ep_prepare_kernel / ep_push_blocks_kernel). cnt_peers: the arrival counters inside the
// symmetric buffers; cnt_off: byte offset of the parity in use. The push may run on a stream of its own.
PRB_API int prb_ep_prepare(void* buf, const int* hist, const int* expert_offset, int* block_rows, void* zero_cnt,
                           int max_blocks, int rank, int R, int E, int H, void* stream) {
  if (R > prb::kEpMaxRanks || (H % 8) || E % R) return -2;
  prb::ep_prepare_kernel<<<E / R, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(buf), hist, expert_offset, block_rows, reinterpret_cast<unsigned*>(zero_cnt),
      max_blocks, rank, R, E, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_ep_push_blocks(const void* x, const int* row_src, const int* local_block_expert, const int* local_off,
                               const int* local_total, const int* counts, const int* send_base,
                               void* const* dst_peers, void* const* cnt_peers, long long cnt_off, int* pos_out,
                               int max_local_blocks, int k, int H, int E, int rank, int R, int cap_rows, int* status,
                               void* stream) {
  if (R > prb::kEpMaxRanks || (H % 8) || E % R || (cnt_off % 4)) return -2;
  if (max_local_blocks <= 0) return 0;
  const int grid = max_local_blocks < 148 * 4 ? max_local_blocks : 148 * 4;
  prb::ep_push_blocks_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), row_src, local_block_expert, local_off, local_total, counts, send_base,
      ep_peers(dst_peers, R), ep_peers(cnt_peers, R), cnt_off, pos_out, k, H, E / R, rank, R, cap_rows, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_ep_recv(void* buf, const int* hist, const int* expert_offset, const int* flags, int rank, int R, int E,
                        int H, int kind, int epoch, int* status, void* stream) {
  prb::ep_recv_kernel<<<E / R, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(buf), hist, expert_offset, flags + kind * R, rank, R, E, H, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// fp8 payload variants (H must be a multiple of 128).
PRB_API int prb_ep_push_fp8(const void* x, const int* topk_idx, const int* slot, const int* local_off,
                            const int* send_base, const int* pos_in, const float* scale, void* const* q_peers,
                            void* const* s_peers, void* const* flag_peers, int* pos_out, unsigned* done_counter,
                            int num_pairs, int k, int H, int E, int rank, int R, int kind, int epoch, int cap_rows,
                            int* status, void* stream) {
  if (R > prb::kEpMaxRanks || (H % 128) || E % R) return -2;
  if (num_pairs <= 0) {
    prb::ep_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(ep_peers(flag_peers, R), rank, R, kind, epoch);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }
  int grid = (num_pairs + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  prb::ep_push_fp8_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), topk_idx, slot, local_off, send_base, pos_in, scale,
      ep_peers(q_peers, R), ep_peers(s_peers, R), ep_peers(flag_peers, R), pos_out, done_counter, num_pairs, k, H, E / R,
      rank, R, kind, epoch, cap_rows, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_ep_recv_fp8(void* buf, const void* q, const float* scales, const int* hist, const int* expert_offset,
                            const int* flags, int rank, int R, int E, int H, int kind, int epoch, int* status,
                            void* stream) {
  if ((H % 128) || E % R) return -2;
  dim3 grid(E / R, 32);
  prb::ep_recv_fp8_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(buf), reinterpret_cast<const uint8_t*>(q), scales, hist, expert_offset,
      flags + kind * R, rank, R, E, H, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// out[i] = scale * sum_r peer_grads[r][off + i], i in [0, n); fp32; off and n multiples of 4.
PRB_API int prb_rs_pull(void* const* peer_grads, long long off, long long n, float scale, float* out, int R,
                        void* stream) {
  if (R > prb::kEpMaxRanks || (off % 4) || (n % 4) || (reinterpret_cast<uintptr_t>(out) & 15)) return -2;
  if (n <= 0) return 0;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  prb::rs_pull_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ep_peers(peer_grads, R), off, n / 4, scale, reinterpret_cast<float4*>(out), R);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Writes `bytes` bytes at `src` (this rank's slice, inside its own buffer at byte offset off_bytes) to
// the same offset of every other rank's buffer.
PRB_API int prb_ag_push(const void* src, void* const* peer_bufs, long long off_bytes, long long bytes, int rank, int R,
                        void* stream) {
  if (R > prb::kEpMaxRanks || (off_bytes % 16) || (bytes % 16) || (reinterpret_cast<uintptr_t>(src) & 15)) return -2;
  if (bytes <= 0 || R < 2) return 0;
  long long blocks = (bytes / 16 + 255) / 256;
  if (blocks > 148 * 2) blocks = 148 * 2;
  prb::ag_push_kernel<<<dim3(static_cast<unsigned>(blocks), R - 1), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(src), ep_peers(peer_bufs, R), off_bytes / 16, bytes / 16, rank, R);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// dst (local, 16-byte aligned) <- src (a peer's or local memory), bytes a multiple of 16; at most `max_ctas` CTAs.
PRB_API int prb_peer_copy(const void* src, void* dst, long long bytes, int max_ctas, void* stream) {
  if ((bytes % 16) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -2;
  if (bytes <= 0) return 0;
  long long blocks = (bytes / 16 + 255) / 256;
  if (max_ctas < 1) max_ctas = 1;
  if (blocks > max_ctas) blocks = max_ctas;
  prb::peer_copy_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// out[i] = sum_r bf16(peer_bufs[r] + slot_off_bytes)[i], i in [0, n): n bf16 elements, a multiple of 8.
PRB_API int prb_slot_pull_reduce(void* const* peer_bufs, long long slot_off_bytes, long long n, void* out, int R,
                                 void* stream) {
  if (R > prb::kEpMaxRanks || (slot_off_bytes % 16) || (n % 8) || (reinterpret_cast<uintptr_t>(out) & 15)) return -2;
  if (n <= 0) return 0;
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  prb::slot_pull_reduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ep_peers(peer_bufs, R), slot_off_bytes / 16, n / 8, reinterpret_cast<uint4*>(out), R);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_ep_signal(void* const* flag_peers, int rank, int R, int kind, int epoch, void* stream) {
  prb::ep_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(ep_peers(flag_peers, R), rank, R, kind, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_ep_wait(const int* flags, int R, int kind, int epoch, int* status, void* stream) {
  prb::ep_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flags + kind * R, R, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// src: R blocks of `bytes` each (multiple of 16); every peer buffer: [2 buffers][R slots of slot_bytes].
PRB_API int prb_a2a_push(const void* src, void* const* buf_peers, void* const* flag_peers, long long bytes,
                         long long slot_bytes, long long buf_off_bytes, unsigned* done_counter, int rank, int R,
                         int kind, int epoch, void* stream) {
  if (R > prb::kEpMaxRanks || (bytes % 16) || (slot_bytes % 16) || (buf_off_bytes % 16)) return -2;
  long long per = (bytes / 16 + 255) / 256;
  int gx = static_cast<int>(per < 1 ? 1 : (per > 148 ? 148 : per));
  prb::a2a_push_kernel<<<dim3(gx, R), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(src), ep_peers(buf_peers, R), ep_peers(flag_peers, R), bytes / 16, slot_bytes / 16,
      buf_off_bytes / 16, done_counter, rank, R, kind, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_a2a_recv(const void* local, void* out, void* const* flag_peers, const int* my_flags, long long bytes,
                         long long slot_bytes, unsigned* done_counter, int rank, int R, int kind_data,
                         int kind_consumed, int epoch, int* status, void* stream) {
  if (R > prb::kEpMaxRanks || (bytes % 16) || (slot_bytes % 16)) return -2;
  long long per = (bytes / 16 + 255) / 256;
  int gx = static_cast<int>(per < 1 ? 1 : (per > 148 ? 148 : per));
  prb::a2a_recv_kernel<<<dim3(gx, R), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(local), reinterpret_cast<uint4*>(out), ep_peers(flag_peers, R), my_flags, bytes / 16,
      slot_bytes / 16, done_counter, rank, R, kind_data, kind_consumed, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_ep_pull(void* const* src_peers, const int* topk_idx, const int* pos, const float* w, const void* g,
                        void* out, float* dw, const int* flags, int T, int k, int H, int E, int R, int kind, int epoch,
                        int* status, void* stream) {
  if (R > prb::kEpMaxRanks || (H % 8) || E % R) return -2;
  if (T <= 0) return 0;
  int grid = T < 148 * 8 ? T : 148 * 8;
  prb::ep_pull_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ep_peers(src_peers, R), topk_idx, pos, w, reinterpret_cast<const __nv_bfloat16*>(g),
      reinterpret_cast<__nv_bfloat16*>(out), dw, flags + kind * R, T, k, H, E / R, R, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// partial_peers: every rank's partial buffer for THIS call (bf16 [rows, cols]); flag_peers: int32 [R] on every
// rank; state: int32 [2] local (call number, CTA counter), zero before the first call. residual / w / out_x may
// be null (no residual add / no norm output). out_h gets the reduced (+ residual) rows.
PRB_API int prb_ar_add_rmsnorm(void* const* partial_peers, void* const* flag_peers, int* state, const void* residual,
                               const void* w, void* out_h, void* out_x, int rows, int cols, float eps, int rank, int R,
                               int* status, void* stream) {
  if (R > prb::kEpMaxRanks || R < 1 || cols % 8 || cols > 4 * 256 * 8) return -2;
  if (out_x != nullptr && w == nullptr) return -2;
  if (rows <= 0) return 0;
  const bool narrow = cols <= 2 * 128 * 8;
  const int cap = 148 * (narrow ? 12 : 3);
  const int grid = rows < cap ? rows : cap;
#define PRB_AR_LAUNCH(MV, TH)                                                                                        \
  prb::ar_add_rmsnorm_kernel<MV, TH><<<grid, TH, 0, reinterpret_cast<cudaStream_t>(stream)>>>(                       \
      ep_peers(partial_peers, R), ep_peers(flag_peers, R), state, reinterpret_cast<const __nv_bfloat16*>(residual),  \
      reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(out_h),                            \
      reinterpret_cast<__nv_bfloat16*>(out_x), rows, cols, eps, rank, R, status)
  if (narrow) PRB_AR_LAUNCH(2, 128); else PRB_AR_LAUNCH(4, 256);
#undef PRB_AR_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
