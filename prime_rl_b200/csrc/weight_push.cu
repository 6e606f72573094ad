// Trainer -> engine weight push over NVLink peer memory. The engine process exports its
// parameter storage with CUDA IPC; the trainer maps it and writes the new values straight
// into place, either as they are (bf16 -> bf16) or quantised on the way to block-scaled fp8
// (e4m3 payload, one fp32 scale per 128 x 128 weight block: scale = amax / 448, the layout of
// the reference's fp8 checkpoints, src/prime_rl/trainer/models/fp8.py). One kernel per tensor:
// read local HBM once, store to the peer once; no staging copy on either side and no library
// kernel touches peer memory.
//
// Takes the place of the layer-wise NCCL broadcast (src/prime_rl/transports/weights/nccl.py)
// and of the filesystem round trip for engines on the same NVSwitch box.
#include "common.cuh"
#include <cuda_fp8.h>

namespace prb {

__global__ void __launch_bounds__(256)
weight_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16, const uint8_t* src_tail,
                   uint8_t* dst_tail, int tail) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
  if (blockIdx.x == 0 && threadIdx.x < tail) dst_tail[threadIdx.x] = src_tail[threadIdx.x];
}

// One CTA per 128 x 128 block of W [N, K] (bf16, row pitch ld). q: e4m3 [N, K] (pitch K),
// scales: fp32 [ceil(N/128), ceil(K/128)]; dequantised value = q * scale.
__global__ void __launch_bounds__(256)
weight_quant_push_kernel(const __nv_bfloat16* __restrict__ w, long long ld, uint8_t* __restrict__ q,
                         float* __restrict__ scales, int N, int K) {
  const int bn = blockIdx.y, bk = blockIdx.x;
  const int r0 = bn * 128, c0 = bk * 128;
  __shared__ float s_red[8];
  __shared__ float s_scale;
  // thread t: row r0 + t / 2, 64 columns starting at c0 + 64 * (t & 1)
  const int r = r0 + (threadIdx.x >> 1), cb = c0 + 64 * (threadIdx.x & 1);
  float v[64];
  float amax = 0.f;
  const bool fast = (r < N) && (cb + 64 <= K) && (ld % 8 == 0) && (K % 16 == 0) &&
                    ((reinterpret_cast<uintptr_t>(w) & 15) == 0) && ((reinterpret_cast<uintptr_t>(q) & 15) == 0);
  if (fast) {
    const uint4* src = reinterpret_cast<const uint4*>(w + static_cast<long long>(r) * ld + cb);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint4 u = src[j];
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
      v[8 * j + 0] = a.x; v[8 * j + 1] = a.y; v[8 * j + 2] = b.x; v[8 * j + 3] = b.y;
      v[8 * j + 4] = c.x; v[8 * j + 5] = c.y; v[8 * j + 6] = d.x; v[8 * j + 7] = d.y;
    }
#pragma unroll
    for (int j = 0; j < 64; ++j) amax = fmaxf(amax, fabsf(v[j]));
  } else {
#pragma unroll
    for (int j = 0; j < 64; ++j) {
      const int c = cb + j;
      v[j] = (r < N && c < K) ? __bfloat162float(w[static_cast<long long>(r) * ld + c]) : 0.f;
      amax = fmaxf(amax, fabsf(v[j]));
    }
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < 8; ++i) m = fmaxf(m, s_red[i]);
    const float sc = fmaxf(m, 1e-12f) / 448.f;
    s_scale = sc;
    scales[static_cast<long long>(bn) * gridDim.x + bk] = sc;
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
  if (fast) {
    uint4* dst = reinterpret_cast<uint4*>(q + static_cast<long long>(r) * K + cb);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int b = 16 * j + 4 * i;
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[b] * inv, v[b + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[b + 2] * inv, v[b + 3] * inv), __NV_SATFINITE, __NV_E4M3);
        o[i] = lo | (hi << 16);
      }
      dst[j] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else if (r < N) {
#pragma unroll
    for (int j = 0; j < 64; j += 2) {
      const int c = cb + j;
      const __nv_fp8x2_storage_t p = __nv_cvt_float2_to_fp8x2(make_float2(v[j] * inv, v[j + 1] * inv), __NV_SATFINITE,
                                                               __NV_E4M3);
      if (c + 1 < K) {
        *reinterpret_cast<__nv_fp8x2_storage_t*>(q + static_cast<long long>(r) * K + c) = p;
      } else if (c < K) {
        q[static_cast<long long>(r) * K + c] = static_cast<uint8_t>(p & 0xff);
      }
    }
  }
}

}  // namespace prb

// handle (64 bytes) and byte offset of `p` inside its allocation: a tensor of a caching
// allocator is a slice of a larger cudaMalloc block, and IPC handles name whole blocks.
PRB_API int prb_ipc_export_range(void* p, void* handle, long long* offset) {
  typedef CUresult (*GetRange)(CUdeviceptr*, size_t*, CUdeviceptr);
  static GetRange fn = nullptr;
  if (!fn) {
    cudaDriverEntryPointQueryResult qres;
    void* sym = nullptr;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &qres) != cudaSuccess || !sym)
      return -1;
    fn = reinterpret_cast<GetRange>(sym);
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  if (fn(&base, &size, reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS) return -2;
  if (cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle), reinterpret_cast<void*>(base)) != cudaSuccess)
    return -3;
  *offset = static_cast<long long>(reinterpret_cast<CUdeviceptr>(p) - base);
  return 0;
}

PRB_API int prb_weight_push(const void* src, void* dst, long long bytes, void* stream) {
  if (bytes <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -4;
  const long long n16 = bytes / 16;
  const int tail = static_cast<int>(bytes - n16 * 16);
  long long grid = (n16 + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  if (grid < 1) grid = 1;
  prb::weight_copy_kernel<<<static_cast<unsigned>(grid), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), n16,
      reinterpret_cast<const uint8_t*>(src) + n16 * 16, reinterpret_cast<uint8_t*>(dst) + n16 * 16, tail);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

PRB_API int prb_weight_push_fp8(const void* w, long long ld, void* q, float* scales, int N, int K, void* stream) {
  if (N <= 0 || K <= 0) return 0;
  if (K % 2) return -4;
  dim3 grid((K + 127) / 128, (N + 127) / 128);
  prb::weight_quant_push_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(w), ld, reinterpret_cast<uint8_t*>(q), scales, N, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
