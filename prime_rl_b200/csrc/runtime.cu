// Thread/device binding for the C entry points.
//
// The library carries its own (static) CUDA runtime. PyTorch runs autograd backward on
// worker threads on which this runtime instance has not made a context current yet; driver
// entry points such as cuTensorMapEncodeTiled then fail with CUDA_ERROR_INVALID_CONTEXT.
// prb_bind_device makes the primary context of `dev` current on the calling thread (once
// per thread and device).
#include "common.cuh"

PRB_API int prb_bind_device(int dev) {
  static thread_local int bound = -1;
  if (bound == dev) return 0;
  if (cudaSetDevice(dev) != cudaSuccess) return -1;
  if (cudaFree(0) != cudaSuccess) return -2;
  bound = dev;
  return 0;
}

PRB_API int prb_sm_count() {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}
