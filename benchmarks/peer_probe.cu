// Link probe: how fast can SM-issued loads / stores move bytes between this GPU and a peer
// (or this GPU's own memory)?  The fused sparse and dense kernels move their data exactly
// this way, so these figures are the denominators of their NVLink rooflines.
// No counterpart in the reference (its transport is brpc over TCP).
// Built on demand by p2p_microbench.py as a small extension of its own (it is a measuring tool,
// not part of the library).
#include <cuda_runtime.h>
#include <torch/extension.h>
#include <c10/cuda/CUDAStream.h>

namespace {

// mode 0: dst[i] = src[i], one 16-byte element per thread per iteration (grid-stride)
// mode 1: same with four independent elements in flight per thread
// mode 2: dst[i] = value (no load): pure store stream
// mode 3: dst[i] = src[i]; src[i] = 0
// A trailing system-scope fence by every thread makes the kernel time include the write drain.
__global__ void __launch_bounds__(1024, 1) peer_copy_kernel(float4* __restrict__ dst, const float4* __restrict__ src, long long n16,
                                                            int mode, int fence) {
  const long long nth = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (mode == 0) {
    for (long long i = tid; i < n16; i += nth) dst[i] = __ldcg(&src[i]);
  } else if (mode == 1) {
    for (long long base = tid; base < n16; base += 4 * nth) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) if (base + u * nth < n16) v[u] = __ldcg(&src[base + u * nth]);
#pragma unroll
      for (int u = 0; u < 4; ++u) if (base + u * nth < n16) dst[base + u * nth] = v[u];
    }
  } else if (mode == 2) {
    const float4 v = make_float4(1.f, 2.f, 3.f, 4.f);
    for (long long i = tid; i < n16; i += nth) dst[i] = v;
  } else {
    // mode 3: move-and-clear (the source is zeroed behind the copy, as the gradient shipping does)
    float4* s = const_cast<float4*>(src);
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long i = tid; i < n16; i += nth) { dst[i] = s[i]; s[i] = z; }
  }
  if (fence) __threadfence_system();
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("peer_copy", [](int64_t dst, int64_t src, int64_t nbytes, int mode, int blocks, int threads, bool fence) {
    TORCH_CHECK(nbytes % 16 == 0 && dst % 16 == 0 && src % 16 == 0, "peer_copy wants 16-byte aligned pointers and size");
    TORCH_CHECK(threads >= 32 && threads <= 1024 && blocks >= 1, "bad launch shape");
    peer_copy_kernel<<<blocks, threads, 0, c10::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<float4*>(dst), reinterpret_cast<const float4*>(src), nbytes / 16, mode, fence ? 1 : 0);
  }, "SM-issued copy between raw (possibly peer) addresses; link bandwidth probe");
}
