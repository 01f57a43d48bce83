// Dense parameter path: every dense parameter of the model lives in ONE flat fp32 array
// (plus a bf16 shadow used by the tensor-core GEMMs); the gradient is a flat array of the
// same layout.  One kernel per step does what the reference spreads over
// DenseTablePushPull RPCs (core/kernels/dense_table_ops.cc:130-252), the per-shard
// optimizer (core/ps/optimizer/adam_kernel.cc:46-55, ada_grad_kernel.cc:42-48) and the
// copy back into the framework variables (dense_table_ops.cc:199-244):
//
//   world == 1 : Adam / AdaGrad over the whole array.
//   world  > 1 : each GPU owns the contiguous chunk ceil(P/world) (dense_table.cc:46-58).
//                Inside one cooperative kernel: cross-GPU "gradients ready" barrier ->
//                reduce the owned chunk over all GPUs (NVSwitch multimem.ld_reduce when a
//                multicast mapping exists, peer loads otherwise) -> optimizer update on the
//                fp32 master + state -> write the new fp32 and bf16 weights into every
//                GPU's replica (multimem.st or peer stores) -> "weights written" barrier.
//
// The gradient array is re-zeroed by the kernel so the next backward can accumulate into it.
#include <cuda_bf16.h>
#include "dense_step.cuh"
#include "tn_ops.h"

namespace tn {

namespace {

constexpr int kDThreads = 256;

using namespace dense;

__global__ void __launch_bounds__(kDThreads) dense_local_kernel(const DenseStepArgs a) {
  const DenseOptParams& o = a.opt;
  const float b1p = __ldcg(&o.state[0]) * o.beta1, b2p = __ldcg(&o.state[1]) * o.beta2;
  const float lr = __ldcg(&o.state[2]);
  const float alpha = lr * sqrtf(1.f - b2p) / (1.f - b1p);
  const long long n4 = a.n >> 2;
  float* W = a.W[0]; float* G = a.G[0];
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 g = reinterpret_cast<float4*>(G)[i];
    g.x *= a.grad_scale; g.y *= a.grad_scale; g.z *= a.grad_scale; g.w *= a.grad_scale;
    float4 w = reinterpret_cast<float4*>(W)[i];
    float4 s0 = reinterpret_cast<float4*>(a.s0)[i], s1 = reinterpret_cast<float4*>(a.s1)[i];
    if (o.kind == 0) {
      adam4(o, alpha, g, w, s0, s1);
    } else {
      float4 s2 = reinterpret_cast<float4*>(a.s2)[i];
      adagrad4(o, lr, g, w, s0, s1, s2);
      reinterpret_cast<float4*>(a.s2)[i] = s2;
    }
    reinterpret_cast<float4*>(a.s0)[i] = s0;
    reinterpret_cast<float4*>(a.s1)[i] = s1;
    reinterpret_cast<float4*>(W)[i] = w;
    if (a.Wb[0]) reinterpret_cast<uint2*>(a.Wb[0])[i] = f4_to_bf16x4(w);
    reinterpret_cast<float4*>(G)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  finish_step(o, b1p, b2p);
}

__global__ void __launch_bounds__(kDThreads) dense_fused_kernel(const __grid_constant__ DenseStepArgs a) {
  dense::fused_step<dense::kDenseUnroll>(a, (int)blockIdx.x, (int)gridDim.x);
}

}  // namespace

int dense_step_ctas_per_sm() {
  int per_sm = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dense_fused_kernel, kDThreads, 0);
  return per_sm < 1 ? 1 : per_sm;
}

cudaError_t launch_dense_step(const DenseStepArgs& a, cudaStream_t st) {
  if (a.n % 4 || a.chunk % 4) return cudaErrorInvalidValue;
  if (a.world == 1) {
    long long n4 = a.n >> 2;
    int blocks = (int)((n4 + kDThreads - 1) / kDThreads);
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 8) blocks = 148 * 8;
    dense_local_kernel<<<blocks, kDThreads, 0, st>>>(a);
    return cudaGetLastError();
  }
  int dev = 0, per_sm = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dense_fused_kernel, kDThreads, 0);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long n4 = a.chunk >> 2;
  int blocks = (int)((n4 + kDThreads - 1) / kDThreads);
  if (blocks < 1) blocks = 1;
  blocks = (blocks + kDenseUnroll - 1) / kDenseUnroll;
  int cap = sms * (per_sm < 1 ? 1 : per_sm);      // as many warps as fit: the loop is bound by loads in flight
  if (blocks > cap) blocks = cap;
  if (a.max_ctas > 0 && blocks > a.max_ctas) blocks = a.max_ctas;
  if (blocks < 1) blocks = 1;
  void* params[] = {(void*)&a};
  return cudaLaunchCooperativeKernel((const void*)dense_fused_kernel, dim3(blocks), dim3(kDThreads), params, 0, st);
}

}  // namespace tn
