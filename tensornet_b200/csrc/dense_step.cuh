// Device code of the multi-GPU dense step, shared by the stand-alone dense kernel (dense_fused.cu) and by the sparse
// push kernel (sparse_fused.cu), which can carry the dense step of a small parameter array on a few CTAs of its own
// grid so that the two exchanges of a training step overlap instead of running back to back.
//
// What it replaces in the reference: DenseTablePushPull RPCs (core/kernels/dense_table_ops.cc:130-252), the per-shard
// optimizer (core/ps/optimizer/adam_kernel.cc:46-55, ada_grad_kernel.cc:42-48) and the copy back into the framework
// variables (dense_table_ops.cc:199-244).
#pragma once
#include <cuda_bf16.h>
#include "tn_device.cuh"
#include "tn_types.h"

namespace tn {
namespace dense {


__device__ __forceinline__ void adam4(const DenseOptParams& o, float alpha, float4 g, float4& w, float4& m, float4& v) {
#define TN_ADAM1(c) \
  m.c += (g.c - m.c) * (1.f - o.beta1); \
  v.c += (g.c * g.c - v.c) * (1.f - o.beta2); \
  w.c -= m.c * alpha / (sqrtf(v.c) + o.eps);
  TN_ADAM1(x) TN_ADAM1(y) TN_ADAM1(z) TN_ADAM1(w)
#undef TN_ADAM1
}
// Dense AdaGrad: state s0 = d2sum, s1 = g2sum, s2 = m.
__device__ __forceinline__ void adagrad4(const DenseOptParams& o, float lr, float4 g, float4& w, float4& d2, float4& g2, float4& m) {
#define TN_ADAG1(c) \
  d2.c = o.grad_decay * d2.c + 1.f; \
  g2.c = o.grad_decay * g2.c + g.c * g.c; \
  m.c += (g.c - m.c) * (1.f - o.mom_decay); \
  w.c -= lr * m.c / (sqrtf(g2.c) / sqrtf(d2.c) + o.eps);
  TN_ADAG1(x) TN_ADAG1(y) TN_ADAG1(z) TN_ADAG1(w)
#undef TN_ADAG1
}

__device__ __forceinline__ uint2 f4_to_bf16x4(float4 w) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
  return make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

__device__ __forceinline__ float4 mm_ld_reduce_f4(const float* mc) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(mc) : "memory");
  return r;
}
__device__ __forceinline__ void mm_st_f4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void mm_st_b32x2(void* mc, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.bf16x2 [%0], {%1,%2};" ::"l"(mc), "r"(v.x), "r"(v.y) : "memory");
}

// The running beta powers live in device memory (state[0], state[1]); state[2] is the
// learning rate, state[3] (as unsigned) a ticket counter.  Every thread derives this step's
// powers from the stored ones; the last CTA to finish stores them back.
__device__ __forceinline__ void finish_step(const DenseOptParams& o, float b1p, float b2p) {
  __shared__ bool s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    unsigned t = atomicAdd(reinterpret_cast<unsigned*>(o.state) + 3, 1u);
    s_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    o.state[0] = b1p;
    o.state[1] = b2p;
    reinterpret_cast<unsigned*>(o.state)[3] = 0u;
  }
}

// Cross-GPU barrier run by CTA 0 (threads < world), then released to the grid by the caller's
// grid barrier.  flags: [2][kMaxWorld] words per GPU; `which` selects the row.
__device__ __forceinline__ bool peer_barrier(const DenseStepArgs& a, int which, unsigned long long epoch, int phase, int bid) {
  bool ok = true;
  if (bid == 0 && threadIdx.x < a.world) {
    const int p = threadIdx.x;
    if (p != a.rank) {
      st_release_sys_u64(a.sig[p] + which * kMaxWorld + a.rank, epoch << 32);
      unsigned long long v;
      ok = wait_flag_ge(a.sig[a.rank] + which * kMaxWorld + p, epoch, &v, a.wait_ns, a.status, phase, p);
    }
  }
  return ok;
}

// Optimizer update of one 4-element group of the owned chunk: reduced gradient in, new weight out.
__device__ __forceinline__ float4 dense_update4(const DenseStepArgs& a, float alpha, float lr, float4 g, long long i, long long li) {
  const DenseOptParams& o = a.opt;
  g.x *= a.grad_scale; g.y *= a.grad_scale; g.z *= a.grad_scale; g.w *= a.grad_scale;
  float4 w = reinterpret_cast<float4*>(a.W[a.rank])[i];
  float4 s0 = reinterpret_cast<float4*>(a.s0)[li], s1 = reinterpret_cast<float4*>(a.s1)[li];   // state is indexed within the chunk
  if (o.kind == 0) {
    adam4(o, alpha, g, w, s0, s1);
  } else {
    float4 s2 = reinterpret_cast<float4*>(a.s2)[li];
    adagrad4(o, lr, g, w, s0, s1, s2);
    reinterpret_cast<float4*>(a.s2)[li] = s2;
  }
  reinterpret_cast<float4*>(a.s0)[li] = s0;
  reinterpret_cast<float4*>(a.s1)[li] = s1;
  return w;
}

constexpr int kDenseUnroll = 4;   // independent 16-byte reductions in flight per thread (NVLink round trips overlap)

// The whole multi-GPU step as seen by CTA `bid` of the `nb` CTAs that share the work (their own barrier words in
// a.bar).  Every CTA of the group must call it; returns after the group's exit bookkeeping.
template <int kUnroll>
__device__ __forceinline__ void fused_step(const DenseStepArgs& a, const int bid, const int nb) {
  const DenseOptParams& o = a.opt;
  GridSync gs;
  gs.init(a.bar, a.status, a.wait_ns, (unsigned)nb);
  const float b1p = __ldcg(&o.state[0]) * o.beta1, b2p = __ldcg(&o.state[1]) * o.beta2;
  const float lr = __ldcg(&o.state[2]);
  const float alpha = lr * sqrtf(1.f - b2p) / (1.f - b1p);
  const unsigned long long epoch = __ldcg(a.epoch) + 1ull;
  const int W = a.world, R = a.rank;
  const long long chunk4 = a.chunk >> 2;
  const long long lo4 = (long long)R * chunk4;
  long long hi4 = lo4 + chunk4;
  const long long n4 = a.n >> 2;
  if (hi4 > n4) hi4 = n4;
  const long long nth = (long long)nb * blockDim.x;
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
  // Re-zeroing the gradient replicas through the switch costs as much NVLink ingress as the fp32 weights;
  // large arrays are zeroed by their own GPU instead, once every peer has finished reading them.
  const bool zero_remote = !a.zero_local;

  // all GPUs have finished writing their gradients: stream order on each GPU + this barrier.  The caller may skip
  // it when a kernel that ran just before on this stream already waited for every peer to get past its backward
  // pass (the multi-GPU sparse push does: a peer ships its gradient records only after its own backward).
  if (!a.skip_open) {
    peer_barrier(a, 0, epoch, 41, bid);
    if (!gs.sync(42, false)) goto done;
  }

  for (long long base = lo4 + bid * (long long)blockDim.x + threadIdx.x; base < hi4; base += nth * kUnroll) {
    float4 g[kUnroll];
    if (a.G_mc) {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long i = base + u * nth;
        if (i < hi4) g[u] = mm_ld_reduce_f4(a.G_mc + 4 * i);
      }
    } else {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) g[u] = z4;
      for (int p = 0; p < W; ++p) {
        const float* Gp = a.G[(R + p) % W];
        float4 x[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const long long i = base + u * nth;
          if (i < hi4) x[u] = ldcg_f4(Gp + 4 * i);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const long long i = base + u * nth;
          if (i < hi4) { g[u].x += x[u].x; g[u].y += x[u].y; g[u].z += x[u].z; g[u].w += x[u].w; }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long i = base + u * nth;
      if (i >= hi4) continue;
      const float4 w = dense_update4(a, alpha, lr, g[u], i, i - lo4);
      const uint2 wb = f4_to_bf16x4(w);
      if (a.G_mc) {
        mm_st_f4(a.W_mc + 4 * i, w);
        if (a.Wb_mc) mm_st_b32x2(reinterpret_cast<uint2*>(a.Wb_mc) + i, wb);
        if (zero_remote) mm_st_f4(a.G_mc + 4 * i, z4);
        else reinterpret_cast<float4*>(a.G[R])[i] = z4;
      } else {
        for (int p = 0; p < W; ++p) {
          const int d = (R + p) % W;
          reinterpret_cast<float4*>(a.W[d])[i] = w;
          if (a.Wb[d]) reinterpret_cast<uint2*>(a.Wb[d])[i] = wb;
          if (zero_remote || d == R) reinterpret_cast<float4*>(a.G[d])[i] = z4;
        }
      }
    }
  }

  // every owner's chunk has landed in every replica before anyone's next forward starts
  if (!gs.sync(43, true)) goto done;
  if (a.gated && zero_remote) {
    // no closing wait: tell every GPU (this one included) that the owned chunk is in place; the consumer checks
    if (bid == 0 && threadIdx.x < W) st_release_sys_u64(a.sig[threadIdx.x] + 2 * kMaxWorld + R, epoch << 32);
  } else {
    peer_barrier(a, 1, epoch, 44, bid);
    if (a.gated && bid == 0 && threadIdx.x < W)      // keep the gate words current in this mode too
      st_release_sys_u64(a.sig[R] + 2 * kMaxWorld + threadIdx.x, epoch << 32);
  }
  if (!zero_remote) {
    // every peer has read its chunk of this GPU's gradient: clear the part this GPU does not own
    if (!gs.sync(45, false)) goto done;
    float4* Gl = reinterpret_cast<float4*>(a.G[R]);
    for (long long i = bid * (long long)blockDim.x + threadIdx.x; i < n4; i += nth)
      if (i < lo4 || i >= hi4) Gl[i] = z4;
  }
  __syncthreads();
  if (bid == 0 && threadIdx.x == 0) {
    *a.epoch = epoch;
    o.state[0] = b1p;
    o.state[1] = b2p;
  }
done:
  gs.leave();
}


}  // namespace dense
}  // namespace tn
