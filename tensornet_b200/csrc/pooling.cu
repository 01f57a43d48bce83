// Bag pooling over the per-batch unique-row matrix and its backward into the unique
// gradient matrix, plus the un-pooled sequence gather.  Stands in for TensorFlow's
// safe_embedding_lookup_sparse / sequence lookups that the reference calls on its batch
// variable (tensornet/layers/embedding_features.py:283-284,
// tensornet/layers/sequence_embedding_features.py:99-137).
#include "tn_device.cuh"
#include "tn_ops.h"

namespace tn {

namespace {

__device__ __forceinline__ float bag_scale(int combiner, int len) {
  if (len <= 0) return 0.f;
  if (combiner == 1) return 1.f / (float)len;
  if (combiner == 2) return rsqrtf((float)len);
  return 1.f;
}

// One group of G lanes per bag.  Bag g = s * B + b, its ids are positions
// [offsets[g], offsets[g+1]) of `inverse` (or exactly position g when offsets == nullptr).
__global__ void pool_fwd_kernel(const float* __restrict__ U, int ustride, const int* __restrict__ inverse,
                                const int* __restrict__ offsets, int B, int S, int pd, int combiner,
                                float* __restrict__ out, int out_ld, int G) {
  pdl_sync();
  const int lane = threadIdx.x % G;
  const int gid = (blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int ngroups = (gridDim.x * blockDim.x) / G;
  const int nbags = B * S;
  for (int g = gid; g < nbags; g += ngroups) {
    const int s = g / B, b = g - s * B;
    int k0 = g, k1 = g + 1;
    if (offsets) { k0 = offsets[g]; k1 = offsets[g + 1]; }
    const float sc = bag_scale(combiner, k1 - k0);
    float* o = out + (size_t)b * out_ld + (size_t)s * pd;
    for (int d = lane; d < pd; d += G) {
      float acc = 0.f;
      for (int k = k0; k < k1; ++k) {
        int v = inverse[k];
        if (v >= 0) acc += __ldcg(U + (size_t)v * ustride + d);
      }
      o[d] = acc * sc;
    }
  }
}

// pd % 4 == 0: every lane moves float4 chunks.
__global__ void pool_fwd_vec4_kernel(const float* __restrict__ U, int ustride, const int* __restrict__ inverse,
                                     const int* __restrict__ offsets, int B, int S, int pd, int combiner,
                                     float* __restrict__ out, int out_ld, int G) {
  pdl_sync();
  const int lane = threadIdx.x % G;
  const int gid = (blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int ngroups = (gridDim.x * blockDim.x) / G;
  const int nbags = B * S, nch = pd >> 2;
  for (int g = gid; g < nbags; g += ngroups) {
    const int s = g / B, b = g - s * B;
    int k0 = g, k1 = g + 1;
    if (offsets) { k0 = offsets[g]; k1 = offsets[g + 1]; }
    const float sc = bag_scale(combiner, k1 - k0);
    float* o = out + (size_t)b * out_ld + (size_t)s * pd;
    for (int ch = lane; ch < nch; ch += G) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = k0; k < k1; ++k) {
        const int v = inverse[k];
        if (v >= 0) {
          const float4 x = ldcg_f4(U + (size_t)v * ustride + 4 * ch);
          acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
      }
      acc.x *= sc; acc.y *= sc; acc.z *= sc; acc.w *= sc;
      *reinterpret_cast<float4*>(o + 4 * ch) = acc;
    }
  }
}

// dim % 4 == 0 and pd % 4 == 0: vector reductions into the unique-gradient rows.
__global__ void pool_bwd_vec4_kernel(float* __restrict__ gU, int gstride, const int* __restrict__ inverse,
                                     const int* __restrict__ offsets, int B, int S, int pd, int dim, int combiner,
                                     const float* __restrict__ gout, int gout_ld, int G) {
  pdl_sync();
  const int lane = threadIdx.x % G;
  const int gid = (blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int ngroups = (gridDim.x * blockDim.x) / G;
  const int nbags = B * S, nch = dim >> 2;
  for (int g = gid; g < nbags; g += ngroups) {
    const int s = g / B, b = g - s * B;
    int k0 = g, k1 = g + 1;
    if (offsets) { k0 = offsets[g]; k1 = offsets[g + 1]; }
    const float sc = bag_scale(combiner, k1 - k0);
    const float* go = gout + (size_t)b * gout_ld + (size_t)s * pd;
    for (int ch = lane; ch < nch; ch += G) {
      float4 x = *reinterpret_cast<const float4*>(go + 4 * ch);
      x.x *= sc; x.y *= sc; x.z *= sc; x.w *= sc;
      for (int k = k0; k < k1; ++k) {
        const int v = inverse[k];
        if (v >= 0) red_add_f32x4(gU + (size_t)v * gstride + 4 * ch, x);
      }
    }
  }
}

__global__ void pool_bwd_kernel(float* __restrict__ gU, int gstride, const int* __restrict__ inverse,
                                const int* __restrict__ offsets, int B, int S, int pd, int dim, int combiner,
                                const float* __restrict__ gout, int gout_ld, int G) {
  pdl_sync();
  const int lane = threadIdx.x % G;
  const int gid = (blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int ngroups = (gridDim.x * blockDim.x) / G;
  const int nbags = B * S;
  for (int g = gid; g < nbags; g += ngroups) {
    const int s = g / B, b = g - s * B;
    int k0 = g, k1 = g + 1;
    if (offsets) { k0 = offsets[g]; k1 = offsets[g + 1]; }
    const float sc = bag_scale(combiner, k1 - k0);
    const float* go = gout + (size_t)b * gout_ld + (size_t)s * pd;
    for (int d = lane; d < dim; d += G) {   // CVM columns (d >= dim) carry no gradient
      const float x = go[d] * sc;
      for (int k = k0; k < k1; ++k) {
        int v = inverse[k];
        if (v >= 0) atomicAdd(gU + (size_t)v * gstride + d, x);
      }
    }
  }
}

// Sequence gather of one column: element t of example b -> out[b, t, :]; t >= T is dropped,
// positions past the length stay zero (caller zero-fills).  lengths[b] = min(len, T).
__global__ void seq_fwd_kernel(const float* __restrict__ U, int ustride, const int* __restrict__ inverse,
                               const int* __restrict__ offsets, int B, int T, int pd, float* __restrict__ out,
                               int* __restrict__ lengths, int G) {
  pdl_sync();
  const int lane = threadIdx.x % G;
  const int gid = (blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int ngroups = (gridDim.x * blockDim.x) / G;
  for (int g = gid; g < B * T; g += ngroups) {
    const int b = g / T, tt = g - b * T;
    const int k0 = offsets[b], len = offsets[b + 1] - k0;
    if (tt == 0 && lane == 0 && lengths) lengths[b] = len < T ? len : T;
    if (tt >= len) continue;
    const int v = inverse[k0 + tt];
    float* o = out + ((size_t)b * T + tt) * pd;
    for (int d = lane; d < pd; d += G) o[d] = v >= 0 ? __ldcg(U + (size_t)v * ustride + d) : 0.f;
  }
}

__global__ void seq_bwd_kernel(float* __restrict__ gU, int gstride, const int* __restrict__ inverse,
                               const int* __restrict__ offsets, int B, int T, int pd, int dim,
                               const float* __restrict__ gout, int G) {
  pdl_sync();
  const int lane = threadIdx.x % G;
  const int gid = (blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int ngroups = (gridDim.x * blockDim.x) / G;
  for (int g = gid; g < B * T; g += ngroups) {
    const int b = g / T, tt = g - b * T;
    const int k0 = offsets[b], len = offsets[b + 1] - k0;
    if (tt >= len) continue;
    const int v = inverse[k0 + tt];
    if (v < 0) continue;
    const float* go = gout + ((size_t)b * T + tt) * pd;
    for (int d = lane; d < dim; d += G) atomicAdd(gU + (size_t)v * gstride + d, go[d]);
  }
}

inline int grid_for(long long groups, int G, int threads) {
  long long blocks = (groups * G + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return (int)blocks;
}

}  // namespace

void launch_pool_fwd(const float* U, int ustride, const int* inverse, const int* offsets, int B, int S, int pd,
                     int combiner, float* out, int out_ld, cudaStream_t st) {
  if ((pd & 3) == 0 && (out_ld & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    int G = lanes_for_width(pd);
    launch_pdl(pool_fwd_vec4_kernel, dim3(grid_for((long long)B * S, G, 256)), dim3(256), 0, st, U, ustride, inverse, offsets, B, S, pd,
                                                                               combiner, out, out_ld, G);
    return;
  }
  int G = pd >= 32 ? 32 : (pd >= 16 ? 16 : (pd >= 8 ? 8 : (pd >= 4 ? 4 : (pd >= 2 ? 2 : 1))));
  launch_pdl(pool_fwd_kernel, dim3(grid_for((long long)B * S, G, 256)), dim3(256), 0, st, U, ustride, inverse, offsets, B, S, pd, combiner,
                                                                        out, out_ld, G);
}
void launch_pool_bwd(float* gU, int gstride, const int* inverse, const int* offsets, int B, int S, int pd, int dim,
                     int combiner, const float* gout, int gout_ld, cudaStream_t st) {
  if ((pd & 3) == 0 && (dim & 3) == 0 && (gout_ld & 3) == 0 && (reinterpret_cast<uintptr_t>(gout) & 15) == 0) {
    int G = lanes_for_width(dim);
    launch_pdl(pool_bwd_vec4_kernel, dim3(grid_for((long long)B * S, G, 256)), dim3(256), 0, st, gU, gstride, inverse, offsets, B, S, pd, dim,
                                                                               combiner, gout, gout_ld, G);
    return;
  }
  int G = dim >= 32 ? 32 : (dim >= 16 ? 16 : (dim >= 8 ? 8 : (dim >= 4 ? 4 : (dim >= 2 ? 2 : 1))));
  launch_pdl(pool_bwd_kernel, dim3(grid_for((long long)B * S, G, 256)), dim3(256), 0, st, gU, gstride, inverse, offsets, B, S, pd, dim,
                                                                        combiner, gout, gout_ld, G);
}
void launch_seq_fwd(const float* U, int ustride, const int* inverse, const int* offsets, int B, int T, int pd,
                    float* out, int* lengths, cudaStream_t st) {
  int G = pd >= 32 ? 32 : (pd >= 16 ? 16 : (pd >= 8 ? 8 : (pd >= 4 ? 4 : (pd >= 2 ? 2 : 1))));
  launch_pdl(seq_fwd_kernel, dim3(grid_for((long long)B * T, G, 256)), dim3(256), 0, st, U, ustride, inverse, offsets, B, T, pd, out,
                                                                       lengths, G);
}
void launch_seq_bwd(float* gU, int gstride, const int* inverse, const int* offsets, int B, int T, int pd, int dim,
                    const float* gout, cudaStream_t st) {
  int G = dim >= 32 ? 32 : (dim >= 16 ? 16 : (dim >= 8 ? 8 : (dim >= 4 ? 4 : (dim >= 2 ? 2 : 1))));
  launch_pdl(seq_bwd_kernel, dim3(grid_for((long long)B * T, G, 256)), dim3(256), 0, st, gU, gstride, inverse, offsets, B, T, pd, dim, gout, G);
}

}  // namespace tn
