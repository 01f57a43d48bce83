// Serving-side lookup: read-only dictionary probe + per-slot pooling + cast into the padded bf16
// operand of the first dense layer, in one kernel.  The reference's online demo looks every id up
// in a dictionary service, mean-pools multi-valued slots and copies the result into the dense
// graph's feeds (examples/online_serving/main.cc:42-91, graph.cc:25-71); its lookup is a stub
// that returns random vectors.  Signs missing from the dictionary contribute zeros.
#include <cuda_bf16.h>
#include "sparse_table.cuh"
#include "tn_ops.h"

namespace tn {

namespace {

// Bag g = s * B + b holds ids [offsets[g], offsets[g+1]) (or exactly id g when offsets == nullptr).
// dim % 4 == 0; G lanes per bag, each lane owns float4 chunks of the embedding.
__global__ void dict_lookup_pool_kernel(TableView t, const long long* __restrict__ ids, const int* __restrict__ offsets, int B,
                                        int S, int combiner, __nv_bfloat16* __restrict__ out, int ld_out, int ones_col, int G) {
  const int lane = threadIdx.x % G;
  const int gid = (blockIdx.x * blockDim.x + threadIdx.x) / G;
  const int ngroups = (gridDim.x * blockDim.x) / G;
  const int dim = t.dim, nch = dim >> 2, nbags = B * S;
  for (int g = gid; g < nbags; g += ngroups) {
    const int s = g / B, b = g - s * B;
    int k0 = g, k1 = g + 1;
    if (offsets) { k0 = offsets[g]; k1 = offsets[g + 1]; }
    const int len = k1 - k0;
    const float sc = len <= 0 ? 0.f : (combiner == 1 ? 1.f / (float)len : (combiner == 2 ? rsqrtf((float)len) : 1.f));
    __nv_bfloat16* o = out + (size_t)b * ld_out + (size_t)s * dim;
    for (int ch = lane; ch < nch; ch += G) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = k0; k < k1; ++k) {
        const int r = table_find(t, canon_key((unsigned long long)ids[k]));
        if (r >= 0) {
          const float4 x = *reinterpret_cast<const float4*>(t.rows + (size_t)r * t.stride + 4 * ch);
          acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
      }
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * sc, acc.y * sc), hi = __floats2bfloat162_rn(acc.z * sc, acc.w * sc);
      *reinterpret_cast<uint2*>(o + 4 * ch) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
  // tail columns of every row: constant one (bias input of the first layer) and zero padding
  const int tail0 = S * dim, ntail = ld_out - tail0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < B * ntail; i += gridDim.x * blockDim.x) {
    const int b = i / ntail, c = tail0 + (i - b * ntail);
    out[(size_t)b * ld_out + c] = __float2bfloat16(c == ones_col ? 1.f : 0.f);
  }
}

__global__ void sigmoid_kernel(const float* __restrict__ x, float* __restrict__ y, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) y[i] = 1.f / (1.f + expf(-x[i]));
}

}  // namespace

void launch_dict_lookup_pool(const TableView& t, const long long* ids, const int* offsets, int B, int S, int combiner, void* out,
                             int ld_out, int ones_col, cudaStream_t st) {
  int G = lanes_for_width(t.dim);
  long long blocks = ((long long)B * S * G + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  dict_lookup_pool_kernel<<<(int)blocks, 256, 0, st>>>(t, ids, offsets, B, S, combiner, reinterpret_cast<__nv_bfloat16*>(out), ld_out,
                                                     ones_col, G);
}
void launch_sigmoid(const float* x, float* y, int n, cudaStream_t st) {
  int blocks = (n + 255) / 256; if (blocks > 148 * 4) blocks = 148 * 4; if (blocks < 1) blocks = 1;
  sigmoid_kernel<<<blocks, 256, 0, st>>>(x, y, n);
}

}  // namespace tn
