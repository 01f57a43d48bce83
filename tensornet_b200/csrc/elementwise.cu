// Memory-bound pieces of the dense towers, each fused as far as the data flow allows:
//   fm_fwd / fm_bwd            second-order FM term   (examples/common/layers.py:91-100)
//   concat_cast / split_cast   fp32/bf16 pieces -> one padded bf16 GEMM operand with the
//                              constant-one bias column, and the reverse for gradients
//   gemv_fwd / gemv_bwd        the final Dense(1) head (examples/models/deepfm.py:52-57)
//   bce_fwd_bwd                sigmoid + binary cross-entropy + dlogit + CTR/PCTR sums
//                              (examples/main.py:63-74, tensornet/metric/metrics.py:31-104)
//   cross_v1_fwd / bwd         DCN-v1 rank-1 cross layer (examples/common/layers.py:53-59)
#include <cuda_bf16.h>
#include "tn_device.cuh"
#include "tn_ops.h"

namespace tn {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- FM -------------------------------------------------------------------------------
// E: [B, F, D] (row stride ld).  One warp per example; lane d handles component d (D <= 32)
// or strides over D.
__global__ void fm_fwd_kernel(const float* __restrict__ E, int ld, int B, int F, int D, float* __restrict__ out) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int b = warp; b < B; b += nwarps) {
    const float* e = E + (size_t)b * ld;
    float acc = 0.f;
    for (int d = lane; d < D; d += 32) {
      float s = 0.f, sq = 0.f;
      for (int f = 0; f < F; ++f) { float x = e[f * D + d]; s += x; sq += x * x; }
      acc += s * s - sq;
    }
    acc = warp_sum(acc);
    if (lane == 0) out[b] = 0.5f * acc;
  }
}
// gE[b,f,d] = gout[b] * (sum_f E[b,:,d] - E[b,f,d])
__global__ void fm_bwd_kernel(const float* __restrict__ E, int ld, int B, int F, int D, const float* __restrict__ gout,
                              float* __restrict__ gE, int gld, int accumulate) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int b = warp; b < B; b += nwarps) {
    const float* e = E + (size_t)b * ld;
    float* g = gE + (size_t)b * gld;
    const float go = gout[b];
    for (int d = lane; d < D; d += 32) {
      float s = 0.f;
      for (int f = 0; f < F; ++f) s += e[f * D + d];
      for (int f = 0; f < F; ++f) {
        float v = go * (s - e[f * D + d]);
        if (accumulate) g[f * D + d] += v; else g[f * D + d] = v;
      }
    }
  }
}

// Vector variants for D % 4 == 0 with D/4 a power of two <= 32: a row is F*D/4 float4 chunks; lane l
// always sees the same d-chunk (l mod D/4), so per-lane partial sums are combined with xor-shuffles
// over the lanes that share it.
__global__ void fm_fwd_vec_kernel(const float* __restrict__ E, int ld, int B, int F, int D, float* __restrict__ out) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int dq = D >> 2, nch = F * dq;
  for (int b = warp; b < B; b += nwarps) {
    const float4* e = reinterpret_cast<const float4*>(E + (size_t)b * ld);
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    float sq = 0.f;
    for (int c = lane; c < nch; c += 32) {
      const float4 x = e[c];
      s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
      sq += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
    for (int o = 16; o >= dq; o >>= 1) {
      s.x += __shfl_xor_sync(0xffffffffu, s.x, o); s.y += __shfl_xor_sync(0xffffffffu, s.y, o);
      s.z += __shfl_xor_sync(0xffffffffu, s.z, o); s.w += __shfl_xor_sync(0xffffffffu, s.w, o);
    }
    float part = (lane < dq) ? (s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w) : 0.f;
    part = warp_sum(part) - warp_sum(sq);
    if (lane == 0) out[b] = 0.5f * part;
  }
}
__global__ void fm_bwd_vec_kernel(const float* __restrict__ E, int ld, int B, int F, int D, const float* __restrict__ gout,
                                  float* __restrict__ gE, int gld, int accumulate) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int dq = D >> 2, nch = F * dq;
  for (int b = warp; b < B; b += nwarps) {
    const float4* e = reinterpret_cast<const float4*>(E + (size_t)b * ld);
    float4* g = reinterpret_cast<float4*>(gE + (size_t)b * gld);
    const float go = gout[b];
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = lane; c < nch; c += 32) {
      const float4 x = e[c];
      s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
    }
    for (int o = 16; o >= dq; o >>= 1) {
      s.x += __shfl_xor_sync(0xffffffffu, s.x, o); s.y += __shfl_xor_sync(0xffffffffu, s.y, o);
      s.z += __shfl_xor_sync(0xffffffffu, s.z, o); s.w += __shfl_xor_sync(0xffffffffu, s.w, o);
    }
    for (int c = lane; c < nch; c += 32) {
      const float4 x = e[c];
      float4 v = make_float4(go * (s.x - x.x), go * (s.y - x.y), go * (s.z - x.z), go * (s.w - x.w));
      if (accumulate) { const float4 o4 = g[c]; v.x += o4.x; v.y += o4.y; v.z += o4.z; v.w += o4.w; }
      g[c] = v;
    }
  }
}

// ---- concat + cast ----------------------------------------------------------------------
__device__ __forceinline__ float concat_src(const ConcatArgs& a, int b, int c) {
  if (c == a.ones_col) return 1.f;
  int off = 0;
#pragma unroll
  for (int p = 0; p < kMaxPieces; ++p) {
    if (p < a.n_pieces) {
      const int w = a.width[p];
      if (c >= off && c < off + w) {
        const size_t idx = (size_t)b * a.ld[p] + (c - off);
        return a.is_bf16[p] ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.ptr[p])[idx])
                            : reinterpret_cast<const float*>(a.ptr[p])[idx];
      }
      off += w;
    }
  }
  return 0.f;
}
// one thread = 8 consecutive output columns = one 16-byte store (ld_out is a multiple of 8)
__global__ void concat_cast_kernel(const ConcatArgs a) {
  pdl_sync();
  const int cpr = a.ld_out >> 3;
  const long long total = (long long)a.B * cpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i / cpr), c0 = (int)(i - (long long)b * cpr) * 8;
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = concat_src(a, b, c0 + k);
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]), p3 = __floats2bfloat162_rn(v[6], v[7]);
    uint4 o = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                         *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.out) + (size_t)b * a.ld_out + c0) = o;
  }
}
// reverse: bf16 [B, ld_out] -> pieces (each piece written with its own ld); 8 columns per thread
__global__ void split_cast_kernel(const ConcatArgs a) {
  pdl_sync();
  const int cpr = a.ld_out >> 3;
  const long long total = (long long)a.B * cpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i / cpr), c0 = (int)(i - (long long)b * cpr) * 8;
    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.out) + (size_t)b * a.ld_out + c0);
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = c0 + k;
      int off = 0;
      for (int p = 0; p < a.n_pieces; ++p) {
        const int w = a.width[p];
        if (c >= off && c < off + w) {
          if (a.ptr[p]) {
            const size_t idx = (size_t)b * a.ld[p] + (c - off);
            if (a.is_bf16[p]) reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(a.ptr[p]))[idx] = x[k];
            else reinterpret_cast<float*>(const_cast<void*>(a.ptr[p]))[idx] = __bfloat162float(x[k]);
          }
          break;
        }
        off += w;
      }
    }
  }
}

// ---- Dense(1) head -------------------------------------------------------------------------
// y[b] = sum_k Z[b,k] * w[k]   (Z bf16 [B, ld], w fp32 [K]; the bias rides on Z's ones column)
__global__ void gemv_fwd_kernel(const __nv_bfloat16* __restrict__ Z, int ld, int B, int K, const float* __restrict__ w,
                                float* __restrict__ y) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int b = warp; b < B; b += nwarps) {
    const __nv_bfloat16* z = Z + (size_t)b * ld;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc += __bfloat162float(z[k]) * __ldg(w + k);
    acc = warp_sum(acc);
    if (lane == 0) y[b] = acc;
  }
}
// dZ[b,k] = dy[b] * w[k] (bf16, masked where relu_cols > k and Z <= 0);  gw[k] += sum_b dy[b] * Z[b,k]
__global__ void gemv_bwd_kernel(const __nv_bfloat16* __restrict__ Z, int ld, int B, int K, const float* __restrict__ w,
                                const float* __restrict__ dy, __nv_bfloat16* __restrict__ dZ, float* __restrict__ gw,
                                int relu_cols) {
  pdl_sync();
  extern __shared__ float s_gw[];   // [K]
  for (int k = threadIdx.x; k < K; k += blockDim.x) s_gw[k] = 0.f;
  __syncthreads();
  const int rows_per_block = (B + gridDim.x - 1) / gridDim.x;
  const int b0 = blockIdx.x * rows_per_block;
  const int b1 = min(B, b0 + rows_per_block);
  // thread k-strided over columns, loop over the block's rows: coalesced along k
  for (int k = threadIdx.x; k < ld; k += blockDim.x) {
    const float wk = k < K ? __ldg(w + k) : 0.f;
    float acc = 0.f;
    for (int b = b0; b < b1; ++b) {
      const float z = __bfloat162float(Z[(size_t)b * ld + k]);
      const float d = dy[b];
      float g = d * wk;
      if (k < relu_cols && !(z > 0.f)) g = 0.f;
      dZ[(size_t)b * ld + k] = __float2bfloat16(k < K ? g : 0.f);
      acc += d * z;
    }
    if (k < K) s_gw[k] = acc;
  }
  __syncthreads();
  for (int k = threadIdx.x; k < K; k += blockDim.x) atomicAdd(gw + k, s_gw[k]);
}

// Row-per-warp variant for ld <= 512: lane l owns column pairs (2l, 2l+1) + 64*i, keeps w and the
// weight-gradient partial sums in registers, and streams Z / dZ with 4-byte accesses.
__global__ void gemv_bwd_rows_kernel(const __nv_bfloat16* __restrict__ Z, int ld, int B, int K, const float* __restrict__ w,
                                     const float* __restrict__ dy, __nv_bfloat16* __restrict__ dZ, float* __restrict__ gw,
                                     int relu_cols) {
  pdl_sync();
  constexpr int kPairs = 8;
  extern __shared__ float s_gw[];   // [ld]
  for (int k = threadIdx.x; k < ld; k += blockDim.x) s_gw[k] = 0.f;
  __syncthreads();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  float2 wv[kPairs], acc[kPairs];
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    const int c = 64 * i + 2 * lane;
    wv[i].x = c < K ? __ldg(w + c) : 0.f;
    wv[i].y = c + 1 < K ? __ldg(w + c + 1) : 0.f;
    acc[i] = make_float2(0.f, 0.f);
  }
  for (int b = warp; b < B; b += nwarps) {
    const float d = dy[b];
    const __nv_bfloat162* z = reinterpret_cast<const __nv_bfloat162*>(Z + (size_t)b * ld);
    __nv_bfloat162* dz = reinterpret_cast<__nv_bfloat162*>(dZ + (size_t)b * ld);
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
      const int c = 64 * i + 2 * lane;
      if (c < ld) {
        const float2 zz = __bfloat1622float2(z[32 * i + lane]);
        float gx = d * wv[i].x, gy = d * wv[i].y;
        if (c < relu_cols && !(zz.x > 0.f)) gx = 0.f;
        if (c + 1 < relu_cols && !(zz.y > 0.f)) gy = 0.f;
        dz[32 * i + lane] = __floats2bfloat162_rn(gx, gy);
        acc[i].x += d * zz.x;
        acc[i].y += d * zz.y;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    const int c = 64 * i + 2 * lane;
    if (c < K) atomicAdd(&s_gw[c], acc[i].x);
    if (c + 1 < K) atomicAdd(&s_gw[c + 1], acc[i].y);
  }
  __syncthreads();
  for (int k = threadIdx.x; k < K; k += blockDim.x) atomicAdd(gw + k, s_gw[k]);
}

// ---- sigmoid BCE ---------------------------------------------------------------------------
// loss = mean(softplus(l) - y*l) ; dlogit = (sigmoid(l) - y) * scale ; pred = sigmoid(l)
// sums[0] += loss_sum/B, sums[1] += sum(y), sums[2] += sum(pred), sums[3] += B
// nbins > 0: the words behind sums[3] are two histograms of the prediction (u32 counts, nbins buckets over [0, 1]):
// positives (label > 0.5) first, negatives second - what a streaming AUC needs.
__global__ void bce_kernel(const float* __restrict__ logit, const float* __restrict__ label, int B, float* __restrict__ pred,
                           float* __restrict__ dlogit, float grad_scale, float* __restrict__ sums, int nbins) {
  pdl_sync();
  unsigned* hist = reinterpret_cast<unsigned*>(sums + 4);
  float ls = 0.f, ys = 0.f, ps = 0.f;
  for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < B; b += gridDim.x * blockDim.x) {
    const float l = logit[b], y = label[b];
    const float p = 1.f / (1.f + expf(-l));
    const float sp = fmaxf(l, 0.f) + log1pf(expf(-fabsf(l)));
    ls += sp - y * l;
    ys += y;
    ps += p;
    if (pred) pred[b] = p;
    if (dlogit) dlogit[b] = (p - y) * grad_scale;
    if (nbins > 0) atomicAdd(hist + (y > 0.5f ? 0 : nbins) + min(nbins - 1, (int)(p * (float)nbins)), 1u);
  }
  ls = warp_sum(ls); ys = warp_sum(ys); ps = warp_sum(ps);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(&sums[0], ls / (float)B);
    atomicAdd(&sums[1], ys);
    atomicAdd(&sums[2], ps);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&sums[3], (float)B);
}

// ---- DCN-v1 cross layer: y = x0 * (xl . w) + b + xl ---------------------------------------------
__global__ void cross_v1_fwd_kernel(const float* __restrict__ x0, const float* __restrict__ xl, const float* __restrict__ w,
                                    const float* __restrict__ bias, int B, int D, float* __restrict__ y, float* __restrict__ dot) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int b = warp; b < B; b += nwarps) {
    const float* a = x0 + (size_t)b * D; const float* c = xl + (size_t)b * D;
    float s = 0.f;
    for (int d = lane; d < D; d += 32) s += c[d] * w[d];
    s = warp_sum(s);
    if (lane == 0) dot[b] = s;
    for (int d = lane; d < D; d += 32) y[(size_t)b * D + d] = a[d] * s + bias[d] + c[d];
  }
}
// gx0 += gy * s ; gxl = gy + w * (gy . x0) ; gw += xl * (gy . x0) ; gb += gy
__global__ void cross_v1_bwd_kernel(const float* __restrict__ x0, const float* __restrict__ xl, const float* __restrict__ w,
                                    const float* __restrict__ dot, const float* __restrict__ gy, int B, int D,
                                    float* __restrict__ gx0, float* __restrict__ gxl, float* __restrict__ gw, float* __restrict__ gb) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int b = warp; b < B; b += nwarps) {
    const float* a = x0 + (size_t)b * D; const float* c = xl + (size_t)b * D; const float* g = gy + (size_t)b * D;
    float t = 0.f;
    for (int d = lane; d < D; d += 32) t += g[d] * a[d];
    t = warp_sum(t);
    const float s = dot[b];
    for (int d = lane; d < D; d += 32) {
      gx0[(size_t)b * D + d] = g[d] * s;
      gxl[(size_t)b * D + d] = g[d] + w[d] * t;
      atomicAdd(gw + d, c[d] * t);
      atomicAdd(gb + d, g[d]);
    }
  }
}

// g[i] = y[i] > 0 ? g[i] : 0   (bf16, 8 elements per thread)
__global__ void relu_mask_kernel(uint4* __restrict__ g, const uint4* __restrict__ y, long long n8) {
  pdl_sync();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 gv = g[i]; const uint4 yv = y[i];
    __nv_bfloat16* gp = reinterpret_cast<__nv_bfloat16*>(&gv);
    const __nv_bfloat16* yp = reinterpret_cast<const __nv_bfloat16*>(&yv);
#pragma unroll
    for (int k = 0; k < 8; ++k) if (!(__bfloat162float(yp[k]) > 0.f)) gp[k] = __float2bfloat16(0.f);
    g[i] = gv;
  }
}

// DCN-v2 backward, elementwise part of one cross layer (y = x0 * u + x_l, u = W x_l + b), 8 elements per thread:
//   gx0 += g * u   (fp32 accumulator over the layers)      du = g * x0   (bf16, input of the two GEMMs)
// `first` writes gx0 instead of accumulating (no zero fill needed before the first layer).
__global__ void cross_v2_bwd_elem_kernel(const uint4* __restrict__ g, const uint4* __restrict__ u, const uint4* __restrict__ x0,
                                         float4* __restrict__ gx0, uint4* __restrict__ du, long long n8, int first) {
  pdl_sync();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const uint4 gv = g[i], uv = u[i], xv = x0[i];
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
    float4 a = first ? make_float4(0.f, 0.f, 0.f, 0.f) : gx0[2 * i], b = first ? a : gx0[2 * i + 1];
    uint4 dv;
    uint32_t* dp = reinterpret_cast<uint32_t*>(&dv);
    float acc[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 gf = __bfloat1622float2(gp[k]), uf = __bfloat1622float2(up[k]), xf = __bfloat1622float2(xp[k]);
      acc[2 * k] += gf.x * uf.x;
      acc[2 * k + 1] += gf.y * uf.y;
      __nv_bfloat162 d = __floats2bfloat162_rn(gf.x * xf.x, gf.y * xf.y);
      dp[k] = *reinterpret_cast<uint32_t*>(&d);
    }
    gx0[2 * i] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    gx0[2 * i + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    du[i] = dv;
  }
}

// out = bf16(gx0 + g): the gradient that reaches x0 through the residual chain joins the Hadamard terms.
__global__ void cross_v2_bwd_final_kernel(const float4* __restrict__ gx0, const uint4* __restrict__ g, uint4* __restrict__ out, long long n8) {
  pdl_sync();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const float4 a = gx0[2 * i], b = gx0[2 * i + 1];
    const uint4 gv = g[i];
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const float acc[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint4 ov;
    uint32_t* op = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 gf = __bfloat1622float2(gp[k]);
      __nv_bfloat162 d = __floats2bfloat162_rn(acc[2 * k] + gf.x, acc[2 * k + 1] + gf.y);
      op[k] = *reinterpret_cast<uint32_t*>(&d);
    }
    out[i] = ov;
  }
}

inline int blocks_for(long long work, int per_block) {
  long long b = (work + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return (int)b;
}

}  // namespace

static bool fm_vec_ok(const void* p, int ld, int D) {
  const int dq = D >> 2;
  return (D & 3) == 0 && dq >= 1 && dq <= 32 && (dq & (dq - 1)) == 0 && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}
void launch_fm_fwd(const float* E, int ld, int B, int F, int D, float* out, cudaStream_t st) {
  if (fm_vec_ok(E, ld, D)) { launch_pdl(fm_fwd_vec_kernel, dim3(blocks_for(B, 8)), dim3(256), 0, st, E, ld, B, F, D, out); return; }
  launch_pdl(fm_fwd_kernel, dim3(blocks_for(B, 8)), dim3(256), 0, st, E, ld, B, F, D, out);
}
void launch_fm_bwd(const float* E, int ld, int B, int F, int D, const float* gout, float* gE, int gld, int accumulate, cudaStream_t st) {
  if (fm_vec_ok(E, ld, D) && fm_vec_ok(gE, gld, D)) {
    launch_pdl(fm_bwd_vec_kernel, dim3(blocks_for(B, 8)), dim3(256), 0, st, E, ld, B, F, D, gout, gE, gld, accumulate);
    return;
  }
  launch_pdl(fm_bwd_kernel, dim3(blocks_for(B, 8)), dim3(256), 0, st, E, ld, B, F, D, gout, gE, gld, accumulate);
}
void launch_concat_cast(const ConcatArgs& a, cudaStream_t st) {
  launch_pdl(concat_cast_kernel, dim3(blocks_for((long long)a.B * (a.ld_out >> 3), 256)), dim3(256), 0, st, a);
}
void launch_split_cast(const ConcatArgs& a, cudaStream_t st) {
  launch_pdl(split_cast_kernel, dim3(blocks_for((long long)a.B * (a.ld_out >> 3), 256)), dim3(256), 0, st, a);
}
void launch_gemv_fwd(const void* Z, int ld, int B, int K, const float* w, float* y, cudaStream_t st) {
  launch_pdl(gemv_fwd_kernel, dim3(blocks_for(B, 8)), dim3(256), 0, st, reinterpret_cast<const __nv_bfloat16*>(Z), ld, B, K, w, y);
}
void launch_gemv_bwd(const void* Z, int ld, int B, int K, const float* w, const float* dy, void* dZ, float* gw, int relu_cols,
                     cudaStream_t st) {
  if (ld <= 512 && (ld & 1) == 0) {
    int nb = (B + 7) / 8; if (nb > 148 * 2) nb = 148 * 2; if (nb < 1) nb = 1;
    launch_pdl(gemv_bwd_rows_kernel, dim3(nb), dim3(256), ld * sizeof(float), st, reinterpret_cast<const __nv_bfloat16*>(Z), ld, B, K, w, dy,
                                                             reinterpret_cast<__nv_bfloat16*>(dZ), gw, relu_cols);
    return;
  }
  int blocks = B / 32; if (blocks < 1) blocks = 1; if (blocks > 296) blocks = 296;
  if (K * sizeof(float) > 40 * 1024) {   // very wide last layer: the weight copy needs the large-shared-memory opt-in
    static bool opted = false;
    if (!opted) { cudaFuncSetAttribute((const void*)gemv_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); opted = true; }
  }
  launch_pdl(gemv_bwd_kernel, dim3(blocks), dim3(256), K * sizeof(float), st, reinterpret_cast<const __nv_bfloat16*>(Z), ld, B, K, w, dy,
                                                          reinterpret_cast<__nv_bfloat16*>(dZ), gw, relu_cols);
}
void launch_bce(const float* logit, const float* label, int B, float* pred, float* dlogit, float grad_scale, float* sums,
                int nbins, cudaStream_t st) {
  launch_pdl(bce_kernel, dim3(blocks_for(B, 256)), dim3(256), 0, st, logit, label, B, pred, dlogit, grad_scale, sums, nbins);
}
void launch_relu_mask(void* g, const void* y, long long n, cudaStream_t st) {
  launch_pdl(relu_mask_kernel, dim3(blocks_for(n / 8, 256)), dim3(256), 0, st, reinterpret_cast<uint4*>(g), reinterpret_cast<const uint4*>(y), n / 8);
}
void launch_cross_v2_bwd_elem(const void* g, const void* u, const void* x0, float* gx0, void* du, long long n, int first, cudaStream_t st) {
  launch_pdl(cross_v2_bwd_elem_kernel, dim3(blocks_for(n / 8, 256)), dim3(256), 0, st, reinterpret_cast<const uint4*>(g),
             reinterpret_cast<const uint4*>(u), reinterpret_cast<const uint4*>(x0), reinterpret_cast<float4*>(gx0), reinterpret_cast<uint4*>(du),
             n / 8, first);
}
void launch_cross_v2_bwd_final(const float* gx0, const void* g, void* out, long long n, cudaStream_t st) {
  launch_pdl(cross_v2_bwd_final_kernel, dim3(blocks_for(n / 8, 256)), dim3(256), 0, st, reinterpret_cast<const float4*>(gx0),
             reinterpret_cast<const uint4*>(g), reinterpret_cast<uint4*>(out), n / 8);
}
void launch_cross_v1_fwd(const float* x0, const float* xl, const float* w, const float* bias, int B, int D, float* y, float* dot,
                         cudaStream_t st) {
  launch_pdl(cross_v1_fwd_kernel, dim3(blocks_for(B, 8)), dim3(256), 0, st, x0, xl, w, bias, B, D, y, dot);
}
void launch_cross_v1_bwd(const float* x0, const float* xl, const float* w, const float* dot, const float* gy, int B, int D,
                         float* gx0, float* gxl, float* gw, float* gb, cudaStream_t st) {
  launch_pdl(cross_v1_bwd_kernel, dim3(blocks_for(B, 8)), dim3(256), 0, st, x0, xl, w, dot, gy, B, D, gx0, gxl, gw, gb);
}

}  // namespace tn
