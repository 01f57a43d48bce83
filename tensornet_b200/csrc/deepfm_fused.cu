// DeepFM-specific fusions of the memory-bound glue around the tensor-core towers
// (model structure: examples/models/deepfm.py, examples/common/layers.py:72-103 in the reference).
//
//   deepfm_input_fwd : gather the pulled embedding rows of every slot (single-hot), compute the
//                      second-order FM term and write the padded bf16 operand of the first MLP layer
//                      [emb | dense | 1 | 0] in one pass - replaces pool + FM + concat/cast.
//   deepfm_input_bwd : gradient of that operand (bf16, from the first layer's dgrad) plus the FM
//                      gradient, scattered straight into the unique-gradient rows - replaces
//                      split/cast + FM backward + add + pool backward.
//   deepfm_head_loss : Dense(1) over [h | linear | fm | 1], sigmoid cross-entropy, CTR / PCTR sums
//                      and the complete backward of the head (dH with the ReLU mask applied, dLinear,
//                      dFM, weight gradient) in one kernel - the logit gradient depends on nothing
//                      but the logit and the label, so forward and backward of the head are one pass.
#include <cuda_bf16.h>
#include "tn_device.cuh"
#include "tn_ops.h"

namespace tn {

namespace {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// D % 4 == 0, dq = D/4 a power of two <= 32.  One warp per example.
__global__ void deepfm_input_fwd_kernel(const float* __restrict__ U, int ustride, const int* __restrict__ inverse, int B, int S,
                                        int D, const float* __restrict__ dense, int Dd, int ld_dense,
                                        __nv_bfloat16* __restrict__ X0, int ld, float* __restrict__ fm, int lin_col,
                                        float* __restrict__ Lout) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int dq = D >> 2, nch = S * dq;
  for (int b = warp; b < B; b += nwarps) {
    __nv_bfloat16* xrow = X0 + (size_t)b * ld;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    float sq = 0.f;
    // batches of 4 x 32 chunks: first all row indices, then all row gathers, then the arithmetic, so that a
    // warp has four independent loads in flight at each of the two dependent steps
    for (int c0 = 0; c0 < nch; c0 += 128) {
      int v[4];
      float4 x[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = c0 + 32 * k + lane;
        v[k] = c < nch ? __ldg(inverse + (size_t)(c / dq) * B + b) : -1;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = c0 + 32 * k + lane;
        x[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (v[k] >= 0) x[k] = ldcg_f4(U + (size_t)v[k] * ustride + 4 * (c % dq));
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = c0 + 32 * k + lane;
        if (c >= nch) continue;
        s.x += x[k].x; s.y += x[k].y; s.z += x[k].z; s.w += x[k].w;
        sq += x[k].x * x[k].x + x[k].y * x[k].y + x[k].z * x[k].z + x[k].w * x[k].w;
        __nv_bfloat162 lo = __floats2bfloat162_rn(x[k].x, x[k].y), hi = __floats2bfloat162_rn(x[k].z, x[k].w);
        *reinterpret_cast<uint2*>(xrow + 4 * c) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      }
    }
    for (int o = 16; o >= dq; o >>= 1) {
      s.x += __shfl_xor_sync(0xffffffffu, s.x, o); s.y += __shfl_xor_sync(0xffffffffu, s.y, o);
      s.z += __shfl_xor_sync(0xffffffffu, s.z, o); s.w += __shfl_xor_sync(0xffffffffu, s.w, o);
    }
    float part = (lane < dq) ? (s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w) : 0.f;
    part = wsum(part) - wsum(sq);
    if (lane == 0) fm[b] = 0.5f * part;
    if (lin_col >= 0) {   // the slot's linear weight rides in column `lin_col` of the same row
      for (int f = lane; f < S; f += 32) {
        const int v = __ldg(inverse + (size_t)f * B + b);
        Lout[(size_t)b * S + f] = v >= 0 ? __ldcg(U + (size_t)v * ustride + lin_col) : 0.f;
      }
    }
    const int tail0 = S * D;
    for (int j = lane; j < ld - tail0; j += 32) {
      float v = 0.f;
      if (j < Dd) v = dense[(size_t)b * ld_dense + j];
      else if (j == Dd) v = 1.f;
      xrow[tail0 + j] = __float2bfloat16(v);
    }
  }
}

__global__ void deepfm_input_bwd_kernel(const float* __restrict__ U, int ustride, const int* __restrict__ inverse, int B, int S,
                                        int D, const __nv_bfloat16* __restrict__ dX0, int ld, const float* __restrict__ gfm,
                                        float* __restrict__ gU, int gstride, int lin_col, const float* __restrict__ dL) {
  pdl_sync();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int dq = D >> 2, nch = S * dq;
  for (int b = warp; b < B; b += nwarps) {
    const __nv_bfloat16* grow = dX0 + (size_t)b * ld;
    const float gf = gfm[b];
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (nch <= 128) {
      // the usual case: the example's rows stay in registers between the field sum and the gradient
      int v[4];
      float4 x[4];
      uint2 raw[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = 32 * k + lane;
        v[k] = c < nch ? __ldg(inverse + (size_t)(c / dq) * B + b) : -1;
        raw[k] = c < nch ? *reinterpret_cast<const uint2*>(grow + 4 * c) : make_uint2(0u, 0u);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = 32 * k + lane;
        x[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (v[k] >= 0) x[k] = ldcg_f4(U + (size_t)v[k] * ustride + 4 * (c % dq));
        s.x += x[k].x; s.y += x[k].y; s.z += x[k].z; s.w += x[k].w;
      }
      for (int o = 16; o >= dq; o >>= 1) {
        s.x += __shfl_xor_sync(0xffffffffu, s.x, o); s.y += __shfl_xor_sync(0xffffffffu, s.y, o);
        s.z += __shfl_xor_sync(0xffffffffu, s.z, o); s.w += __shfl_xor_sync(0xffffffffu, s.w, o);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = 32 * k + lane;
        if (v[k] < 0) continue;
        const float2 g01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[k].x));
        const float2 g23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[k].y));
        float4 g;
        g.x = g01.x + gf * (s.x - x[k].x);
        g.y = g01.y + gf * (s.y - x[k].y);
        g.z = g23.x + gf * (s.z - x[k].z);
        g.w = g23.y + gf * (s.w - x[k].w);
        red_add_f32x4(gU + (size_t)v[k] * gstride + 4 * (c % dq), g);
      }
    } else {
      for (int c = lane; c < nch; c += 32) {
        const int f = c / dq, dc = c - f * dq;
        const int v = __ldg(inverse + (size_t)f * B + b);
        if (v >= 0) {
          const float4 x = ldcg_f4(U + (size_t)v * ustride + 4 * dc);
          s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
        }
      }
      for (int o = 16; o >= dq; o >>= 1) {
        s.x += __shfl_xor_sync(0xffffffffu, s.x, o); s.y += __shfl_xor_sync(0xffffffffu, s.y, o);
        s.z += __shfl_xor_sync(0xffffffffu, s.z, o); s.w += __shfl_xor_sync(0xffffffffu, s.w, o);
      }
      for (int c = lane; c < nch; c += 32) {
        const int f = c / dq, dc = c - f * dq;
        const int v = __ldg(inverse + (size_t)f * B + b);
        if (v < 0) continue;
        const float4 x = ldcg_f4(U + (size_t)v * ustride + 4 * dc);
        const uint2 raw = *reinterpret_cast<const uint2*>(grow + 4 * c);
        const float2 g01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 g23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        float4 g;
        g.x = g01.x + gf * (s.x - x.x);
        g.y = g01.y + gf * (s.y - x.y);
        g.z = g23.x + gf * (s.z - x.z);
        g.w = g23.y + gf * (s.w - x.w);
        red_add_f32x4(gU + (size_t)v * gstride + 4 * dc, g);
      }
    }
    if (lin_col >= 0) {
      for (int f = lane; f < S; f += 32) {
        const int v = __ldg(inverse + (size_t)f * B + b);
        if (v >= 0) atomicAdd(gU + (size_t)v * gstride + lin_col, dL[(size_t)b * S + f]);
      }
    }
  }
}

// Head + loss + head backward.  w = [ wH (NH) | wL (NL) | wfm | bias ].  ldh <= 512, even.
// sums: [0] += mean loss, [1] += sum(label), [2] += sum(pred), [3] += B; with nbins > 0 the words behind them are the
// two prediction histograms (u32 counts; positives, then negatives) of a streaming AUC.
constexpr int kHeadPairs = 8;
constexpr int kHeadParts = 16;            // partial copies of the weight gradient in the scratch area
constexpr int kHeadPartStride = 576;      // floats per copy: >= 64 * kHeadPairs + 32 + 2, multiple of 4
__global__ void deepfm_head_loss_kernel(const __nv_bfloat16* __restrict__ H, int ldh, int NH, const float* __restrict__ L, int NL,
                                        const float* __restrict__ fm, const float* __restrict__ w, const float* __restrict__ label,
                                        int B, __nv_bfloat16* __restrict__ dH, float* __restrict__ dL, float* __restrict__ dfm,
                                        float* __restrict__ gw, float* __restrict__ sums, int nbins,
                                        float* __restrict__ pred, float* __restrict__ loss_out, float* __restrict__ scratch) {
  pdl_sync();
  extern __shared__ float s_gw[];   // [NH + NL + 2]
  const int NW = NH + NL + 2;
  for (int k = threadIdx.x; k < NW; k += blockDim.x) s_gw[k] = 0.f;
  __syncthreads();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  float2 wv[kHeadPairs], acc[kHeadPairs];
#pragma unroll
  for (int i = 0; i < kHeadPairs; ++i) {
    const int c = 64 * i + 2 * lane;
    wv[i].x = c < NH ? __ldg(w + c) : 0.f;
    wv[i].y = c + 1 < NH ? __ldg(w + c + 1) : 0.f;
    acc[i] = make_float2(0.f, 0.f);
  }
  const float wl = lane < NL ? __ldg(w + NH + lane) : 0.f;       // NL <= 32 linear weights, one per lane
  const float wfm = __ldg(w + NH + NL), bias = __ldg(w + NH + NL + 1);
  float accL = 0.f, accfm = 0.f, accb = 0.f, ls = 0.f, ys = 0.f, ps = 0.f;
  const float invB = 1.f / (float)B;
  for (int b = warp; b < B; b += nwarps) {
    const __nv_bfloat162* z = reinterpret_cast<const __nv_bfloat162*>(H + (size_t)b * ldh);
    float2 zz[kHeadPairs];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kHeadPairs; ++i) {
      const int c = 64 * i + 2 * lane;
      zz[i] = make_float2(0.f, 0.f);
      if (c < ldh) {
        zz[i] = __bfloat1622float2(z[32 * i + lane]);
        dot += zz[i].x * wv[i].x + zz[i].y * wv[i].y;
      }
    }
    const float lv = lane < NL ? L[(size_t)b * NL + lane] : 0.f;
    dot += lv * wl;
    dot = wsum(dot);
    const float f = fm[b], y = label[b];
    const float logit = dot + f * wfm + bias;
    const float p = 1.f / (1.f + expf(-logit));
    const float dl = (p - y) * invB;
    if (lane == 0) {
      ls += fmaxf(logit, 0.f) + log1pf(expf(-fabsf(logit))) - y * logit;
      ys += y; ps += p;
      if (pred) pred[b] = p;
      if (nbins > 0)
        atomicAdd(reinterpret_cast<unsigned*>(sums + 4) + (y > 0.5f ? 0 : nbins) + min(nbins - 1, (int)(p * (float)nbins)), 1u);
      dfm[b] = dl * wfm;
      accfm += dl * f;
      accb += dl;
    }
    if (lane < NL) { dL[(size_t)b * NL + lane] = dl * wl; accL += dl * lv; }
    __nv_bfloat162* dz = reinterpret_cast<__nv_bfloat162*>(dH + (size_t)b * ldh);
#pragma unroll
    for (int i = 0; i < kHeadPairs; ++i) {
      const int c = 64 * i + 2 * lane;
      if (c < ldh) {
        // gradient w.r.t. the ReLU output h, already masked by h > 0 (columns >= NH are the ones / pad columns)
        const float gx = (c < NH && zz[i].x > 0.f) ? dl * wv[i].x : 0.f;
        const float gy = (c + 1 < NH && zz[i].y > 0.f) ? dl * wv[i].y : 0.f;
        dz[32 * i + lane] = __floats2bfloat162_rn(gx, gy);
        acc[i].x += dl * zz[i].x;
        acc[i].y += dl * zz[i].y;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kHeadPairs; ++i) {
    const int c = 64 * i + 2 * lane;
    if (c < NH) atomicAdd(&s_gw[c], acc[i].x);
    if (c + 1 < NH) atomicAdd(&s_gw[c + 1], acc[i].y);
  }
  if (lane < NL) atomicAdd(&s_gw[NH + lane], accL);
  if (lane == 0) {
    atomicAdd(&s_gw[NH + NL], accfm);
    atomicAdd(&s_gw[NH + NL + 1], accb);
    const float l = ls * invB;
    atomicAdd(&sums[0], l);
    atomicAdd(&scratch[0], l);
    atomicAdd(&sums[1], ys);
    atomicAdd(&sums[2], ps);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&sums[3], (float)B);
  __syncthreads();
  // The per-block weight gradients are summed in two steps.  Hundreds of blocks adding to the same few hundred words of
  // `gw` at the same moment queue up behind one another in L2 (that tail used to be most of the kernel); instead a block
  // adds into one of kHeadParts partial copies in the scratch area (a sixteenth of the blocks per copy), and the last
  // block to finish folds the copies into `gw` and leaves them at zero for the next launch.
  float* parts = scratch + 4;                              // [kHeadParts][kHeadPartStride]
  {
    float* mine = parts + (size_t)(blockIdx.x % kHeadParts) * kHeadPartStride;
    const int n4 = NW >> 2;
    for (int k = threadIdx.x; k < n4; k += blockDim.x)
      red_add_f32x4(mine + 4 * k, make_float4(s_gw[4 * k], s_gw[4 * k + 1], s_gw[4 * k + 2], s_gw[4 * k + 3]));
    for (int k = 4 * n4 + threadIdx.x; k < NW; k += blockDim.x) atomicAdd(mine + k, s_gw[k]);
  }
  // The loss is summed in a persistent scratch word that is zero between launches; the last block to finish
  // moves the total into `loss_out` and re-arms the scratch, so the caller never has to clear anything.
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned prev = atomicAdd(reinterpret_cast<unsigned*>(scratch) + 1, 1u);
    s_last = prev == gridDim.x - 1;
    if (s_last) {
      __threadfence();
      *loss_out = atomicExch(&scratch[0], 0.f);
      reinterpret_cast<unsigned*>(scratch)[1] = 0u;
    }
  }
  __syncthreads();
  if (s_last) {
    for (int k = threadIdx.x; k < NW; k += blockDim.x) {
      float sum = 0.f;
#pragma unroll
      for (int q = 0; q < kHeadParts; ++q) {
        float* pq = parts + (size_t)q * kHeadPartStride + k;
        sum += __ldcg(pq);
        *pq = 0.f;
      }
      gw[k] += sum;          // nobody else touches the head's gradient while this kernel runs
    }
  }
}

}  // namespace

const char* launch_deepfm_input_fwd(const float* U, int ustride, const int* inverse, int B, int S, int D, const float* dense, int Dd,
                                    int ld_dense, void* X0, int ld, float* fm, int lin_col, float* Lout, cudaStream_t st) {
  const int dq = D >> 2;
  if ((D & 3) || dq < 1 || dq > 32 || (dq & (dq - 1))) return "deepfm_input: embedding dim must be 4 * 2^k, at most 128";
  if (ld < S * D + Dd + 1 || (ld & 3)) return "deepfm_input: operand row too short";
  int blocks = (B + 7) / 8; if (blocks > 148 * 8) blocks = 148 * 8; if (blocks < 1) blocks = 1;
  cudaError_t e = launch_pdl(deepfm_input_fwd_kernel, dim3(blocks), dim3(256), 0, st, U, ustride, inverse, B, S, D, dense, Dd, ld_dense,
                             reinterpret_cast<__nv_bfloat16*>(X0), ld, fm, lin_col, Lout);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}
const char* launch_deepfm_input_bwd(const float* U, int ustride, const int* inverse, int B, int S, int D, const void* dX0, int ld,
                                    const float* gfm, float* gU, int gstride, int lin_col, const float* dL, cudaStream_t st) {
  const int dq = D >> 2;
  if ((D & 3) || dq < 1 || dq > 32 || (dq & (dq - 1))) return "deepfm_input: embedding dim must be 4 * 2^k, at most 128";
  int blocks = (B + 7) / 8; if (blocks > 148 * 8) blocks = 148 * 8; if (blocks < 1) blocks = 1;
  cudaError_t e = launch_pdl(deepfm_input_bwd_kernel, dim3(blocks), dim3(256), 0, st, U, ustride, inverse, B, S, D,
                             reinterpret_cast<const __nv_bfloat16*>(dX0), ld, gfm, gU, gstride, lin_col, dL);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}
const char* launch_deepfm_head_loss(const void* H, int ldh, int NH, const float* L, int NL, const float* fm, const float* w,
                                    const float* label, int B, void* dH, float* dL, float* dfm, float* gw, float* sums, int nbins,
                                    float* pred, float* loss_out, float* scratch, cudaStream_t st) {
  if (ldh > 64 * kHeadPairs || (ldh & 1)) return "deepfm_head: hidden width must be even and at most 512 columns";
  if (NL > 32) return "deepfm_head: at most 32 linear inputs";
  if (NH + NL + 2 > kHeadPartStride) return "deepfm_head: too many head inputs";
  // two blocks per SM: measured 254 us per DeepFM step against 257 (three) and 264 (four), with scalar or 16-byte
  // reductions of the per-block weight gradient alike
  int blocks = (B + 7) / 8; if (blocks > 148 * 2) blocks = 148 * 2; if (blocks < 1) blocks = 1;
  cudaError_t e = launch_pdl(deepfm_head_loss_kernel, dim3(blocks), dim3(256), (NH + NL + 2) * sizeof(float), st,
                             reinterpret_cast<const __nv_bfloat16*>(H), ldh, NH, L, NL, fm, w, label, B,
                             reinterpret_cast<__nv_bfloat16*>(dH), dL, dfm, gw, sums, nbins, pred, loss_out, scratch);
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace tn
