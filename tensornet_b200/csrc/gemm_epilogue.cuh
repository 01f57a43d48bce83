// Epilogue of the tcgen05 bf16 GEMM kernels (gemm_tcgen05.cu, gemm_2sm.cu): one warp drains its 32 TMEM lanes of an
// accumulator, applies the fused epilogue (bias, ReLU, ReLU mask of the backward pass, "ones" bias column,
// Hadamard / residual step of DCN-v2, fp32 accumulate) and writes whole 64-byte row segments to global memory.
#pragma once
#include "gemm_tcgen05.h"
#include "tc_primitives.cuh"

namespace tn {
namespace gemm_epi {

constexpr int kBytesPerWarp = 6144;   // out block + two auxiliary blocks of 32 rows x 64 B

// `tm_lane`: TMEM address of the warp's lane quarter at the accumulator's first column; `row_base`: global row of
// TMEM lane 0 of that quarter; `n0`: global column of accumulator column 0; the warp takes column chunks
// sub, sub + nsubs, ... (32 columns each for bf16 outputs, 16 for fp32); `sm_out`: kBytesPerWarp bytes of shared
// memory private to the warp.  TMEM gives a lane one ROW of the tile, global memory wants a warp on whole lines:
// blocks of 32 rows x 64 bytes go through shared memory (16-byte pieces, XOR-swizzled so both the row-wise writes
// and the line-wise reads are bank-conflict free) and leave as 64-byte row segments, eight rows per store.
__device__ __forceinline__ void store_rows(const GemmParams& p, uint32_t tm_lane, int row_base, int n0, int BN, int sub,
                                           int nsubs, int lane, uint8_t* sm_out) {
  using namespace tc;
  uint8_t* sm_a0 = sm_out + 2048;
  uint8_t* sm_a1 = sm_out + 4096;
  const int n_store = p.n_store;
  const int lrow = lane >> 2, lpc = lane & 3;          // line-wise mapping: 4 lanes per row
  const bool has_aux = p.mask_aux != nullptr || p.had_x0 != nullptr || p.had_xl != nullptr;
  const bool has_bias = p.bias != nullptr, relu = p.relu != 0;
  const int my_off = lane * 64;
  const int my_sw = (lane >> 1) & 3;
  if (!p.out_f32) {
    // auxiliary operands of chunk c0 (ReLU mask, or x0 / xl of the Hadamard step): global -> registers
    auto load_aux = [&](int c0, uint4* va, uint4* vb) {
      if (!has_aux) return;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = 8 * i + lrow;
        const int grow = row_base + r, gcol = n0 + c0 + lpc * 8;
        va[i] = make_uint4(0u, 0u, 0u, 0u);
        vb[i] = va[i];
        if (grow < p.M && gcol + 8 <= p.ld_aux) {
          const size_t off = (size_t)grow * p.ld_aux + gcol;
          if (p.mask_aux) va[i] = *reinterpret_cast<const uint4*>(p.mask_aux + off);
          else {
            if (p.had_x0) va[i] = *reinterpret_cast<const uint4*>(p.had_x0 + off);
            vb[i] = *reinterpret_cast<const uint4*>(p.had_xl + off);
          }
        }
      }
    };
    // registers -> the warp's shared-memory blocks, where the row-wise pass below finds them
    auto stash_aux = [&](const uint4* va, const uint4* vb) {
      if (!has_aux) return;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = 8 * i + lrow;
        const int so = r * 64 + ((lpc ^ ((r >> 1) & 3)) << 4);
        *reinterpret_cast<uint4*>(sm_a0 + so) = va[i];
        if (!p.mask_aux) *reinterpret_cast<uint4*>(sm_a1 + so) = vb[i];
      }
      __syncwarp();
    };
    auto issue_acc = [&](int c0, uint32_t* acc) {
      tmem_ld16_nowait(tm_lane + (uint32_t)c0, acc);
      if (c0 + 16 < BN) tmem_ld16_nowait(tm_lane + (uint32_t)(c0 + 16), acc + 16);
      else {
#pragma unroll
        for (int j = 16; j < 32; ++j) acc[j] = 0u;
      }
    };
    // epilogue math of chunk c0 on the loaded accumulators, then the line-wise stores
    auto finish = [&](int c0, const uint32_t* acc) {
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) {
        const int nb = n0 + c0 + pc * 8;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(acc[pc * 8 + j]);
        if (has_bias) {
#pragma unroll
          for (int j = 0; j < 8; ++j) if (nb + j < p.N) v[j] += __ldg(p.bias + nb + j);
        }
        if (relu) {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.f);
        }
        const int so = my_off + ((pc ^ my_sw) << 4);
        if (has_aux) {
          const uint4 a0 = *reinterpret_cast<const uint4*>(sm_a0 + so);
          const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&a0);
          if (p.mask_aux) {   // backward of ReLU: keep the gradient where the forward activation was positive
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 m2 = __bfloat1622float2(h0[k]);
              if (!(m2.x > 0.f)) v[2 * k] = 0.f;
              if (!(m2.y > 0.f)) v[2 * k + 1] = 0.f;
            }
          } else {            // DCN-v2: x0 * (acc + bias) + xl, or just + xl when there is no x0
            const uint4 a1 = *reinterpret_cast<const uint4*>(sm_a1 + so);
            const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&a1);
            if (p.aux_out) {  // keep u = acc + bias for the backward pass; this lane owns the slot it just read
              *reinterpret_cast<uint4*>(sm_a1 + so) =
                  make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
            }
            if (p.had_x0) {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float2 x0 = __bfloat1622float2(h0[k]), xl = __bfloat1622float2(h1[k]);
                v[2 * k] = x0.x * v[2 * k] + xl.x;
                v[2 * k + 1] = x0.y * v[2 * k + 1] + xl.y;
              }
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float2 xl = __bfloat1622float2(h1[k]);
                v[2 * k] += xl.x;
                v[2 * k + 1] += xl.y;
              }
            }
          }
        }
        if (nb + 8 > p.N) {   // only the piece that straddles N pays for the ones / padding columns
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int n = nb + j;
            if (n >= p.N) v[j] = (n == p.ones_col) ? 1.f : 0.f;
          }
        }
        *reinterpret_cast<uint4*>(sm_out + so) =
            make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
      }
      __syncwarp();
      const int gcol = n0 + c0 + lpc * 8;
      const bool col_ok = gcol < n_store && c0 + lpc * 8 < BN;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = 8 * i + lrow;
        const int grow = row_base + r;
        if (grow < p.M && col_ok) {
          const int sl = r * 64 + ((lpc ^ ((r >> 1) & 3)) << 4);
          const uint4 o = *reinterpret_cast<const uint4*>(sm_out + sl);
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)grow * p.ldc + gcol;
          if (gcol + 8 <= n_store) {
            *reinterpret_cast<uint4*>(dst) = o;
          } else {
            const __nv_bfloat16* ob = reinterpret_cast<const __nv_bfloat16*>(&o);
            for (int j = 0; j < n_store - gcol; ++j) dst[j] = ob[j];
          }
          if (p.aux_out && gcol + 8 <= p.ld_aux)
            *reinterpret_cast<uint4*>(p.aux_out + (size_t)grow * p.ld_aux + gcol) = *reinterpret_cast<const uint4*>(sm_a1 + sl);
        }
      }
      __syncwarp();
    };
    const int step = 32 * nsubs;
    auto live = [&](int c0) { return c0 < BN && n0 + c0 < n_store; };      // warp-uniform
    for (int c0 = 32 * sub; live(c0); c0 += step) {
      uint4 va[4], vb[4];
      uint32_t acc[32];
      load_aux(c0, va, vb);
      stash_aux(va, vb);
      issue_acc(c0, acc);
      tmem_ld_wait();
      finish(c0, acc);
    }
  } else {
    auto finish32 = [&](int c0, const uint32_t* acc) {
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) {
        const int nb = n0 + c0 + pc * 4;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[j] = __uint_as_float(acc[pc * 4 + j]);
          if (has_bias && nb + j < p.N) v[j] += __ldg(p.bias + nb + j);
          if (relu) v[j] = fmaxf(v[j], 0.f);
          if (nb + j >= p.N) v[j] = (nb + j == p.ones_col) ? 1.f : 0.f;
        }
        *reinterpret_cast<float4*>(sm_out + my_off + ((pc ^ my_sw) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
      }
      __syncwarp();
      const int gcol = n0 + c0 + lpc * 4;
      const bool col_ok = gcol < n_store && c0 + lpc * 4 < BN;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = 8 * i + lrow;
        const int grow = row_base + r;
        if (grow < p.M && col_ok) {
          const float4 o = *reinterpret_cast<const float4*>(sm_out + r * 64 + ((lpc ^ ((r >> 1) & 3)) << 4));
          float* dst = reinterpret_cast<float*>(p.C) + (size_t)grow * p.ldc + gcol;
          if (gcol + 4 <= n_store) {
            if (p.accumulate) red_add_f32x4(dst, o); else *reinterpret_cast<float4*>(dst) = o;
          } else {
            const float ov[4] = {o.x, o.y, o.z, o.w};
            for (int j = 0; j < n_store - gcol; ++j) {
              if (p.accumulate) atomicAdd(dst + j, ov[j]); else dst[j] = ov[j];
            }
          }
        }
      }
      __syncwarp();
    };
    const int step = 16 * nsubs;
    auto live = [&](int c0) { return c0 < BN && n0 + c0 < n_store; };      // warp-uniform
    for (int c0 = 16 * sub; live(c0); c0 += step) {
      uint32_t acc[16];
      tmem_ld16_nowait(tm_lane + (uint32_t)c0, acc);
      tmem_ld_wait();
      finish32(c0, acc);
    }
  }
}

}  // namespace gemm_epi
}  // namespace tn
