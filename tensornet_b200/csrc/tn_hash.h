// Host/device shared arithmetic: key hashing, shard ownership, row layout and the
// counter-based row initialiser.  Included by both the g++-built CPU oracle and the
// nvcc-built sm_100a kernels so that the two produce the same table contents.
//
// Reference behaviour restated here:
//   * row owner            = sign % shard_num            (core/kernels/sparse_table_ops.cc:221)
//   * in-rank block        = ((sign>>32)|(sign<<32)) % 8  (core/ps/optimizer/optimizer_kernel.h:248-252,556)
//   * row init             = N(0, 1/sqrt(dim)) * initial_scale, zeros in inference mode
//                            (core/ps/optimizer/ada_grad_kernel.cc:78-103)
// The reference seeds its generator from the clock; here the value is a pure function of
// (table seed, sign, element) so CPU and GPU agree whatever the insertion order is.
#pragma once
#include <cstdint>
#include <cmath>

#if defined(__CUDACC__)
#define TN_HD __host__ __device__ __forceinline__
#else
#define TN_HD inline
#endif

namespace tn {

constexpr uint64_t kEmptyKey = 0xFFFFFFFFFFFFFFFFull;
constexpr int kSparseBlockNum = 8;

enum OptKind : int { kAdaGrad = 0, kAdam = 1, kFtrl = 2 };

TN_HD uint64_t mix64(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull;
  x ^= x >> 33;
  return x;
}

// The all-ones sign is the table's empty marker; it is folded onto its neighbour.
TN_HD uint64_t canon_key(uint64_t sign) { return sign == kEmptyKey ? kEmptyKey - 1 : sign; }

TN_HD int owner_of(uint64_t sign, int world) { return (int)(sign % (uint64_t)world); }
TN_HD int block_of(uint64_t sign) { return (int)(((sign >> 32) | (sign << 32)) % (uint64_t)kSparseBlockNum); }

TN_HD int round_up4(int x) { return (x + 3) & ~3; }

// Floats per stored row.  Layout (all fp32 unless noted):
//   AdaGrad: w[dim] | g2sum | show | click | no_show_days(int32)
//   Adam   : w[dim] | m[dim] | v[dim] | show | delta_show(int32)
//   Ftrl   : w[dim] | z[dim] | n[dim] | show | delta_show(int32)
TN_HD int row_floats(int kind, int dim) { return kind == kAdaGrad ? dim + 4 : 3 * dim + 2; }
TN_HD int row_stride(int kind, int dim) { return round_up4(row_floats(kind, dim)); }

TN_HD float u01_24(uint32_t x) { return ((float)(x & 0xFFFFFFu) + 0.5f) * (1.0f / 16777216.0f); }

// Element `i` of the initial weight vector of `sign`: Box-Muller over two 24-bit uniforms
// drawn from a hash of (seed, sign, i).  stddev = 1/sqrt(dim), then scaled.
TN_HD float init_weight(uint64_t seed, uint64_t sign, int i, int dim, float initial_scale) {
  uint64_t h = mix64(sign ^ mix64(seed + 0x9E3779B97F4A7C15ull * (uint64_t)(i + 1)));
  float u1 = u01_24((uint32_t)(h >> 40));
  float u2 = u01_24((uint32_t)(h >> 8));
  float r = sqrtf(-2.0f * logf(u1));
  float z = r * cosf(6.28318530717958647692f * u2);
  return z * (1.0f / sqrtf((float)dim)) * initial_scale;
}

struct SparseOptParams {
  int kind;             // OptKind
  float lr;
  float eps;
  float beta1, beta2;   // Adam
  float initial_g2sum;  // AdaGrad
  float initial_scale;
  float ftrl_beta, lambda1, lambda2;
  int zero_init;        // inference mode: new rows are all-zero
  uint64_t seed;
};

}  // namespace tn
