// Host interface of the one-kernel MLP tower (mlp_fused.cu).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>

namespace tn {

constexpr int kMlpMaxLayers = 4;

// One step of a chain.  W is the layer's bf16 weight matrix [n_rows, ldw] (row n = output feature n, column k = input
// feature k, the bias in column K of the augmented input).
//   forward  chain: out[M, ld_out] = relu?(in[:, :k_cols] . W[:, :k_cols]^T), column n_rows := 1, later columns := 0
//   backward chain: out[M, ld_out] = in[:, :n_rows] . W[:, :k_cols], columns >= n_valid := 0, masked by mask > 0
struct MlpChainLayer {
  const void* w = nullptr;
  int n_rows = 0, k_cols = 0, ldw = 0;
  void* out = nullptr;       // bf16 [M, ld_out]
  int ld_out = 0;
  int relu = 0;              // forward only
  int n_valid = 0;           // backward only
  const void* mask = nullptr;   // backward only: bf16 [M, ld_mask], the forward activation this gradient belongs to
  int ld_mask = 0;
};

struct MlpChainDesc {
  int L = 0;
  int M = 0;
  int backward = 0;
  const void* in = nullptr;  // bf16 [M, ld_in]: chain input (forward: with the constant-one column; backward: dL/d(output))
  int in_cols = 0, ld_in = 0;
  MlpChainLayer layer[kMlpMaxLayers];     // in the order the chain visits them
  // as in GemmDesc: the first weight tile waits until every owner's chunk of the dense array has landed
  const unsigned long long* gate_flags = nullptr;
  const unsigned long long* gate_epoch = nullptr;
  int gate_world = 0;
  unsigned long long gate_wait_ns = 0;
  int split = 0;             // 0 = choose, 1 = one CTA per stripe, 2 = a pair of CTAs per stripe
  int* status = nullptr;
  unsigned long long* prof = nullptr;   // optional [16] timestamps of CTA 0: start, data ready, then per step: A ready, accumulator ready, epilogue done
};

struct MlpChainParams {
  int L, M, backward, kt_in, kt_max;
  int split;                     // CTAs per 128-row stripe: 1, or 2 (a cluster of two that share the stripe's output columns)
  int stages;                    // weight tiles in flight
  uint32_t stage_bytes;
  int n_lo[kMlpMaxLayers][2];    // first accumulator column of CTA r of a stripe in step i
  int n_cnt[kMlpMaxLayers][2];   // its number of accumulator columns
  int n_acc[kMlpMaxLayers];      // accumulator columns of step i (all CTAs of a stripe together)
  int n_valid[kMlpMaxLayers];    // columns that take accumulator values
  int ones_col[kMlpMaxLayers];   // column written as 1.0 (-1: none)
  int out_cols[kMlpMaxLayers];   // columns written to the next A operand (multiple of 64)
  int kt[kMlpMaxLayers];         // k-blocks contracted in step i
  int box_rows[kMlpMaxLayers][2];   // rows per weight TMA copy (forward), per CTA of a stripe
  int relu[kMlpMaxLayers];
  const __nv_bfloat16* mask[kMlpMaxLayers];
  int ld_mask[kMlpMaxLayers];
  const unsigned long long* gate_flags;
  const unsigned long long* gate_epoch;
  int gate_world;
  unsigned long long gate_wait_ns;
  int* status;
  unsigned long long* prof;
};

// nullptr when the tower fits the one-kernel path, otherwise the reason it does not
const char* mlp_chain_supported(const MlpChainDesc& d);
// Returns nullptr on success, otherwise a static error string.
const char* mlp_chain(const MlpChainDesc& d, cudaStream_t stream);

}  // namespace tn
