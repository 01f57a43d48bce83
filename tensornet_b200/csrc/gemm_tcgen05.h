// Host interface of the tcgen05 bf16 GEMM family (gemm_tcgen05.cu).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>

namespace tn {

// Problem description: C[M,N] (+)= epilogue( sum_k A(m,k) * B(n,k) ).
struct GemmDesc {
  int M = 0, N = 0, K = 0;
  const void* A = nullptr;   // bf16.  a_mn == 0: [M, K] row-major (lda >= K);  a_mn == 1: [K, M] row-major (lda >= M)
  const void* B = nullptr;   // bf16.  b_mn == 0: [N, K] row-major (ldb >= K);  b_mn == 1: [K, N] row-major (ldb >= N)
  int lda = 0, ldb = 0;
  int a_mn = 0, b_mn = 0;
  void* C = nullptr;         // bf16 or fp32 [M, ldc]
  int ldc = 0;
  int out_f32 = 0;
  int accumulate = 0;        // fp32 only: C += result (atomic vector adds, required for split_k > 1)
  int relu = 0;
  const float* bias = nullptr;      // optional fp32 [N], added before ReLU
  const void* mask_aux = nullptr;   // optional bf16 [M, ld_aux]: result is zeroed where mask_aux <= 0
  const void* had_x0 = nullptr;     // optional bf16 [M, ld_aux]: result = had_x0 * result + had_xl
  const void* had_xl = nullptr;     // with had_x0 == nullptr: result = result + had_xl (residual add)
  void* aux_out = nullptr;          // optional bf16 [M, ld_aux]: receives the result before the Hadamard step (acc + bias)
  int ld_aux = 0;
  int ones_col = -1;         // column (>= N) that is written as 1.0: the bias input of the next layer
  int n_store = 0;           // columns written per row (>= N; columns past N get 0, or 1 at ones_col)
  int split_k = 0;           // 0 = choose (only fp32 accumulate outputs may be split)
  int BN = 0;                // tile N override (0 = choose)
  int m_halves = 0;          // 128-row accumulators per CTA: 1, 2 (256-row tile sharing one B tile) or 0 = choose
  // Weight gate ("all-gather fused with the GEMM"): the B operand lives in an array whose chunks other GPUs
  // write during the dense optimizer step.  When gate_flags is set the TMA producer first waits (bounded) until
  // each of the gate_world flag words carries at least the epoch stored at *gate_epoch in its high 32 bits, then
  // orders the asynchronous proxy behind those writes.  The operand itself is always read from local memory.
  const unsigned long long* gate_flags = nullptr;
  const unsigned long long* gate_epoch = nullptr;
  int gate_world = 0;
  unsigned long long gate_wait_ns = 0;
  int* status = nullptr;     // device error words
  unsigned long long* prof = nullptr;   // optional [16] timestamps of CTA (0,0,0) for pipeline diagnosis
};

// Kernel-side parameter block.
struct GemmParams {
  int M, N, K, BN, a_mn, b_mn, k_tiles_per_split, m_halves, raster_group;
  void* C;
  int ldc, out_f32, accumulate, relu;
  const __nv_bfloat16* mask_aux;
  const __nv_bfloat16* had_x0;
  const __nv_bfloat16* had_xl;
  __nv_bfloat16* aux_out;
  int ld_aux, ones_col, n_store;
  const float* bias;
  const unsigned long long* gate_flags;
  const unsigned long long* gate_epoch;
  int gate_world;
  unsigned long long gate_wait_ns;
  int* status;
  unsigned long long* prof;
};

// Returns nullptr on success, otherwise a static error string.
const char* gemm_bf16(const GemmDesc& d, cudaStream_t stream);

}  // namespace tn
