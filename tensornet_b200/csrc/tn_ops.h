// Host-callable launchers of the non-fused kernels.  All take raw device pointers and a
// stream so the translation units that define them do not need the PyTorch headers.
#pragma once
#include <cuda_runtime.h>
#include "tn_types.h"

namespace tn {

// pooling.cu
void launch_pool_fwd(const float* U, int ustride, const int* inverse, const int* offsets, int B, int S, int pd,
                     int combiner, float* out, int out_ld, cudaStream_t st);
void launch_pool_bwd(float* gU, int gstride, const int* inverse, const int* offsets, int B, int S, int pd, int dim,
                     int combiner, const float* gout, int gout_ld, cudaStream_t st);
void launch_seq_fwd(const float* U, int ustride, const int* inverse, const int* offsets, int B, int T, int pd,
                    float* out, int* lengths, cudaStream_t st);
void launch_seq_bwd(float* gU, int gstride, const int* inverse, const int* offsets, int B, int T, int pd, int dim,
                    const float* gout, cudaStream_t st);

// table_ops.cu
void launch_table_insert_keys(const TableView& t, const long long* keys, int n, int* out_rows, int* status, cudaStream_t st);
void launch_table_lookup(const TableView& t, const long long* keys, int n, int* out_rows, cudaStream_t st);
void launch_table_decay(const TableView& t, int kind, float rate, int delta_days, cudaStream_t st);
void launch_table_rebuild_index(const TableView& t, int n, int* status, cudaStream_t st);
void launch_table_keep_mask(const TableView& t, int kind, const ExportRule& rule, int n, unsigned char* keep, cudaStream_t st);
void launch_table_export(const TableView& t, int kind, const ExportRule& rule, int r0, int r1, int* counts, int* cursors,
                         unsigned long long* out_keys, float* out_rows, int rf, cudaStream_t st);

// elementwise.cu
constexpr int kMaxPieces = 6;
struct ConcatArgs {
  int B;
  int n_pieces;
  const void* ptr[kMaxPieces];   // piece p: [B, width[p]] with row stride ld[p], fp32 or bf16
  int width[kMaxPieces];
  int ld[kMaxPieces];
  int is_bf16[kMaxPieces];
  void* out;                     // bf16 [B, ld_out]; columns past the pieces are 0, ones_col is 1
  int ld_out;
  int ones_col;                  // -1 for none
};
void launch_fm_fwd(const float* E, int ld, int B, int F, int D, float* out, cudaStream_t st);
void launch_fm_bwd(const float* E, int ld, int B, int F, int D, const float* gout, float* gE, int gld, int accumulate, cudaStream_t st);
void launch_concat_cast(const ConcatArgs& a, cudaStream_t st);
void launch_split_cast(const ConcatArgs& a, cudaStream_t st);
void launch_gemv_fwd(const void* Z, int ld, int B, int K, const float* w, float* y, cudaStream_t st);
void launch_gemv_bwd(const void* Z, int ld, int B, int K, const float* w, const float* dy, void* dZ, float* gw, int relu_cols,
                     cudaStream_t st);
void launch_bce(const float* logit, const float* label, int B, float* pred, float* dlogit, float grad_scale, float* sums,
                int nbins, cudaStream_t st);
void launch_cross_v1_fwd(const float* x0, const float* xl, const float* w, const float* bias, int B, int D, float* y, float* dot,
                         cudaStream_t st);
void launch_cross_v1_bwd(const float* x0, const float* xl, const float* w, const float* dot, const float* gy, int B, int D,
                         float* gx0, float* gxl, float* gw, float* gb, cudaStream_t st);
void launch_relu_mask(void* g, const void* y, long long n, cudaStream_t st);
void launch_cross_v2_bwd_elem(const void* g, const void* u, const void* x0, float* gx0, void* du, long long n, int first, cudaStream_t st);
void launch_cross_v2_bwd_final(const float* gx0, const void* g, void* out, long long n, cudaStream_t st);

// deepfm_fused.cu  (return nullptr or a static error string)
const char* launch_deepfm_input_fwd(const float* U, int ustride, const int* inverse, int B, int S, int D, const float* dense, int Dd,
                                    int ld_dense, void* X0, int ld, float* fm, int lin_col, float* Lout, cudaStream_t st);
const char* launch_deepfm_input_bwd(const float* U, int ustride, const int* inverse, int B, int S, int D, const void* dX0, int ld,
                                    const float* gfm, float* gU, int gstride, int lin_col, const float* dL, cudaStream_t st);
const char* launch_deepfm_head_loss(const void* H, int ldh, int NH, const float* L, int NL, const float* fm, const float* w,
                                    const float* label, int B, void* dH, float* dL, float* dfm, float* gw, float* sums, int nbins,
                                    float* pred, float* loss_out, float* scratch, cudaStream_t st);

// unique.cu
void launch_unique_assign(const long long* ids, int n, const float* labels, unsigned long long* dd_keys, int* dd_vals,
                          unsigned scratch_cap, unsigned long long* uniq, int cap, int* inverse, float* show, float* click,
                          int* count, int* status, cudaStream_t st);

// bn.cu
void launch_bn_batch_stats(const float* x, int ld, int B, int C, const float* center, double* batch, cudaStream_t st);
void launch_bn_table_append(const BnTableView& t, double* batch, cudaStream_t st);
void launch_bn_table_refresh(const BnTableView& t, cudaStream_t st);
void launch_bn_table_sync(const BnTableView& t, const BnSyncView& s, double* scratch, cudaStream_t st);
void launch_bn_apply_fwd(const float* x, int ldx, int B, int C, const float* mean, const float* var, const float* gamma,
                         const float* beta, float eps, float* y, int ldy, cudaStream_t st);
void launch_bn_apply_bwd(const float* dy, int ldd, const float* x, int ldx, int B, int C, const float* mean, const float* var,
                         const float* gamma, float eps, float* dx, int ldo, float* gg, float* gb, cudaStream_t st);

// serving.cu
void launch_dict_lookup_pool(const TableView& t, const long long* ids, const int* offsets, int B, int S, int combiner, void* out,
                             int ld_out, int ones_col, cudaStream_t st);
void launch_sigmoid(const float* x, float* y, int n, cudaStream_t st);

}  // namespace tn
