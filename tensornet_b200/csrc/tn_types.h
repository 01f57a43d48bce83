// Plain-old-data views passed by value to kernels; includable from host-only code.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "tn_hash.h"

namespace tn {

constexpr int kMaxWorld = 8;

// Lanes cooperating on one row: power of two >= ceil(width/4), at most 32.
inline int lanes_for_width_host(int width_floats) {
  int chunks = (width_floats + 3) / 4, g = 1;
  while (g < chunks && g < 32) g <<= 1;
  return g;
}

// Open-addressing key array -> row index into a dense row slab.
struct TableView {
  unsigned long long* keys;      // [cap]  kEmptyKey when free
  int* slots;                    // [cap]  row index, -1 until the inserter publishes it
  float* rows;                   // [row_cap * stride]
  unsigned long long* row_keys;  // [row_cap] sign owning each row (for dump / rebuild)
  unsigned long long* row_tag;   // [row_cap] (epoch << 32) | kTagNew | owner-unique index of the step
  int* n_rows;                   // rows in use
  unsigned cap_mask;             // cap - 1 (cap is a power of two)
  int row_cap;
  int dim;
  int stride;                    // floats per row
  int use_cvm;                   // pulled rows carry two extra columns (show, ln(click+1)-ln(show+1))
};

// Per-table exchange state.  Arrays indexed by peer hold that peer's copy of a buffer in the
// symmetric heap (entry [rank] is this GPU's own copy); the rest is private to this GPU.
struct SparseCommView {
  int world, rank;
  int capo;      // capacity of one (sender, owner) segment, in unique signs; multiple of 4
  int gstride;   // floats per gradient record: round_up4(dim + 2)  = grad[dim] | show | click
  int ustride;   // floats per pulled row: round_up4(dim + 2 * use_cvm)
  unsigned long long* inbox_ids[kMaxWorld];  // [sender][capo]            written by senders
  float* gU_peer[kMaxWorld];                 // [owner][capo][gstride]    every GPU's gradient records; owners read their segment of each
  float* cnts_peer[kMaxWorld];               // [owner][capo][2]          (show, click) of each record, likewise
  float* U[kMaxWorld];                       // [owner][capo][ustride]    written by owners
  unsigned long long* sig[kMaxWorld];        // [4][kMaxWorld] flag words (epoch << 32 | payload)
  unsigned long long* stage_ids;             // [owner][capo] outgoing signs, grouped by owner
  float* gU;                                 // [owner][capo][gstride] gradient wrt the pulled rows
  float* cnts;                               // [owner][capo][2] show / click counts of the batch per distinct sign
  int* cnt;                                  // [world] running per-owner unique counts (zero between steps)
  int* cnt_saved;                            // [world] per-owner unique counts of the current step
  int* req_n;                                // [world] as owner: number of signs requested by each sender
  int* req_row;                              // [sender][capo] as owner: row of each request (+flags)
  int* req_ou;                               // [sender][capo] as owner: owner-unique index of each request
  int* ou_row;                               // [world*capo]   owner-unique index -> row (or -1 for a hole)
  int* ocount;                               // number of owner-unique indices handed out this step
  float* acc;                                // [world*capo][gstride] gradient accumulator (zero between steps)
  unsigned long long* dd_keys;               // per-batch dedup scratch (all kEmptyKey between steps)
  int* dd_vals;
  unsigned dd_mask;
  unsigned long long* epoch;                 // step counter of the table
  unsigned* bar;                             // [2] grid barrier words (zero between launches)
  int* status;                               // [4] error words
  unsigned long long wait_ns;                // budget of every wait inside the kernels
  unsigned long long* prof;                  // optional [16] phase timestamps (globaltimer ns) by CTA 0: pull 0..5 (6 = slowest CTA's end of the row return), push 8..13 (14 / 15 = after the own records / after the wait for the peers)
};

struct PullArgs {
  SparseCommView c;
  TableView tbl;
  const TableView* tbl_dev;   // when not null: the same descriptor in device memory, read at kernel start instead of `tbl`
  SparseOptParams opt;
  const long long* ids;   // [n_ids] raw signs of the batch (all columns of the layer)
  int n_ids;
  int* inverse;           // [n_ids] out: virtual row (owner * capo + position) of every id
  const float* labels;    // optional click labels: labels[i % label_mod] (label_mod > 0) or labels[i]
  int label_mod;
  int training;           // count show/click and prepare the push bookkeeping
  int lookup_only;        // never insert: signs the table does not hold come back as zero rows (serving)
  int lanes;              // lanes per row in the row-copy phase
  int tile_rows;          // > 0: rows per shared-memory tile of the staged row return; capo is a multiple of it
  int front_done;         // dedup, id dispatch and inverse map of this batch already ran (launch_sparse_pull_front)
};

struct PushArgs {
  SparseCommView c;
  TableView tbl;
  const TableView* tbl_dev;   // as in PullArgs
  SparseOptParams opt;
  int lanes;
};

// Dense optimizer hyper-parameters.  kind 0 = Adam (TF-style running beta powers), 1 = AdaGrad.
struct DenseOptParams {
  int kind;
  float beta1, beta2, eps;
  float grad_decay, mom_decay;   // AdaGrad
  float* state;                  // device: [0]=beta1^t [1]=beta2^t [2]=learning rate [3]=ticket (u32)
};

struct DenseStepArgs {
  DenseOptParams opt;
  long long n;          // padded length of the flat array (multiple of 4)
  long long chunk;      // elements owned per GPU (multiple of 4); n for world == 1
  int world, rank;
  float grad_scale;     // 1/world for the mean gradient
  int skip_open;        // world > 1: this launch does not need the opening "gradients ready" barrier (see dense_fused.cu)
  int max_ctas;         // world > 1: cap on the cooperative grid (0 = fill the GPU); a small cap leaves SMs to a kernel on another stream
  int gated;            // world > 1: publish per-owner "chunk written" flags (row 2 of sig) instead of waiting in a closing barrier;
                        // the first kernel that reads the weights waits on them (GemmDesc::gate_flags)
  int zero_local;       // world > 1: each GPU clears its own gradient replica after the closing barrier
  float* W[kMaxWorld];  // fp32 master replica of every GPU
  float* G[kMaxWorld];  // fp32 gradient of every GPU
  void* Wb[kMaxWorld];  // bf16 shadow of every GPU (may be null)
  float* W_mc;          // NVSwitch multicast mappings of the same three arrays, or null
  float* G_mc;
  void* Wb_mc;
  float* s0;            // optimizer state of the owned chunk: Adam m | AdaGrad d2sum
  float* s1;            //                                      Adam v | AdaGrad g2sum
  float* s2;            //                                               AdaGrad m
  unsigned long long* sig[kMaxWorld];   // [3][kMaxWorld] flag words per GPU: gradients ready, weights written (barrier), weights written (gate)
  unsigned long long* epoch;
  unsigned* bar;
  int* status;
  unsigned long long wait_ns;
};

// Save-time eviction rule (the reference's DeleteByShow): AdaGrad rows go when `show < show_threshold`
// or / and (logic 0 / 1) `no_show_days > no_show_days`; Ftrl rows when `show < show_threshold`.
struct ExportRule {
  int enabled;
  float show_threshold;
  int no_show_days;
  int logic;
};

// Device-resident batch-norm statistics table (all arrays have C entries unless noted).
struct BnTableView {
  int C;
  int pctr;                 // 1: squared sums are deviations from the current mean and `var` reports them raw
  double moment;            // moving-window momentum
  long long max_count;      // records after which the window starts sliding (0 = never)
  double* total_sum;
  double* total_sum_err;    // Kahan compensation terms
  double* total_sq;
  double* total_sq_err;
  double* total_count;
  double* inc;              // [3][C] pending increments (sum, squared sum, count) for the cross-GPU exchange
  float* mean;              // moments the layer normalises with
  float* var;
};
struct BnSyncView {
  int world, rank;
  const double* inc[kMaxWorld];          // every GPU's pending increments
  unsigned long long* sig[kMaxWorld];    // [2][kMaxWorld] flag words per GPU
  unsigned long long* epoch;
  int* status;
  unsigned long long wait_ns;
};

// Dedup, id dispatch to the owners and inverse map of a batch as plain (non-cooperative) kernels, to be run on a
// second stream under the previous step's forward / backward; the pull of that batch then runs with front_done = 1.
cudaError_t launch_sparse_pull_front(const PullArgs& args, cudaStream_t stream);
cudaError_t launch_dense_step(const DenseStepArgs& a, cudaStream_t st);
int dense_step_ctas_per_sm();      // resident CTAs of the multi-GPU dense kernel per SM
cudaError_t launch_sparse_pull(const PullArgs& args, int work_items, cudaStream_t stream);
cudaError_t launch_sparse_push(const PushArgs& args, int work_items, int max_ctas, const DenseStepArgs* dense, cudaStream_t stream);

}  // namespace tn
