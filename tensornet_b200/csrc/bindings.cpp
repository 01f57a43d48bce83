// Python bindings of the sm_100a kernels (module tensornet_b200._ext._tn_cuda).
// Storage is owned by torch tensors created on the Python side; the objects here only keep
// raw device pointers (plus a reference to the tensors) so a kernel launch costs one call.
#include <torch/extension.h>
#include <ATen/cuda/CachingHostAllocator.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cstring>
#include <string>
#include <vector>

#include "gemm_tcgen05.h"
#include "mlp_fused.h"
#include "tn_ops.h"
#include "tn_types.h"

namespace py = pybind11;

namespace {

template <typename T>
T* ptr_of(const at::Tensor& t) { return reinterpret_cast<T*>(t.data_ptr()); }
template <typename T>
T* ptr_of(int64_t p) { return reinterpret_cast<T*>(static_cast<uintptr_t>(p)); }

// Every binding that launches a kernel fetches the stream exactly once, so this doubles as the
// count of kernels this library has launched (or recorded into a CUDA graph).
std::atomic<long long> g_launches{0};
cudaStream_t cur_stream() {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return at::cuda::getCurrentCUDAStream().stream();
}

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

tn::SparseOptParams opt_from_dict(const py::dict& d) {
  tn::SparseOptParams o{};
  o.kind = d["kind"].cast<int>();
  o.lr = d["lr"].cast<float>();
  o.eps = d["eps"].cast<float>();
  o.beta1 = d["beta1"].cast<float>();
  o.beta2 = d["beta2"].cast<float>();
  o.initial_g2sum = d["initial_g2sum"].cast<float>();
  o.initial_scale = d["initial_scale"].cast<float>();
  o.ftrl_beta = d["ftrl_beta"].cast<float>();
  o.lambda1 = d["lambda1"].cast<float>();
  o.lambda2 = d["lambda2"].cast<float>();
  o.zero_init = d["zero_init"].cast<int>();
  o.seed = d["seed"].cast<uint64_t>();
  return o;
}

tn::TableView table_from_dict(const py::dict& d) {
  tn::TableView t{};
  t.keys = ptr_of<unsigned long long>(d["keys"].cast<at::Tensor>());
  t.slots = ptr_of<int>(d["slots"].cast<at::Tensor>());
  t.rows = ptr_of<float>(d["rows"].cast<at::Tensor>());
  t.row_keys = ptr_of<unsigned long long>(d["row_keys"].cast<at::Tensor>());
  t.row_tag = ptr_of<unsigned long long>(d["row_tag"].cast<at::Tensor>());
  t.n_rows = ptr_of<int>(d["n_rows"].cast<at::Tensor>());
  int64_t cap = d["keys"].cast<at::Tensor>().numel();
  TORCH_CHECK(cap > 0 && (cap & (cap - 1)) == 0, "table capacity must be a power of two");
  t.cap_mask = (unsigned)(cap - 1);
  t.row_cap = (int)d["row_keys"].cast<at::Tensor>().numel();
  t.dim = d["dim"].cast<int>();
  t.stride = d["stride"].cast<int>();
  t.use_cvm = d["use_cvm"].cast<int>();
  return t;
}

// One embedding table + its exchange buffers.
struct SparseCtx {
  tn::SparseCommView c{};
  tn::TableView t{};
  tn::SparseOptParams o{};
  int pull_lanes = 1, push_lanes = 1;
  int tile_rows = 0;   // staged row return of the pull (0 = rows go straight to the requester's matrix)
  py::dict keep;   // keeps the tensors alive
  at::Tensor tbl_dev;  // the table descriptor in device memory (what launches inside CUDA graphs read)

  void upload_table() {
    if (!tbl_dev.defined()) {
      at::Tensor rows = keep["table"].cast<py::dict>()["rows"].cast<at::Tensor>();
      tbl_dev = at::empty({(int64_t)((sizeof(tn::TableView) + 7) / 8)}, at::TensorOptions().dtype(at::kLong).device(rows.device()));
    }
    // stream-ordered with the launches around it; the source is copied out before the call returns (pageable memory)
    check(cudaMemcpyAsync(tbl_dev.data_ptr(), &t, sizeof(tn::TableView), cudaMemcpyHostToDevice, at::cuda::getCurrentCUDAStream().stream()),
          "table descriptor upload");
  }

  SparseCtx(py::dict table, py::dict comm, py::dict opt) {
    keep["table"] = table; keep["comm"] = comm;
    t = table_from_dict(table);
    upload_table();
    o = opt_from_dict(opt);
    c.world = comm["world"].cast<int>();
    c.rank = comm["rank"].cast<int>();
    c.capo = comm["capo"].cast<int>();
    c.gstride = comm["gstride"].cast<int>();
    c.ustride = comm["ustride"].cast<int>();
    TORCH_CHECK(c.world >= 1 && c.world <= tn::kMaxWorld, "world must be 1..8");
    TORCH_CHECK(c.capo % 4 == 0, "segment capacity must be a multiple of 4");
    auto inbox = comm["inbox_ids"].cast<std::vector<int64_t>>();
    auto gU_peer = comm["gU_peer"].cast<std::vector<int64_t>>();
    auto cnts_peer = comm["cnts_peer"].cast<std::vector<int64_t>>();
    auto U = comm["U"].cast<std::vector<int64_t>>();
    auto sig = comm["sig"].cast<std::vector<int64_t>>();
    TORCH_CHECK((int)inbox.size() == c.world && (int)gU_peer.size() == c.world && (int)cnts_peer.size() == c.world && (int)U.size() == c.world &&
                    (int)sig.size() == c.world, "peer pointer tables must have `world` entries");
    for (int p = 0; p < c.world; ++p) {
      c.inbox_ids[p] = ptr_of<unsigned long long>(inbox[p]);
      c.gU_peer[p] = ptr_of<float>(gU_peer[p]);
      c.cnts_peer[p] = ptr_of<float>(cnts_peer[p]);
      c.U[p] = ptr_of<float>(U[p]);
      c.sig[p] = ptr_of<unsigned long long>(sig[p]);
    }
    c.stage_ids = ptr_of<unsigned long long>(comm["stage_ids"].cast<at::Tensor>());
    c.gU = ptr_of<float>(comm["gU"].cast<at::Tensor>());
    c.cnts = ptr_of<float>(comm["cnts"].cast<at::Tensor>());
    c.cnt = ptr_of<int>(comm["cnt"].cast<at::Tensor>());
    c.cnt_saved = ptr_of<int>(comm["cnt_saved"].cast<at::Tensor>());
    c.req_n = ptr_of<int>(comm["req_n"].cast<at::Tensor>());
    c.req_row = ptr_of<int>(comm["req_row"].cast<at::Tensor>());
    c.req_ou = ptr_of<int>(comm["req_ou"].cast<at::Tensor>());
    c.ou_row = ptr_of<int>(comm["ou_row"].cast<at::Tensor>());
    c.ocount = ptr_of<int>(comm["ocount"].cast<at::Tensor>());
    c.acc = ptr_of<float>(comm["acc"].cast<at::Tensor>());
    at::Tensor ddk = comm["dd_keys"].cast<at::Tensor>();
    int64_t ddcap = ddk.numel();
    TORCH_CHECK(ddcap >= 2 && (ddcap & (ddcap - 1)) == 0, "dedup scratch must be a power of two");
    c.dd_keys = ptr_of<unsigned long long>(ddk);
    c.dd_vals = ptr_of<int>(comm["dd_vals"].cast<at::Tensor>());
    c.dd_mask = (unsigned)(ddcap - 1);
    c.epoch = ptr_of<unsigned long long>(comm["epoch"].cast<at::Tensor>());
    c.bar = ptr_of<unsigned>(comm["bar"].cast<at::Tensor>());
    c.status = ptr_of<int>(comm["status"].cast<at::Tensor>());
    c.wait_ns = comm["wait_ns"].cast<uint64_t>();
    c.prof = comm.contains("prof") && !comm["prof"].is_none() ? ptr_of<unsigned long long>(comm["prof"].cast<at::Tensor>()) : nullptr;
    pull_lanes = tn::lanes_for_width_host((c.ustride + 3) / 4);   // each lane keeps up to four 16-byte chunks in flight
    {
      // Lanes per row in the row update.  Fewer lanes per row = more rows in flight per warp, which is what the
      // update is short of (dependent random accesses): with 1 M ids per batch, two 16-byte chunks per lane take the
      // push from 169 to 131 us at dim 64 and four from 318 to 233 us at dim 128; short rows (dim 20) are best at one.
      const int cpl = t.dim >= 128 ? 4 : (t.dim >= 32 ? 2 : 1);
      push_lanes = tn::lanes_for_width_host((t.dim + cpl - 1) / cpl);
    }
    if (!comm.contains("staged_return") || comm["staged_return"].cast<bool>()) {
      // rows per tile: whole 128-byte lines per tile, about 4 KiB of shared memory per warp at most
      int tr = 32;
      while (tr > 8 && tr * c.ustride * 4 > 4096) tr >>= 1;
      const int rpp = 32 / pull_lanes;
      const bool fits = (size_t)tr * c.ustride * 4 * 32 <= 160 * 1024;
      if (fits && tr % rpp == 0 && c.capo % tr == 0 && (tr * c.ustride * 4) % 128 == 0) tile_rows = tr;
    }
  }

  void set_opt(py::dict opt) { o = opt_from_dict(opt); }
  // The shard's arrays were replaced (growth, compaction): launches already recorded in CUDA graphs pick the new ones up.
  void set_table(py::dict table) { keep["table"] = table; t = table_from_dict(table); upload_table(); }

  // Dedup, id dispatch and inverse map of a batch ahead of its pull (plain kernels on the current stream).
  void front(at::Tensor ids, at::Tensor inverse) {
    TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "ids: contiguous int64 CUDA tensor");
    TORCH_CHECK(inverse.scalar_type() == at::kInt && inverse.numel() >= ids.numel(), "inverse: int32, one per id");
    c10::cuda::CUDAGuard guard(ids.device());
    tn::PullArgs a{};
    a.c = c; a.tbl = t; a.opt = o;
    a.ids = ptr_of<const long long>(ids);
    a.n_ids = (int)ids.numel();
    a.inverse = ptr_of<int>(inverse);
    a.training = 1;
    check(tn::launch_sparse_pull_front(a, cur_stream()), "sparse_pull_front launch");
    g_launches.fetch_add(1, std::memory_order_relaxed);      // two kernels
  }

  void pull(at::Tensor ids, at::Tensor inverse, c10::optional<at::Tensor> labels, int label_mod, bool training, bool lookup_only,
            bool front_done) {
    TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "ids: contiguous int64 CUDA tensor");
    TORCH_CHECK(inverse.scalar_type() == at::kInt && inverse.numel() >= ids.numel(), "inverse: int32, one per id");
    c10::cuda::CUDAGuard guard(ids.device());
    tn::PullArgs a{};
    a.c = c; a.tbl = t; a.opt = o;
    a.tbl_dev = reinterpret_cast<const tn::TableView*>(tbl_dev.data_ptr());
    a.ids = ptr_of<const long long>(ids);
    a.n_ids = (int)ids.numel();
    a.inverse = ptr_of<int>(inverse);
    a.labels = labels.has_value() ? ptr_of<const float>(*labels) : nullptr;
    a.label_mod = label_mod;
    a.training = training ? 1 : 0;
    a.lookup_only = lookup_only ? 1 : 0;
    TORCH_CHECK(!(training && lookup_only), "a training pull creates rows; lookup_only is for inference");
    a.front_done = front_done ? 1 : 0;
    a.lanes = pull_lanes;
    a.tile_rows = tile_rows;
    long long work = (long long)a.n_ids * (pull_lanes > 4 ? pull_lanes / 2 : 2);
    if (work > (1ll << 30)) work = 1ll << 30;
    check(tn::launch_sparse_pull(a, (int)work, cur_stream()), "sparse_pull_fused launch");
  }

  // `dense`: the dense step of the same training step (DenseCtx::rider_args), carried by a few CTAs of this launch.
  void push(int64_t work_hint, int max_ctas, const tn::DenseStepArgs* dense) {
    tn::PushArgs a{};
    a.c = c; a.tbl = t; a.opt = o; a.lanes = push_lanes;
    a.tbl_dev = reinterpret_cast<const tn::TableView*>(tbl_dev.data_ptr());
    long long work = work_hint * push_lanes;
    if (work > (1ll << 30)) work = 1ll << 30;
    check(tn::launch_sparse_push(a, (int)work, max_ctas, dense, cur_stream()), "sparse_push_fused launch");
  }
};

struct DenseCtx {
  tn::DenseStepArgs a{};
  py::dict keep;
  DenseCtx(py::dict d) {
    keep = d;
    a.opt.kind = d["kind"].cast<int>();
    a.opt.beta1 = d["beta1"].cast<float>();
    a.opt.beta2 = d["beta2"].cast<float>();
    a.opt.eps = d["eps"].cast<float>();
    a.opt.grad_decay = d["grad_decay"].cast<float>();
    a.opt.mom_decay = d["mom_decay"].cast<float>();
    a.opt.state = ptr_of<float>(d["state"].cast<at::Tensor>());
    a.n = d["n"].cast<long long>();
    a.chunk = d["chunk"].cast<long long>();
    a.world = d["world"].cast<int>();
    a.rank = d["rank"].cast<int>();
    a.grad_scale = d["grad_scale"].cast<float>();
    // small arrays: the owner re-zeroes every replica's gradient through the switch (no extra grid barrier);
    // large ones: each GPU clears its own replica after the closing barrier (no NVLink bytes)
    a.gated = d.contains("gated") ? d["gated"].cast<int>() : 0;
    a.zero_local = d.contains("zero_local") ? d["zero_local"].cast<int>() : (a.world > 1 && a.n > (1ll << 21) ? 1 : 0);
    auto W = d["W"].cast<std::vector<int64_t>>();
    auto G = d["G"].cast<std::vector<int64_t>>();
    auto Wb = d["Wb"].cast<std::vector<int64_t>>();
    auto sig = d["sig"].cast<std::vector<int64_t>>();
    TORCH_CHECK((int)W.size() == a.world && (int)G.size() == a.world && (int)Wb.size() == a.world, "peer tables");
    for (int p = 0; p < a.world; ++p) {
      a.W[p] = ptr_of<float>(W[p]); a.G[p] = ptr_of<float>(G[p]); a.Wb[p] = ptr_of<void>(Wb[p]);
      a.sig[p] = p < (int)sig.size() ? ptr_of<unsigned long long>(sig[p]) : nullptr;
    }
    a.W_mc = ptr_of<float>(d["W_mc"].cast<int64_t>());
    a.G_mc = ptr_of<float>(d["G_mc"].cast<int64_t>());
    a.Wb_mc = ptr_of<void>(d["Wb_mc"].cast<int64_t>());
    a.s0 = ptr_of<float>(d["s0"].cast<at::Tensor>());
    a.s1 = ptr_of<float>(d["s1"].cast<at::Tensor>());
    a.s2 = d.contains("s2") && !d["s2"].is_none() ? ptr_of<float>(d["s2"].cast<at::Tensor>()) : nullptr;
    a.epoch = ptr_of<unsigned long long>(d["epoch"].cast<at::Tensor>());
    a.bar = ptr_of<unsigned>(d["bar"].cast<at::Tensor>());
    a.status = ptr_of<int>(d["status"].cast<at::Tensor>());
    a.wait_ns = d["wait_ns"].cast<uint64_t>();
  }
  void step(bool skip_open) {
    tn::DenseStepArgs b = a;
    b.skip_open = skip_open ? 1 : 0;
    check(tn::launch_dense_step(b, cur_stream()), "dense step launch");
  }
  // Arguments for a launch in which the sparse push kernel carries this step: the opening "gradients ready"
  // barrier is always run (the carrying CTAs start together with the push, before any peer has been heard from).
  tn::DenseStepArgs rider_args() const {
    tn::DenseStepArgs b = a;
    b.skip_open = 0;
    return b;
  }
  void set_gated(bool g) { a.gated = g ? 1 : 0; }
  void set_max_ctas(int n) { a.max_ctas = n; }
};

// Device-resident batch-norm table and the per-step kernels of the layer.
struct BnCtx {
  tn::BnTableView t{};
  tn::BnSyncView s{};
  bool has_sync = false;
  double* batch = nullptr;     // [3][C] per-step scratch, kept zero between steps
  double* scratch = nullptr;   // [3][C] sum of the peers' increments during an exchange
  py::dict keep;
  BnCtx(py::dict d) {
    keep = d;
    t.C = d["C"].cast<int>();
    t.pctr = d["pctr"].cast<int>();
    t.moment = d["moment"].cast<double>();
    t.max_count = d["max_count"].cast<long long>();
    t.total_sum = ptr_of<double>(d["total_sum"].cast<at::Tensor>());
    t.total_sum_err = ptr_of<double>(d["total_sum_err"].cast<at::Tensor>());
    t.total_sq = ptr_of<double>(d["total_sq"].cast<at::Tensor>());
    t.total_sq_err = ptr_of<double>(d["total_sq_err"].cast<at::Tensor>());
    t.total_count = ptr_of<double>(d["total_count"].cast<at::Tensor>());
    t.inc = ptr_of<double>(d["inc"].cast<at::Tensor>());
    t.mean = ptr_of<float>(d["mean"].cast<at::Tensor>());
    t.var = ptr_of<float>(d["var"].cast<at::Tensor>());
    batch = ptr_of<double>(d["batch"].cast<at::Tensor>());
    scratch = ptr_of<double>(d["scratch"].cast<at::Tensor>());
    s.world = d["world"].cast<int>();
    s.rank = d["rank"].cast<int>();
    if (s.world > 1) {
      auto inc = d["inc_ptrs"].cast<std::vector<int64_t>>();
      auto sig = d["sig_ptrs"].cast<std::vector<int64_t>>();
      TORCH_CHECK((int)inc.size() == s.world && (int)sig.size() == s.world, "peer tables");
      for (int p = 0; p < s.world; ++p) { s.inc[p] = ptr_of<const double>(inc[p]); s.sig[p] = ptr_of<unsigned long long>(sig[p]); }
      s.epoch = ptr_of<unsigned long long>(d["epoch"].cast<at::Tensor>());
      s.status = ptr_of<int>(d["status"].cast<at::Tensor>());
      s.wait_ns = d["wait_ns"].cast<uint64_t>();
      has_sync = true;
    }
  }
  // sums of one batch -> totals, increments and moments (two launches)
  void push(at::Tensor x, bool centered) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.dim() == 2 && x.size(1) == t.C && x.stride(1) == 1, "x must be fp32 [B, C]");
    c10::cuda::CUDAGuard guard(x.device());
    tn::launch_bn_batch_stats(ptr_of<float>(x), (int)x.stride(0), (int)x.size(0), t.C, centered ? t.mean : nullptr, batch, cur_stream());
    tn::launch_bn_table_append(t, batch, cur_stream());
  }
  // fold a record the host has staged in `batch`
  void append_staged() { tn::launch_bn_table_append(t, batch, cur_stream()); }
  void refresh() { tn::launch_bn_table_refresh(t, cur_stream()); }
  void sync() {
    if (has_sync) tn::launch_bn_table_sync(t, s, scratch, cur_stream());
  }
  void apply_fwd(at::Tensor x, at::Tensor mean, at::Tensor var, c10::optional<at::Tensor> gamma, c10::optional<at::Tensor> beta, double eps,
                 at::Tensor y) {
    c10::cuda::CUDAGuard guard(x.device());
    tn::launch_bn_apply_fwd(ptr_of<float>(x), (int)x.stride(0), (int)x.size(0), t.C, ptr_of<float>(mean), ptr_of<float>(var), gamma ? ptr_of<float>(*gamma) : nullptr,
                            beta ? ptr_of<float>(*beta) : nullptr, (float)eps, ptr_of<float>(y), (int)y.stride(0), cur_stream());
  }
  void apply_bwd(at::Tensor dy, at::Tensor x, at::Tensor mean, at::Tensor var, c10::optional<at::Tensor> gamma, double eps,
                 c10::optional<at::Tensor> dx, c10::optional<at::Tensor> gg, c10::optional<at::Tensor> gb) {
    c10::cuda::CUDAGuard guard(x.device());
    tn::launch_bn_apply_bwd(ptr_of<float>(dy), (int)dy.stride(0), ptr_of<float>(x), (int)x.stride(0), (int)x.size(0), t.C,
                            ptr_of<float>(mean), ptr_of<float>(var),
                            gamma ? ptr_of<float>(*gamma) : nullptr, (float)eps, dx ? ptr_of<float>(*dx) : nullptr,
                            dx ? (int)dx->stride(0) : 0, gg ? ptr_of<float>(*gg) : nullptr, gb ? ptr_of<float>(*gb) : nullptr, cur_stream());
  }
};

// A metric-sum buffer is fp32[4] or fp32[4 + 2 * nbins]: the tail holds the two u32 prediction histograms of the AUC.
static int hist_bins(const at::Tensor& sums) {
  TORCH_CHECK(sums.scalar_type() == at::kFloat && sums.is_contiguous() && sums.numel() >= 4 && (sums.numel() - 4) % 2 == 0,
              "metric sums must be fp32[4] or fp32[4 + 2 * nbins]");
  return (int)((sums.numel() - 4) / 2);
}

void gemm(at::Tensor A, at::Tensor B, at::Tensor C, int M, int N, int K, int lda, int ldb, int ldc, bool a_mn, bool b_mn,
          bool accumulate, bool relu, c10::optional<at::Tensor> bias, c10::optional<at::Tensor> mask_aux,
          c10::optional<at::Tensor> had_x0, c10::optional<at::Tensor> had_xl, int ld_aux, int ones_col, int n_store,
          int split_k, int BN, at::Tensor status, c10::optional<at::Tensor> prof, c10::optional<at::Tensor> gate_flags,
          c10::optional<at::Tensor> gate_epoch, int gate_world, uint64_t gate_wait_ns, int m_halves, c10::optional<at::Tensor> aux_out) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && C.is_cuda(), "gemm: CUDA tensors");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16, "gemm: bf16 operands");
  c10::cuda::CUDAGuard guard(A.device());
  tn::GemmDesc d;
  d.M = M; d.N = N; d.K = K; d.A = A.data_ptr(); d.B = B.data_ptr(); d.lda = lda; d.ldb = ldb;
  d.a_mn = a_mn; d.b_mn = b_mn; d.C = C.data_ptr(); d.ldc = ldc;
  d.out_f32 = C.scalar_type() == at::kFloat;
  TORCH_CHECK(d.out_f32 || C.scalar_type() == at::kBFloat16, "gemm: C must be fp32 or bf16");
  d.accumulate = accumulate; d.relu = relu;
  d.bias = bias.has_value() ? ptr_of<const float>(*bias) : nullptr;
  d.mask_aux = mask_aux.has_value() ? mask_aux->data_ptr() : nullptr;
  d.had_x0 = had_x0.has_value() ? had_x0->data_ptr() : nullptr;
  d.had_xl = had_xl.has_value() ? had_xl->data_ptr() : nullptr;
  d.ld_aux = ld_aux; d.ones_col = ones_col; d.n_store = n_store; d.split_k = split_k; d.BN = BN;
  d.status = ptr_of<int>(status);
  d.prof = prof.has_value() ? ptr_of<unsigned long long>(*prof) : nullptr;
  d.m_halves = m_halves;
  if (aux_out.has_value()) {
    TORCH_CHECK(aux_out->scalar_type() == at::kBFloat16 && aux_out->stride(0) == ld_aux, "gemm: aux_out must be bf16 with row stride ld_aux");
    d.aux_out = aux_out->data_ptr();
  }
  if (gate_flags.has_value()) {
    TORCH_CHECK(gate_epoch.has_value() && gate_world >= 1 && gate_world <= tn::kMaxWorld, "gemm: gate wants flags, epoch and a world size");
    d.gate_flags = ptr_of<const unsigned long long>(*gate_flags);
    d.gate_epoch = ptr_of<const unsigned long long>(*gate_epoch);
    d.gate_world = gate_world;
    d.gate_wait_ns = gate_wait_ns;
  }
  const char* err = tn::gemm_bf16(d, cur_stream());
  if (err) throw std::runtime_error(err);
}

// One-kernel MLP chain.  weights[i]: bf16 [N_i, ld]; outs[i]: bf16 [M, ld_out_i] (forward: activations; backward: input
// gradients); masks[i] (backward): the activation whose ReLU the gradient passes through, or None.
tn::MlpChainDesc chain_desc(bool backward, const at::Tensor& x, int in_cols, const std::vector<at::Tensor>& weights,
                            const std::vector<int>& n_rows, const std::vector<int>& k_cols, const std::vector<at::Tensor>& outs,
                            const std::vector<int>& relu, const std::vector<int>& n_valid,
                            const std::vector<c10::optional<at::Tensor>>& masks, const at::Tensor& status) {
  const int L = (int)weights.size();
  TORCH_CHECK(L >= 1 && L <= tn::kMlpMaxLayers && (int)outs.size() == L && (int)n_rows.size() == L && (int)k_cols.size() == L,
              "mlp_chain: 1..4 layers with one output each");
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "mlp_chain: input must be a bf16 matrix");
  tn::MlpChainDesc d;
  d.L = L; d.M = (int)x.size(0); d.backward = backward ? 1 : 0;
  d.in = x.data_ptr(); d.in_cols = in_cols; d.ld_in = (int)x.stride(0);
  d.status = ptr_of<int>(status);
  for (int i = 0; i < L; ++i) {
    const at::Tensor& w = weights[i];
    const at::Tensor& o = outs[i];
    TORCH_CHECK(w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.stride(1) == 1, "mlp_chain: weights must be bf16 matrices");
    TORCH_CHECK(o.scalar_type() == at::kBFloat16 && o.dim() == 2 && o.stride(1) == 1 && o.size(0) == x.size(0), "mlp_chain: bad output");
    TORCH_CHECK(n_rows[i] <= w.size(0) && k_cols[i] <= w.stride(0), "mlp_chain: layer shape exceeds the weight matrix");
    tn::MlpChainLayer& l = d.layer[i];
    l.w = w.data_ptr(); l.n_rows = n_rows[i]; l.k_cols = k_cols[i]; l.ldw = (int)w.stride(0);
    l.out = o.data_ptr(); l.ld_out = (int)o.stride(0);
    l.relu = i < (int)relu.size() ? relu[i] : 0;
    l.n_valid = i < (int)n_valid.size() ? n_valid[i] : 0;
    if (i < (int)masks.size() && masks[i].has_value()) {
      const at::Tensor& mk = *masks[i];
      TORCH_CHECK(mk.scalar_type() == at::kBFloat16 && mk.dim() == 2 && mk.size(0) == x.size(0), "mlp_chain: bad mask");
      l.mask = mk.data_ptr(); l.ld_mask = (int)mk.stride(0);
    }
  }
  return d;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  py::class_<SparseCtx>(m, "SparseCtx")
      .def(py::init<py::dict, py::dict, py::dict>())
      .def("set_opt", &SparseCtx::set_opt)
      .def("set_table", &SparseCtx::set_table)
      .def("pull", &SparseCtx::pull, py::arg("ids"), py::arg("inverse"), py::arg("labels"), py::arg("label_mod"), py::arg("training"),
           py::arg("lookup_only") = false, py::arg("front_done") = false)
      .def("push", [](SparseCtx& self, int64_t work_hint, int max_ctas, py::object dense) {
        if (dense.is_none()) { self.push(work_hint, max_ctas, nullptr); return; }
        const tn::DenseStepArgs d = dense.cast<DenseCtx&>().rider_args();
        self.push(work_hint, max_ctas, &d);
      }, py::arg("work_hint"), py::arg("max_ctas") = 0, py::arg("dense") = py::none())
      .def("front", &SparseCtx::front, py::arg("ids"), py::arg("inverse"));
  py::class_<BnCtx>(m, "BnCtx")
      .def(py::init<py::dict>())
      .def("push", &BnCtx::push)
      .def("append_staged", &BnCtx::append_staged)
      .def("refresh", &BnCtx::refresh)
      .def("sync", &BnCtx::sync)
      .def("apply_fwd", &BnCtx::apply_fwd)
      .def("apply_bwd", &BnCtx::apply_bwd);
  py::class_<DenseCtx>(m, "DenseCtx").def(py::init<py::dict>()).def("step", &DenseCtx::step, py::arg("skip_open") = false).def("set_gated", &DenseCtx::set_gated).def("set_max_ctas", &DenseCtx::set_max_ctas);
  m.def("dense_ctas_per_sm", [] { return tn::dense_step_ctas_per_sm(); });
  m.def("mlp_chain", [](bool backward, at::Tensor x, int in_cols, std::vector<at::Tensor> weights, std::vector<int> n_rows,
                        std::vector<int> k_cols, std::vector<at::Tensor> outs, std::vector<int> relu, std::vector<int> n_valid,
                        std::vector<c10::optional<at::Tensor>> masks, at::Tensor status, c10::optional<at::Tensor> gate_flags,
                        c10::optional<at::Tensor> gate_epoch, int gate_world, uint64_t gate_wait_ns, bool probe_only,
                        c10::optional<at::Tensor> prof, int split) {
    c10::cuda::CUDAGuard guard(x.device());
    tn::MlpChainDesc d = chain_desc(backward, x, in_cols, weights, n_rows, k_cols, outs, relu, n_valid, masks, status);
    d.split = split;
    if (prof.has_value()) {
      TORCH_CHECK(prof->scalar_type() == at::kLong && prof->numel() >= 16, "mlp_chain: prof must be int64[16]");
      d.prof = ptr_of<unsigned long long>(*prof);
    }
    if (gate_flags.has_value()) {
      d.gate_flags = ptr_of<const unsigned long long>(*gate_flags);
      d.gate_epoch = ptr_of<const unsigned long long>(*gate_epoch);
      d.gate_world = gate_world;
      d.gate_wait_ns = gate_wait_ns;
    }
    if (probe_only) {
      const char* why = tn::mlp_chain_supported(d);
      return std::string(why ? why : "");
    }
    const char* err = tn::mlp_chain(d, cur_stream());
    if (err) throw std::runtime_error(err);
    return std::string();
  }, py::arg("backward"), py::arg("x"), py::arg("in_cols"), py::arg("weights"), py::arg("n_rows"), py::arg("k_cols"), py::arg("outs"),
     py::arg("relu"), py::arg("n_valid"), py::arg("masks"), py::arg("status"), py::arg("gate_flags") = py::none(),
     py::arg("gate_epoch") = py::none(), py::arg("gate_world") = 0, py::arg("gate_wait_ns") = 0, py::arg("probe_only") = false, py::arg("prof") = py::none(), py::arg("split") = 0,
     "a whole MLP tower (forward, or the input-gradient chain of the backward pass) in one kernel");
  m.def("gemm", &gemm, py::arg("A"), py::arg("B"), py::arg("C"), py::arg("M"), py::arg("N"), py::arg("K"), py::arg("lda"),
        py::arg("ldb"), py::arg("ldc"), py::arg("a_mn"), py::arg("b_mn"), py::arg("accumulate"), py::arg("relu"), py::arg("bias"),
        py::arg("mask_aux"), py::arg("had_x0"), py::arg("had_xl"), py::arg("ld_aux"), py::arg("ones_col"), py::arg("n_store"),
        py::arg("split_k"), py::arg("BN"), py::arg("status"), py::arg("prof") = py::none(),
        py::arg("gate_flags") = py::none(), py::arg("gate_epoch") = py::none(), py::arg("gate_world") = 0, py::arg("gate_wait_ns") = 0,
        py::arg("m_halves") = 0, py::arg("aux_out") = py::none());
  m.def("launch_count", []() { return g_launches.load(); });

  // ---- per-step host path of a replayed training step --------------------------------------------
  // One call instead of a dozen Python-level stream / event / copy calls: wait (on the copy stream) until the replay
  // that last read these input buffers is over, copy the step's inputs host -> device, record their arrival and make
  // the compute stream wait for it.  Streams and events come as the handles torch exposes (cuda_stream, cuda_event).
  m.def("stage_inputs", [](std::vector<at::Tensor> dsts, std::vector<at::Tensor> srcs, int64_t copy_stream, int64_t main_stream,
                           int64_t done_event, int64_t copied_event, int64_t read_event) {
    TORCH_CHECK(dsts.size() == srcs.size(), "stage_inputs: one source per destination");
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(copy_stream), ms = reinterpret_cast<cudaStream_t>(main_stream);
    if (done_event) check(cudaStreamWaitEvent(cs, reinterpret_cast<cudaEvent_t>(done_event), 0), "cudaStreamWaitEvent");
    // the loss of the step that last used this buffer set has been read back (it lives in the same captured memory)
    if (read_event) check(cudaStreamWaitEvent(cs, reinterpret_cast<cudaEvent_t>(read_event), 0), "cudaStreamWaitEvent");
    for (size_t i = 0; i < dsts.size(); ++i) {
      const at::Tensor& d = dsts[i];
      const at::Tensor& h = srcs[i];
      TORCH_CHECK(d.is_cuda() && !h.is_cuda() && d.is_contiguous() && h.is_contiguous() && d.nbytes() == h.nbytes() &&
                      d.scalar_type() == h.scalar_type(),
                  "stage_inputs: leaf ", i, " must be a contiguous host tensor of the static buffer's type and size");
      check(cudaMemcpyAsync(d.data_ptr(), h.data_ptr(), d.nbytes(), cudaMemcpyHostToDevice, cs), "cudaMemcpyAsync");
      // a page-locked source from torch's host allocator must not be handed out again before the copy has run
      // (what Tensor.copy_(non_blocking=True) does behind the scenes); a no-op for other host memory
      if (h.is_pinned())
        at::getHostAllocator(at::kCUDA)->record_event(const_cast<void*>(h.storage().data()), h.storage().data_ptr().get_context(),
                                                      c10::cuda::getStreamFromExternal(cs, d.device().index()).unwrap());
    }
    check(cudaEventRecord(reinterpret_cast<cudaEvent_t>(copied_event), cs), "cudaEventRecord");
    check(cudaStreamWaitEvent(ms, reinterpret_cast<cudaEvent_t>(copied_event), 0), "cudaStreamWaitEvent");
  });
  // 4-byte device scalar -> slot of a pinned ring, then an event behind it (the loss of a step on its way to the host)
  // `wait_event` != 0: the copy runs on a stream of its own behind that event (the end of the step), so the compute
  // stream carries nothing between two replayed steps.
  m.def("read_scalar_async", [](at::Tensor pinned, int64_t slot, at::Tensor src, int64_t stream, int64_t event, int64_t wait_event) {
    TORCH_CHECK(!pinned.is_cuda() && pinned.scalar_type() == at::kFloat && slot >= 0 && slot < pinned.numel(), "bad ring slot");
    TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kFloat && src.numel() == 1, "source: one float on the device");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (wait_event) check(cudaStreamWaitEvent(st, reinterpret_cast<cudaEvent_t>(wait_event), 0), "cudaStreamWaitEvent");
    check(cudaMemcpyAsync(pinned.data_ptr<float>() + slot, src.data_ptr(), sizeof(float), cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync");
    check(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), st), "cudaEventRecord");
  });

  // ---- CUDA IPC peer memory (fallback transport for the symmetric heap) --------------------------
  m.def("ipc_alloc", [](int64_t nbytes) {
    void* p = nullptr;
    check(cudaMalloc(&p, (size_t)nbytes), "cudaMalloc");
    check(cudaMemset(p, 0, (size_t)nbytes), "cudaMemset");
    cudaIpcMemHandle_t h;
    check(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle");
    return py::make_tuple((int64_t)reinterpret_cast<uintptr_t>(p), py::bytes(reinterpret_cast<const char*>(&h), sizeof(h)));
  });
  m.def("ipc_open", [](py::bytes handle) {
    std::string hs = handle;
    TORCH_CHECK(hs.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, hs.data(), sizeof(h));
    void* p = nullptr;
    check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    return (int64_t)reinterpret_cast<uintptr_t>(p);
  });
  m.def("ipc_close", [](int64_t p) { cudaIpcCloseMemHandle(ptr_of<void>(p)); });
  m.def("ipc_free", [](int64_t p) { cudaFree(ptr_of<void>(p)); });
  m.def("tensor_from_ptr", [](int64_t p, int64_t nbytes, int device) {
    auto opts = at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device);
    return at::from_blob(ptr_of<void>(p), {nbytes}, opts);
  });

  m.def("pool_fwd", [](at::Tensor U, int ustride, at::Tensor inverse, c10::optional<at::Tensor> offsets, int B, int S, int pd,
                       int combiner, at::Tensor out, int out_ld) {
    c10::cuda::CUDAGuard guard(U.device());
    tn::launch_pool_fwd(ptr_of<float>(U), ustride, ptr_of<int>(inverse), offsets ? ptr_of<int>(*offsets) : nullptr, B, S, pd,
                        combiner, ptr_of<float>(out), out_ld, cur_stream());
  });
  m.def("pool_bwd", [](at::Tensor gU, int gstride, at::Tensor inverse, c10::optional<at::Tensor> offsets, int B, int S, int pd,
                       int dim, int combiner, at::Tensor gout, int gout_ld) {
    c10::cuda::CUDAGuard guard(gU.device());
    tn::launch_pool_bwd(ptr_of<float>(gU), gstride, ptr_of<int>(inverse), offsets ? ptr_of<int>(*offsets) : nullptr, B, S, pd,
                        dim, combiner, ptr_of<float>(gout), gout_ld, cur_stream());
  });
  m.def("seq_fwd", [](at::Tensor U, int ustride, at::Tensor inverse, at::Tensor offsets, int B, int T, int pd, at::Tensor out,
                      at::Tensor lengths) {
    c10::cuda::CUDAGuard guard(U.device());
    tn::launch_seq_fwd(ptr_of<float>(U), ustride, ptr_of<int>(inverse), ptr_of<int>(offsets), B, T, pd, ptr_of<float>(out),
                       ptr_of<int>(lengths), cur_stream());
  });
  m.def("seq_bwd", [](at::Tensor gU, int gstride, at::Tensor inverse, at::Tensor offsets, int B, int T, int pd, int dim,
                      at::Tensor gout) {
    c10::cuda::CUDAGuard guard(gU.device());
    tn::launch_seq_bwd(ptr_of<float>(gU), gstride, ptr_of<int>(inverse), ptr_of<int>(offsets), B, T, pd, dim,
                       ptr_of<float>(gout), cur_stream());
  });
  m.def("table_insert_keys", [](py::dict table, at::Tensor keys, at::Tensor out_rows, at::Tensor status) {
    c10::cuda::CUDAGuard guard(keys.device());
    tn::launch_table_insert_keys(table_from_dict(table), ptr_of<long long>(keys), (int)keys.numel(), ptr_of<int>(out_rows),
                                 ptr_of<int>(status), cur_stream());
  });
  m.def("table_lookup", [](py::dict table, at::Tensor keys, at::Tensor out_rows) {
    c10::cuda::CUDAGuard guard(keys.device());
    tn::launch_table_lookup(table_from_dict(table), ptr_of<long long>(keys), (int)keys.numel(), ptr_of<int>(out_rows), cur_stream());
  });
  m.def("table_rebuild_index", [](py::dict table, int n, at::Tensor status) {
    tn::TableView t = table_from_dict(table);
    TORCH_CHECK(n >= 0 && n <= t.row_cap, "table_rebuild_index: more rows than the slab holds");
    c10::cuda::CUDAGuard guard(status.device());
    tn::launch_table_rebuild_index(t, n, ptr_of<int>(status), cur_stream());
  }, "fill an all-empty key array from the signs of rows [0, n)");
  m.def("table_keep_mask", [](py::dict table, int kind, bool evict, float show_threshold, int no_show_days, int logic, int n,
                              at::Tensor keep) {
    TORCH_CHECK(keep.scalar_type() == at::kByte && keep.numel() >= n, "table_keep_mask: keep must be uint8[n]");
    tn::ExportRule rule{evict ? 1 : 0, show_threshold, no_show_days, logic};
    c10::cuda::CUDAGuard guard(keep.device());
    tn::launch_table_keep_mask(table_from_dict(table), kind, rule, n, keep.data_ptr<unsigned char>(), cur_stream());
  }, "keep[r] = 0 for the rows the save-time eviction rule drops");
  m.def("table_decay", [](py::dict table, int kind, float rate, int delta_days) {
    tn::launch_table_decay(table_from_dict(table), kind, rate, delta_days, cur_stream());
  });
  m.def("table_export", [](py::dict table, int kind, bool evict, float show_threshold, int no_show_days, int logic, int r0, int r1,
                           at::Tensor counts, at::Tensor cursors, at::Tensor out_keys, at::Tensor out_rows) {
    TORCH_CHECK(counts.numel() >= 8 && cursors.numel() >= 8 && out_rows.dim() == 2 && out_rows.is_contiguous(), "table_export buffers");
    TORCH_CHECK(out_keys.numel() >= r1 - r0 && out_rows.size(0) >= r1 - r0, "table_export: staging buffers smaller than the row range");
    tn::ExportRule rule{evict ? 1 : 0, show_threshold, no_show_days, logic};
    c10::cuda::CUDAGuard guard(out_rows.device());
    tn::launch_table_export(table_from_dict(table), kind, rule, r0, r1, ptr_of<int>(counts), ptr_of<int>(cursors),
                            ptr_of<unsigned long long>(out_keys), ptr_of<float>(out_rows), (int)out_rows.size(1), cur_stream());
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }, "filter rows [r0, r1) by the save-time eviction rule and pack them grouped by block file");
  m.def("fm_fwd", [](at::Tensor E, int ld, int B, int F, int D, at::Tensor out) {
    c10::cuda::CUDAGuard guard(E.device());
    tn::launch_fm_fwd(ptr_of<float>(E), ld, B, F, D, ptr_of<float>(out), cur_stream());
  });
  m.def("fm_bwd", [](at::Tensor E, int ld, int B, int F, int D, at::Tensor gout, at::Tensor gE, int gld, bool accumulate) {
    c10::cuda::CUDAGuard guard(E.device());
    tn::launch_fm_bwd(ptr_of<float>(E), ld, B, F, D, ptr_of<float>(gout), ptr_of<float>(gE), gld, accumulate, cur_stream());
  });
  auto concat_like = [](bool split) {
    return [split](std::vector<c10::optional<at::Tensor>> pieces, std::vector<int> widths, std::vector<int> lds, at::Tensor out,
                   int B, int ld_out, int ones_col) {
      TORCH_CHECK(pieces.size() <= (size_t)tn::kMaxPieces && pieces.size() == widths.size() && lds.size() == widths.size(),
                  "concat: at most 6 pieces");
      c10::cuda::CUDAGuard guard(out.device());
      tn::ConcatArgs a{};
      a.B = B; a.n_pieces = (int)pieces.size(); a.out = out.data_ptr(); a.ld_out = ld_out; a.ones_col = ones_col;
      for (size_t p = 0; p < pieces.size(); ++p) {
        a.width[p] = widths[p]; a.ld[p] = lds[p];
        if (pieces[p].has_value()) {
          a.ptr[p] = pieces[p]->data_ptr();
          a.is_bf16[p] = pieces[p]->scalar_type() == at::kBFloat16;
          TORCH_CHECK(a.is_bf16[p] || pieces[p]->scalar_type() == at::kFloat, "concat: fp32 or bf16 pieces");
        } else {
          a.ptr[p] = nullptr; a.is_bf16[p] = 0;
        }
      }
      if (split) tn::launch_split_cast(a, cur_stream()); else tn::launch_concat_cast(a, cur_stream());
    };
  };
  m.def("concat_cast", concat_like(false));
  m.def("split_cast", concat_like(true));
  m.def("gemv_fwd", [](at::Tensor Z, int ld, int B, int K, at::Tensor w, at::Tensor y) {
    c10::cuda::CUDAGuard guard(Z.device());
    tn::launch_gemv_fwd(Z.data_ptr(), ld, B, K, ptr_of<float>(w), ptr_of<float>(y), cur_stream());
  });
  m.def("gemv_bwd", [](at::Tensor Z, int ld, int B, int K, at::Tensor w, at::Tensor dy, at::Tensor dZ, at::Tensor gw, int relu_cols) {
    c10::cuda::CUDAGuard guard(Z.device());
    tn::launch_gemv_bwd(Z.data_ptr(), ld, B, K, ptr_of<float>(w), ptr_of<float>(dy), dZ.data_ptr(), ptr_of<float>(gw), relu_cols,
                        cur_stream());
  });
  m.def("bce", [](at::Tensor logit, at::Tensor label, c10::optional<at::Tensor> pred, c10::optional<at::Tensor> dlogit,
                  float grad_scale, at::Tensor sums) {
    c10::cuda::CUDAGuard guard(logit.device());
    tn::launch_bce(ptr_of<float>(logit), ptr_of<float>(label), (int)logit.numel(), pred ? ptr_of<float>(*pred) : nullptr,
                   dlogit ? ptr_of<float>(*dlogit) : nullptr, grad_scale, ptr_of<float>(sums), hist_bins(sums), cur_stream());
  });
  m.def("deepfm_input_fwd", [](at::Tensor U, int ustride, at::Tensor inverse, int B, int S, int D, c10::optional<at::Tensor> dense,
                               at::Tensor X0, at::Tensor fm, int lin_col, c10::optional<at::Tensor> Lout) {
    c10::cuda::CUDAGuard guard(U.device());
    const int Dd = dense ? (int)dense->size(1) : 0;
    const char* err = tn::launch_deepfm_input_fwd(ptr_of<float>(U), ustride, ptr_of<int>(inverse), B, S, D,
                                                  dense ? ptr_of<float>(*dense) : nullptr, Dd, dense ? (int)dense->stride(0) : 0,
                                                  X0.data_ptr(), (int)X0.stride(0), ptr_of<float>(fm), Lout ? lin_col : -1,
                                                  Lout ? ptr_of<float>(*Lout) : nullptr, cur_stream());
    if (err) throw std::runtime_error(err);
  });
  m.def("deepfm_input_bwd", [](at::Tensor U, int ustride, at::Tensor inverse, int B, int S, int D, at::Tensor dX0, at::Tensor gfm,
                               at::Tensor gU, int gstride, int lin_col, c10::optional<at::Tensor> dL) {
    c10::cuda::CUDAGuard guard(U.device());
    const char* err = tn::launch_deepfm_input_bwd(ptr_of<float>(U), ustride, ptr_of<int>(inverse), B, S, D, dX0.data_ptr(),
                                                  (int)dX0.stride(0), ptr_of<float>(gfm), ptr_of<float>(gU), gstride, dL ? lin_col : -1,
                                                  dL ? ptr_of<float>(*dL) : nullptr, cur_stream());
    if (err) throw std::runtime_error(err);
  });
  m.def("deepfm_head_loss", [](at::Tensor H, int NH, c10::optional<at::Tensor> L, at::Tensor fm, at::Tensor w, at::Tensor label,
                               at::Tensor dH, c10::optional<at::Tensor> dL, at::Tensor dfm, at::Tensor gw, at::Tensor sums,
                               c10::optional<at::Tensor> pred, at::Tensor loss_out, at::Tensor scratch) {
    c10::cuda::CUDAGuard guard(H.device());
    TORCH_CHECK(scratch.numel() >= 4 + 16 * 576 && scratch.scalar_type() == at::kFloat && (reinterpret_cast<uintptr_t>(scratch.data_ptr()) & 15) == 0,
                "deepfm_head_loss: scratch must be fp32[4 + 16 * 576], 16-byte aligned, zero between calls");
    const int NL = L ? (int)L->size(1) : 0;
    TORCH_CHECK(w.numel() == NH + NL + 2, "deepfm_head_loss: weight must be [NH + NL + 2]");
    const char* err = tn::launch_deepfm_head_loss(H.data_ptr(), (int)H.stride(0), NH, L ? ptr_of<float>(*L) : nullptr, NL,
                                                  ptr_of<float>(fm), ptr_of<float>(w), ptr_of<float>(label), (int)H.size(0),
                                                  dH.data_ptr(), dL ? ptr_of<float>(*dL) : nullptr, ptr_of<float>(dfm),
                                                  ptr_of<float>(gw), ptr_of<float>(sums), hist_bins(sums),
                                                  pred ? ptr_of<float>(*pred) : nullptr,
                                                  ptr_of<float>(loss_out), ptr_of<float>(scratch), cur_stream());
    if (err) throw std::runtime_error(err);
  });
  m.def("unique_assign", [](at::Tensor ids, c10::optional<at::Tensor> labels, at::Tensor dd_keys, at::Tensor dd_vals, at::Tensor uniq,
                            at::Tensor inverse, c10::optional<at::Tensor> show, c10::optional<at::Tensor> click, at::Tensor count,
                            at::Tensor status) {
    c10::cuda::CUDAGuard guard(ids.device());
    const int64_t cap2 = dd_keys.numel();
    TORCH_CHECK(cap2 >= 2 && (cap2 & (cap2 - 1)) == 0 && dd_vals.numel() >= cap2, "unique_assign: scratch must be a power of two");
    TORCH_CHECK(ids.scalar_type() == at::kLong && ids.is_contiguous() && inverse.numel() >= ids.numel(), "unique_assign: bad ids / inverse");
    g_launches.fetch_add(2, std::memory_order_relaxed);
    tn::launch_unique_assign(ptr_of<long long>(ids), (int)ids.numel(), labels ? ptr_of<float>(*labels) : nullptr,
                             ptr_of<unsigned long long>(dd_keys), ptr_of<int>(dd_vals), (unsigned)cap2,
                             ptr_of<unsigned long long>(uniq), (int)uniq.numel(), ptr_of<int>(inverse),
                             show ? ptr_of<float>(*show) : nullptr, click ? ptr_of<float>(*click) : nullptr, ptr_of<int>(count),
                             ptr_of<int>(status), cur_stream());
  });
  m.def("dict_lookup_pool", [](py::dict table, at::Tensor ids, c10::optional<at::Tensor> offsets, int B, int S, int combiner,
                               at::Tensor out, int ld_out, int ones_col) {
    c10::cuda::CUDAGuard guard(ids.device());
    tn::TableView t = table_from_dict(table);
    TORCH_CHECK(t.dim % 4 == 0, "dict_lookup_pool: dim must be a multiple of 4");
    tn::launch_dict_lookup_pool(t, ptr_of<long long>(ids), offsets ? ptr_of<int>(*offsets) : nullptr, B, S, combiner, out.data_ptr(),
                                ld_out, ones_col, cur_stream());
  });
  m.def("sigmoid", [](at::Tensor x, at::Tensor y) {
    c10::cuda::CUDAGuard guard(x.device());
    tn::launch_sigmoid(ptr_of<float>(x), ptr_of<float>(y), (int)x.numel(), cur_stream());
  });
  m.def("cross_v2_bwd_elem", [](at::Tensor g, at::Tensor u, at::Tensor x0, at::Tensor gx0, at::Tensor du, bool first) {
    TORCH_CHECK(g.is_contiguous() && u.is_contiguous() && x0.is_contiguous() && gx0.is_contiguous() && du.is_contiguous(), "contiguous operands");
    TORCH_CHECK(g.numel() % 8 == 0 && u.numel() == g.numel() && x0.numel() == g.numel() && gx0.numel() == g.numel() && du.numel() == g.numel(), "sizes");
    TORCH_CHECK(g.scalar_type() == at::kBFloat16 && gx0.scalar_type() == at::kFloat, "g / u / x0 / du are bf16, gx0 is fp32");
    c10::cuda::CUDAGuard guard(g.device());
    tn::launch_cross_v2_bwd_elem(g.data_ptr(), u.data_ptr(), x0.data_ptr(), ptr_of<float>(gx0), du.data_ptr(), g.numel(), first ? 1 : 0, cur_stream());
  });
  m.def("cross_v2_bwd_final", [](at::Tensor gx0, at::Tensor g, at::Tensor out) {
    TORCH_CHECK(gx0.is_contiguous() && g.is_contiguous() && out.is_contiguous() && g.numel() % 8 == 0 && gx0.numel() == g.numel() && out.numel() == g.numel(), "operands");
    c10::cuda::CUDAGuard guard(g.device());
    tn::launch_cross_v2_bwd_final(ptr_of<float>(gx0), g.data_ptr(), out.data_ptr(), g.numel(), cur_stream());
  });
  m.def("relu_mask", [](at::Tensor g, at::Tensor y) {
    c10::cuda::CUDAGuard guard(g.device());
    TORCH_CHECK(g.numel() % 8 == 0 && g.numel() == y.numel(), "relu_mask: numel must be a multiple of 8");
    tn::launch_relu_mask(g.data_ptr(), y.data_ptr(), g.numel(), cur_stream());
  });
  m.def("cross_v1_fwd", [](at::Tensor x0, at::Tensor xl, at::Tensor w, at::Tensor bias, at::Tensor y, at::Tensor dot) {
    c10::cuda::CUDAGuard guard(x0.device());
    tn::launch_cross_v1_fwd(ptr_of<float>(x0), ptr_of<float>(xl), ptr_of<float>(w), ptr_of<float>(bias), (int)x0.size(0),
                            (int)x0.size(1), ptr_of<float>(y), ptr_of<float>(dot), cur_stream());
  });
  m.def("cross_v1_bwd", [](at::Tensor x0, at::Tensor xl, at::Tensor w, at::Tensor dot, at::Tensor gy, at::Tensor gx0,
                           at::Tensor gxl, at::Tensor gw, at::Tensor gb) {
    c10::cuda::CUDAGuard guard(x0.device());
    tn::launch_cross_v1_bwd(ptr_of<float>(x0), ptr_of<float>(xl), ptr_of<float>(w), ptr_of<float>(dot), ptr_of<float>(gy),
                            (int)x0.size(0), (int)x0.size(1), ptr_of<float>(gx0), ptr_of<float>(gxl), ptr_of<float>(gw),
                            ptr_of<float>(gb), cur_stream());
  });
}
