// Global batch-norm statistics on the GPU.
//
// The reference keeps, per feature and in double precision, the running sum, squared sum and
// count with Kahan-compensated adds and a moving-window decay once `max_count` records have been
// seen (core/ps/table/bn_table.cc:65-121); the layer pushes one batch's sums per step and
// normalises with the table's moments (tensornet/layers/normalization_layer.py:129-177), and the
// ranks exchange their increments by RPC (core/kernels/bn_table_ops.cc:86-159,233-299).
//
// Here the table lives in device memory and a training step of the layer is three small kernels
// with no host round trip, so it can sit inside a captured CUDA graph:
//   bn_batch_stats   per-feature sum and squared sum (optionally around a centre) in fp64
//   bn_table_append  fold the batch into the totals, refresh the fp32 moments, re-zero the scratch
//   bn_apply_fwd/bwd normalise with the moments (moments are constants for the backward pass)
// and, when the layer is synchronised, every `sync_freq` steps
//   bn_table_sync    cross-GPU exchange of the pending increments by peer loads, bracketed by
//                    bounded flag handshakes.
#include "tn_device.cuh"
#include "tn_ops.h"

namespace tn {

namespace {

constexpr int kBnCols = 32;    // columns per CTA
constexpr int kBnRows = 8;     // row lanes per CTA (256 threads)

__global__ void __launch_bounds__(kBnCols * kBnRows) bn_batch_stats_kernel(const float* __restrict__ x, int ld, int B, int C,
                                                                          const float* __restrict__ center, double* batch,
                                                                          int rows_per_cta) {
  __shared__ double s_sum[kBnRows][kBnCols], s_sq[kBnRows][kBnCols];
  const int cl = threadIdx.x % kBnCols, rl = threadIdx.x / kBnCols;
  const int c = blockIdx.x * kBnCols + cl;
  const int r0 = blockIdx.y * rows_per_cta;
  const int r1 = min(B, r0 + rows_per_cta);
  double s = 0.0, q = 0.0;
  if (c < C) {
    const float ctr = center ? center[c] : 0.f;
    for (int r = r0 + rl; r < r1; r += kBnRows) {
      const double v = (double)x[(size_t)r * ld + c];
      const double d = v - (double)ctr;
      s += v;
      q += d * d;
    }
  }
  s_sum[rl][cl] = s;
  s_sq[rl][cl] = q;
  __syncthreads();
  if (rl == 0 && c < C) {
#pragma unroll
    for (int k = 1; k < kBnRows; ++k) { s += s_sum[k][cl]; q += s_sq[k][cl]; }
    atomicAdd(&batch[c], s);
    atomicAdd(&batch[C + c], q);
    if (blockIdx.y == 0) batch[2 * C + c] = (double)B;     // every feature saw B records
  }
}

__device__ __forceinline__ double block_max(double v) {
  __shared__ double s_w[32];
  __shared__ double s_out;
  for (int off = 16; off > 0; off >>= 1) v = fmax(v, __shfl_xor_sync(0xffffffffu, v, off));
  if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    double w = threadIdx.x < (blockDim.x + 31) / 32 ? s_w[threadIdx.x] : -1.0;
    for (int off = 16; off > 0; off >>= 1) w = fmax(w, __shfl_xor_sync(0xffffffffu, w, off));
    if (threadIdx.x == 0) s_out = w;
  }
  __syncthreads();
  const double r = s_out;
  __syncthreads();
  return r;
}

// One Kahan-compensated table update of feature c with (as, aq, ac); `decay_k` < 0 selects the plain path.
__device__ __forceinline__ void bn_fold(const BnTableView& t, int c, double as, double aq, double ac, double decay_k) {
  double ts = t.total_sum[c], te = t.total_sum_err[c], tq = t.total_sq[c], tqe = t.total_sq_err[c];
  if (decay_k >= 0.0) {
    ts *= (1.0 - decay_k); as *= decay_k;
    tq *= (1.0 - decay_k); aq *= decay_k;
  } else {
    t.total_count[c] += ac;
  }
  double y = as - te, u = ts + y;
  te = (u - ts) - y; ts = u;
  y = aq - tqe; u = tq + y;
  tqe = (u - tq) - y; tq = u;
  t.total_sum[c] = ts; t.total_sum_err[c] = te; t.total_sq[c] = tq; t.total_sq_err[c] = tqe;
}

__device__ __forceinline__ void bn_moments(const BnTableView& t, int c) {
  const double n = t.total_count[c];
  const bool ok = n != 0.0 && n == n;
  const double mean = ok ? t.total_sum[c] / n : 0.0;
  t.mean[c] = (float)mean;
  if (t.pctr) {
    t.var[c] = (float)t.total_sq[c];
  } else {
    const float m = (float)mean, sm = ok ? (float)(t.total_sq[c] / n) : 0.f;
    t.var[c] = ok ? fmaxf(sm - m * m, 0.f) : 1.f;     // no record yet: identity scale, the layer's initial moving variance
  }
}

// `acc` = [3][C] sums to fold in.  Decides between plain accumulation and the moving window exactly as the
// host table does: window mode once max(total_count) exceeds max_count, with ratio = max(acc_count) / max(total_count).
__device__ void bn_append_block(const BnTableView& t, const double* acc, bool is_local, bool zero_acc) {
  const int C = t.C;
  double cur = 0.0, am = 0.0;
  for (int c = threadIdx.x; c < C; c += blockDim.x) { cur = fmax(cur, t.total_count[c]); am = fmax(am, acc[2 * C + c]); }
  cur = floor(block_max(cur));
  am = floor(block_max(am));
  const bool window = t.max_count > 0 && cur > (double)t.max_count;
  const double k = window ? (1.0 - t.moment) * (am / cur) : -1.0;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const double as = acc[c], aq = acc[C + c], ac = acc[2 * C + c];
    if (is_local) { t.inc[c] += as; t.inc[C + c] += aq; t.inc[2 * C + c] += ac; }
    bn_fold(t, c, as, aq, ac, k);
    bn_moments(t, c);
    if (zero_acc) { const_cast<double*>(acc)[c] = 0.0; const_cast<double*>(acc)[C + c] = 0.0; const_cast<double*>(acc)[2 * C + c] = 0.0; }
  }
}

__global__ void __launch_bounds__(1024) bn_table_append_kernel(const BnTableView t, double* batch) {
  bn_append_block(t, batch, true, true);
}

__global__ void __launch_bounds__(1024) bn_table_refresh_moments_kernel(const BnTableView t) {
  for (int c = threadIdx.x; c < t.C; c += blockDim.x) bn_moments(t, c);
}

// Cross-GPU exchange.  One CTA per GPU: (1) tell every peer "my increments are final" and wait for theirs,
// (2) sum the peers' increments with peer loads into `scratch` and fold them in as one non-local append,
// (3) tell every peer "I have read yours" and wait for the same, (4) clear the own increments.
__global__ void __launch_bounds__(1024) bn_table_sync_kernel(const BnTableView t, const BnSyncView s, double* scratch) {
  __shared__ int s_fail;
  const int C = t.C, W = s.world, R = s.rank;
  const unsigned long long epoch = __ldcg(s.epoch) + 1ull;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < W && threadIdx.x != R) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys_u64(s.sig[p] + R, epoch << 32);
    unsigned long long v;
    if (!wait_flag_ge(s.sig[R] + p, epoch, &v, s.wait_ns, s.status, 61, p)) s_fail = 1;
  }
  __syncthreads();
  if (s_fail) return;
  for (int i = threadIdx.x; i < 3 * C; i += blockDim.x) {
    double a = 0.0;
    for (int k = 1; k < W; ++k) {
      const double* pi = s.inc[(R + k) % W];
      a += __ldcg(&pi[i]);
    }
    scratch[i] = a;
  }
  __syncthreads();
  bn_append_block(t, scratch, false, true);
  __syncthreads();
  if (threadIdx.x < W && threadIdx.x != R) {
    const int p = threadIdx.x;
    st_release_sys_u64(s.sig[p] + kMaxWorld + R, epoch << 32);
    unsigned long long v;
    if (!wait_flag_ge(s.sig[R] + kMaxWorld + p, epoch, &v, s.wait_ns, s.status, 62, p)) s_fail = 1;
  }
  __syncthreads();
  if (s_fail) return;
  for (int i = threadIdx.x; i < 3 * C; i += blockDim.x) t.inc[i] = 0.0;
  if (threadIdx.x == 0) *s.epoch = epoch;
}

__global__ void bn_apply_fwd_kernel(const float* __restrict__ x, int ldx, int B, int C, const float* __restrict__ mean,
                                    const float* __restrict__ var, const float* __restrict__ gamma, const float* __restrict__ beta,
                                    float eps, float* __restrict__ y, int ldy) {
  const long long n = (long long)B * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / C), c = (int)(i - (long long)r * C);
    float v = (x[(size_t)r * ldx + c] - mean[c]) * rsqrtf(var[c] + eps);
    if (gamma) v *= gamma[c];
    if (beta) v += beta[c];
    y[(size_t)r * ldy + c] = v;
  }
}

// dx = dy * gamma * rsqrt(var + eps); dgamma = sum dy * xhat; dbeta = sum dy (accumulated into gg / gb).
__global__ void __launch_bounds__(kBnCols * kBnRows) bn_apply_bwd_kernel(const float* __restrict__ dy, int ldd, const float* __restrict__ x,
                                                                        int ldx, int B, int C, const float* __restrict__ mean,
                                                                        const float* __restrict__ var, const float* __restrict__ gamma,
                                                                        float eps, float* __restrict__ dx, int ldo, float* gg, float* gb,
                                                                        int rows_per_cta) {
  __shared__ float s_g[kBnRows][kBnCols], s_b[kBnRows][kBnCols];
  const int cl = threadIdx.x % kBnCols, rl = threadIdx.x / kBnCols;
  const int c = blockIdx.x * kBnCols + cl;
  const int r0 = blockIdx.y * rows_per_cta, r1 = min(B, r0 + rows_per_cta);
  float ag = 0.f, ab = 0.f;
  if (c < C) {
    const float rs = rsqrtf(var[c] + eps), m = mean[c], gm = gamma ? gamma[c] : 1.f;
    for (int r = r0 + rl; r < r1; r += kBnRows) {
      const float d = dy[(size_t)r * ldd + c];
      ag += d * (x[(size_t)r * ldx + c] - m) * rs;
      ab += d;
      if (dx) dx[(size_t)r * ldo + c] = d * gm * rs;
    }
  }
  s_g[rl][cl] = ag;
  s_b[rl][cl] = ab;
  __syncthreads();
  if (rl == 0 && c < C) {
#pragma unroll
    for (int k = 1; k < kBnRows; ++k) { ag += s_g[k][cl]; ab += s_b[k][cl]; }
    if (gg) atomicAdd(&gg[c], ag);
    if (gb) atomicAdd(&gb[c], ab);
  }
}

inline int rows_per_cta_for(int B, int C) {
  const int col_tiles = (C + kBnCols - 1) / kBnCols;
  int want_y = (148 * 4 + col_tiles - 1) / col_tiles;       // enough CTAs to fill the GPU
  if (want_y < 1) want_y = 1;
  int rows = (B + want_y - 1) / want_y;
  if (rows < 64) rows = 64;
  return rows;
}

}  // namespace

void launch_bn_batch_stats(const float* x, int ld, int B, int C, const float* center, double* batch, cudaStream_t st) {
  const int rows = rows_per_cta_for(B, C);
  dim3 grid((C + kBnCols - 1) / kBnCols, (B + rows - 1) / rows);
  bn_batch_stats_kernel<<<grid, kBnCols * kBnRows, 0, st>>>(x, ld, B, C, center, batch, rows);
}
void launch_bn_table_append(const BnTableView& t, double* batch, cudaStream_t st) { bn_table_append_kernel<<<1, 1024, 0, st>>>(t, batch); }
void launch_bn_table_refresh(const BnTableView& t, cudaStream_t st) { bn_table_refresh_moments_kernel<<<1, 1024, 0, st>>>(t); }
void launch_bn_table_sync(const BnTableView& t, const BnSyncView& s, double* scratch, cudaStream_t st) {
  bn_table_sync_kernel<<<1, 1024, 0, st>>>(t, s, scratch);
}
void launch_bn_apply_fwd(const float* x, int ldx, int B, int C, const float* mean, const float* var, const float* gamma,
                         const float* beta, float eps, float* y, int ldy, cudaStream_t st) {
  long long n = (long long)B * C;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  bn_apply_fwd_kernel<<<blocks, 256, 0, st>>>(x, ldx, B, C, mean, var, gamma, beta, eps, y, ldy);
}
void launch_bn_apply_bwd(const float* dy, int ldd, const float* x, int ldx, int B, int C, const float* mean, const float* var,
                         const float* gamma, float eps, float* dx, int ldo, float* gg, float* gb, cudaStream_t st) {
  const int rows = rows_per_cta_for(B, C);
  dim3 grid((C + kBnCols - 1) / kBnCols, (B + rows - 1) / rows);
  bn_apply_bwd_kernel<<<grid, kBnCols * kBnRows, 0, st>>>(dy, ldd, x, ldx, B, C, mean, var, gamma, eps, dx, ldo, gg, gb, rows);
}

}  // namespace tn
