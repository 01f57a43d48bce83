// A whole MLP tower in ONE kernel per direction.
//
// The reference builds its towers from Keras Dense layers (examples/models/deepfm.py:43-44,
// examples/models/wide_deep.py).  Run layer by layer, each of the 8192 x 400 x 430 GEMMs of the
// DeepFM tower leaves the tensor cores idle most of the time: a launch, a pipeline ramp and an
// epilogue per layer, and the activations go out to L2 and come back.  Here a CTA owns a stripe
// of 128 examples and walks through all layers of the chain:
//
//   * the stripe's activations stay in shared memory, in the 128-byte-swizzled K-major layout that
//     tcgen05.mma reads its A operand from; the epilogue of one layer writes the A operand of the
//     next one there directly (bias via the constant-one column, ReLU or ReLU-mask applied);
//   * the weights of all layers stream through a ring of TMA tiles (each CTA fetches its own);
//   * the accumulator of a layer (up to 448 columns) lives in tensor memory;
//   * each layer's output also leaves by TMA store, because the backward pass needs it;
//   * with `split == 2` a stripe belongs to a PAIR of CTAs (a thread-block cluster of two): each computes about half of
//     a layer's output columns, so it streams half of the weights and all 148 SMs work on a batch of 8192; the
//     epilogue writes every 16-byte piece into both CTAs' activation buffers (distributed shared memory), and the
//     two hand over through mbarriers in each other's shared memory.  Every CTA fetches its own weight tiles.
//
// Forward chain:   H_l = relu(H_{l-1} . W_l^T)            W_l bf16 [N_l, ld] K-major, bias in column K_l
// Backward chain:  dH_{l-1} = (dH_l . W_l) * [H_{l-1} > 0]    same W_l read as an MN-major operand
//
// Every wait is bounded; when one runs out the CTA records an error, drains its copies, frees its
// tensor memory and returns.
#include <cstdio>
#include <cstdlib>
#include "mlp_fused.h"
#include "tc_primitives.cuh"

namespace tn {

using namespace tc;

namespace {

constexpr int kRows = 128;                 // examples per CTA (UMMA M)
constexpr int kKB = 64;                    // contraction elements per k-block: one 128-byte swizzle row of bf16
constexpr int kTileBytes = kRows * kKB * 2;   // one k-block of the A operand: 16 KiB
constexpr int kEpiWarps = 16;
constexpr int kThreads = 32 * (2 + kEpiWarps);   // warp 0 TMA, warp 1 MMA + TMEM owner, 16 epilogue warps
constexpr int kMaxStages = 4;

__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory"); }

struct ChainMaps {
  CUtensorMap in;                       // chain input [M, cols]
  CUtensorMap w[kMlpMaxLayers][2];      // weights of step i, as seen by CTA 0 / CTA 1 of a pair (box heights differ)
  CUtensorMap out[kMlpMaxLayers];       // output of step i [M, cols]
};

__global__ void __launch_bounds__(kThreads, 1) mlp_chain_kernel(const __grid_constant__ ChainMaps maps, const MlpChainParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kMaxStages];
  __shared__ __align__(8) uint64_t s_in;        // chain input has landed in the A buffer
  __shared__ __align__(8) uint64_t s_a;         // the epilogue(s) have written the next A operand (one arrival per CTA of the pair)
  __shared__ __align__(8) uint64_t s_acc;       // all MMAs of a step have completed
  __shared__ __align__(8) uint64_t s_peer;      // the other CTA of the pair has finished the MMAs of a step
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort_i;
  __shared__ int s_epi_ok;
  volatile int* s_abort = &s_abort_i;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_smem = base;                                     // kt_max tiles of 16 KiB
  const uint32_t b_smem = base + (uint32_t)p.kt_max * kTileBytes;   // p.stages stages of p.stage_bytes
  const int split = p.split;                                         // CTAs per stripe: 1, or 2 (a cluster of two)
  const int rank = split == 2 ? (int)cluster_ctarank() : 0;
  const int m0 = (int)(blockIdx.x / split) * kRows;
  const int kStages = p.stages;
  unsigned long long* prof = (p.prof && blockIdx.x == 0) ? p.prof : nullptr;
  if (prof && threadIdx.x == 0) prof[0] = globaltimer_ns();

  if (threadIdx.x == 0) {
    *s_abort = 0;
    for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&s_full[s]), 1); mbar_init(smem_u32(&s_empty[s]), 1); }
    mbar_init(smem_u32(&s_in), 1);
    mbar_init(smem_u32(&s_a), (uint32_t)split);
    mbar_init(smem_u32(&s_acc), 1);
    mbar_init(smem_u32(&s_peer), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.in)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&maps.w[0][rank])) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (split == 2) {     // the other CTA's barriers must be initialised before anything arrives on them
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  // everything above touches no tensor data and may overlap the tail of the previous kernel in the stream
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (prof && threadIdx.x == 0) prof[1] = globaltimer_ns();

  if (warp == 0) {
    // ------------------------------- TMA producer ---------------------------------------
    if (lane == 0) {
      bool ok = true;
      if (p.gate_flags != nullptr) {
        // every owner's chunk of the dense weight array has landed in this GPU's replica
        const unsigned long long want = __ldcg(p.gate_epoch);
        for (int q = 0; q < p.gate_world && ok; ++q) {
          const unsigned long long t0 = globaltimer_ns();
          unsigned spins = 0;
          while ((ld_acquire_sys_u64(p.gate_flags + q) >> 32) < want) {
            if (((++spins) & 63u) == 0 && globaltimer_ns() - t0 > p.gate_wait_ns) { ok = false; break; }
            __nanosleep(64);
          }
          if (!ok) set_status(p.status, kPeerWaitTimeout, 70, q);
        }
        asm volatile("fence.proxy.async;" ::: "memory");
        if (!ok) *s_abort = 1;
      }
      if (ok) {
        // the stripe of the chain input: kt_in tiles straight into the A buffer
        const uint32_t bin = smem_u32(&s_in);
        mbar_expect_tx(bin, (uint32_t)p.kt_in * kTileBytes);
        for (int j = 0; j < p.kt_in; ++j) tma_load_2d(a_smem + j * kTileBytes, &maps.in, j * kKB, m0, bin);
      }
      int it = 0;
      for (int i = 0; i < p.L && ok; ++i) {
        const int kt = p.kt[i];
        for (int k = 0; k < kt && ok; ++k, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (uint32_t)(it / kStages) & 1u;
          if (!mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, s_abort)) { *s_abort = 1; ok = false; break; }
          const uint32_t full = smem_u32(&s_full[s]);
          const uint32_t dst = b_smem + s * p.stage_bytes;
          const int n_lo = p.n_lo[i][rank], n_cnt = p.n_cnt[i][rank];      // this CTA's accumulator columns
          if (!p.backward) {
            // K-major weights: rows n of W_l, 64 contraction columns; box_rows rows per copy
            const int br = p.box_rows[i][rank];
            const int nbox = n_cnt / br;
            mbar_expect_tx(full, (uint32_t)n_cnt * kKB * 2);
            for (int b = 0; b < nbox; ++b) tma_load_2d(dst + b * br * kKB * 2, &maps.w[i][rank], k * kKB, n_lo + b * br, full);
          } else {
            // MN-major weights: 64 contraction rows n of W_l, output columns in chunks of 64
            const int nch = n_cnt / 64;
            mbar_expect_tx(full, (uint32_t)nch * 8192u);
            for (int c = 0; c < nch; ++c) tma_load_2d(dst + c * 8192, &maps.w[i][rank], n_lo + 64 * c, k * kKB, full);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -----------------------------------------
    if (lane == 0) {
      bool ok = true;
      int it = 0;
      for (int i = 0; i < p.L && ok; ++i) {
        // A operand of this step: the chain input (TMA) or what the epilogue of the previous step wrote
        if (i == 0) ok = mbar_wait(smem_u32(&s_in), 0u, s_abort);
        else ok = mbar_wait_cluster(smem_u32(&s_a), (uint32_t)(i - 1) & 1u, s_abort);
        if (!ok) { *s_abort = 1; break; }
        // the A operand was written through the generic proxy (by this CTA's epilogue and, in a pair, by the other
        // CTA's): order those writes before the tensor core's reads
        asm volatile("fence.proxy.async;" ::: "memory");
        tc_fence_after();
        if (prof) prof[2 + 3 * i] = globaltimer_ns();
        const int n_acc = p.n_cnt[i][rank];
        const int n0 = n_acc > 256 ? 256 : n_acc, n1 = n_acc - n0;
        const uint32_t bmn = p.backward ? 1u : 0u;
        const uint32_t idesc0 = (1u << 4) | (1u << 7) | (1u << 10) | (bmn << 16) | ((uint32_t)(n0 >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
        const uint32_t idesc1 = (1u << 4) | (1u << 7) | (1u << 10) | (bmn << 16) | ((uint32_t)(n1 >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
        const uint32_t b_lbo = p.backward ? 8192u : 16u, b_kstep = p.backward ? 2048u : 32u;
        // second accumulator half: rows 256.. of a K-major stage (128 B each) or chunks 4.. of an MN-major one (8 KiB each)
        const uint32_t b_half = p.backward ? 4u * 8192u : 256u * 128u;
        const int kt = p.kt[i];
        for (int k = 0; k < kt && ok; ++k, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (uint32_t)(it / kStages) & 1u;
          if (!mbar_wait(smem_u32(&s_full[s]), ph, s_abort)) { *s_abort = 1; ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = a_smem + k * kTileBytes;
          const uint32_t b_base = b_smem + s * p.stage_bytes;
#pragma unroll
          for (int kk = 0; kk < kKB / 16; ++kk) {
            const uint64_t ad = make_smem_desc(a_base + kk * 32, 16u, 1024u);
            const uint32_t acc = (k > 0 || kk > 0) ? 1u : 0u;
            umma_f16(tmem, ad, make_smem_desc(b_base + kk * b_kstep, b_lbo, 1024u), idesc0, acc);
            if (n1 > 0) umma_f16(tmem + 256u, ad, make_smem_desc(b_base + b_half + kk * b_kstep, b_lbo, 1024u), idesc1, acc);
          }
          umma_commit(smem_u32(&s_empty[s]));   // frees the stage once the MMAs have read it
        }
        if (ok) umma_commit(smem_u32(&s_acc));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue (warps 2..17) ------------------------------
    // A warp may read the TMEM lane quarter (warp % 4); four warps share a quarter and take 32-column chunks in turn.
    const int ew = warp - 2;
    const int q = warp & 3;
    const int sub = ew >> 2;
    const int r = q * 32 + lane;                      // row of the stripe this thread owns
    const int grow = m0 + r;
    const uint32_t tm_lane = tmem + ((uint32_t)(q * 32) << 16);
    const bool leader = (ew == 0 && lane == 0);
    const int rsw = r & 7;
    const uint32_t peer = (uint32_t)(rank ^ 1);
    for (int i = 0; i < p.L; ++i) {
      // one thread waits for the accumulator and for the stores that still read the A buffer (and, in a pair, for the
      // other CTA to be done with its MMAs, which read the buffer this epilogue is about to write into); everybody else
      // learns the outcome behind a barrier, so the sixteen warps always agree on whether to go on
      if (leader) {
        int ok = mbar_wait(smem_u32(&s_acc), (uint32_t)i & 1u, s_abort) ? 1 : 0;
        tma_store_wait_read();
        if (split == 2) {
          mbar_arrive_remote(map_to_cta(smem_u32(&s_peer), peer));
          if (ok && !mbar_wait_cluster(smem_u32(&s_peer), (uint32_t)i & 1u, s_abort)) ok = 0;
        }
        if (!ok) *s_abort = 1;
        s_epi_ok = ok;
        if (prof) prof[3 + 3 * i] = globaltimer_ns();
      }
      epi_barrier();
      if (!s_epi_ok) break;
      tc_fence_after();
      const int n_valid = p.n_valid[i], out_cols = p.out_cols[i], ones_col = p.ones_col[i];
      const int n_lo = p.n_lo[i][rank], n_cnt = p.n_cnt[i][rank];
      // columns this CTA produces: its accumulator columns, and for the last CTA of a stripe also the constant tail
      const int c_lo = n_lo, c_hi = (rank == split - 1) ? out_cols : n_lo + n_cnt;
      const __nv_bfloat16* mask = p.mask[i];
      const int ld_mask = p.ld_mask[i];
      const bool relu = p.relu[i] != 0;
      for (int c0 = c_lo + 32 * sub; c0 < c_hi; c0 += 32 * (kEpiWarps / 4)) {
        uint32_t acc[32];
        if (c0 < n_lo + n_cnt) {
          tmem_ld32_nowait(tm_lane + (uint32_t)(c0 - n_lo), acc);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = 0u;
        }
        uint4 mv[4];
        if (mask != nullptr) {
#pragma unroll
          for (int pc = 0; pc < 4; ++pc) {
            const int col = c0 + pc * 8;
            mv[pc] = make_uint4(0u, 0u, 0u, 0u);
            if (grow < p.M && col + 8 <= ld_mask) mv[pc] = __ldg(reinterpret_cast<const uint4*>(mask + (size_t)grow * ld_mask + col));
          }
        }
        const bool plain = c0 + 32 <= n_valid && c0 + 32 <= n_lo + n_cnt;      // warp-uniform: no constant columns in this chunk
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {
          const int colp = c0 + pc * 8;
          if (colp >= c_hi) break;                    // a CTA's range need not end on a chunk boundary
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float x = __uint_as_float(acc[pc * 8 + j]);
            if (relu) x = fmaxf(x, 0.f);
            if (!plain) {
              const int col = colp + j;
              if (col >= n_valid || col >= n_lo + n_cnt) x = (col == ones_col) ? 1.f : 0.f;
            }
            v[j] = x;
          }
          if (mask != nullptr) {      // backward of ReLU: keep the gradient where the forward activation was positive
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&mv[pc]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float2 m2 = __bfloat1622float2(h2[k]);
              if (!(m2.x > 0.f)) v[2 * k] = 0.f;
              if (!(m2.y > 0.f)) v[2 * k + 1] = 0.f;
            }
          }
          const uint4 o = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
          const uint32_t dst = a_smem + (uint32_t)(colp >> 6) * kTileBytes + (uint32_t)r * 128u + (uint32_t)(((((colp & 63) >> 3)) ^ rsw) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w) : "memory");
          if (split == 2)     // the same piece into the other CTA's activation buffer
            asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(map_to_cta(dst, peer)), "r"(o.x), "r"(o.y), "r"(o.z),
                         "r"(o.w)
                         : "memory");
        }
      }
      // the A operand of the next step (and the source of this step's stores) is complete once everybody - in a pair:
      // of both CTAs - is here
      tc_fence_before();
      asm volatile("fence.proxy.async;" ::: "memory");
      epi_barrier();
      if (leader) {
        if (prof) prof[4 + 3 * i] = globaltimer_ns();
        bool ok = true;
        if (split == 2) {
          mbar_arrive_local_cluster(smem_u32(&s_a));
          mbar_arrive_remote(map_to_cta(smem_u32(&s_a), peer));
          // the tiles this CTA stores hold columns the other one wrote: wait for its arrival too
          ok = mbar_wait_cluster(smem_u32(&s_a), (uint32_t)i & 1u, s_abort);
          asm volatile("fence.proxy.async;" ::: "memory");
          if (!ok) *s_abort = 1;
        } else if (i + 1 < p.L) {
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&s_a)) : "memory");
        }
        if (ok) {
          const int nt = out_cols >> 6;
          const int t_lo = split == 2 ? (rank == 0 ? 0 : (nt + 1) / 2) : 0;
          const int t_hi = split == 2 ? (rank == 0 ? (nt + 1) / 2 : nt) : nt;
          for (int j = t_lo; j < t_hi; ++j) tma_store_2d(&maps.out[i], j * kKB, m0, a_smem + j * kTileBytes);
          tma_store_commit();
        }
      }
    }
    if (leader) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (*s_abort) {
    // a wait ran out: report, give copies in flight time to land, then release TMEM
    if (threadIdx.x == 0) set_status(p.status, kMbarTimeout, 31, (int)blockIdx.x);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  if (split == 2) {     // neither CTA of a pair may leave while the other can still write into its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
}

int largest_box(int n) {   // largest divisor of n that is a multiple of 8 and at most 256
  for (int d = 256; d >= 8; d -= 8)
    if (n % d == 0) return d;
  return 0;
}

}  // namespace

// Column split of one step between the CTAs of a stripe.  Forward widths split on multiples of 16 (a tensor-core N),
// backward widths on multiples of 64 (one MN-major chunk).
static void split_columns(int n_acc, int split, bool backward, int lo[2], int cnt[2]) {
  if (split == 1) { lo[0] = 0; cnt[0] = n_acc; lo[1] = n_acc; cnt[1] = 0; return; }
  const int g = backward ? 64 : 16;
  int half = ((n_acc + 1) / 2 + g - 1) / g * g;
  if (half > 256) half = 256;
  lo[0] = 0; cnt[0] = half; lo[1] = half; cnt[1] = n_acc - half;
}

struct ChainPlan {
  MlpChainParams p;
  size_t smem;
  const char* error;
};

static ChainPlan plan_chain(const MlpChainDesc& d, int split) {
  ChainPlan pl{};
  MlpChainParams& p = pl.p;
  pl.error = nullptr;
  if (d.L < 1 || d.L > kMlpMaxLayers) { pl.error = "mlp_chain: 1..4 layers"; return pl; }
  if (d.M <= 0) { pl.error = "mlp_chain: empty batch"; return pl; }
  p.L = d.L; p.M = d.M; p.backward = d.backward; p.split = split;
  p.kt_in = (d.in_cols + kKB - 1) / kKB;
  int kt_max = p.kt_in, stage = 0, kt_prev = p.kt_in;
  for (int i = 0; i < d.L; ++i) {
    const MlpChainLayer& l = d.layer[i];
    if (l.n_rows <= 0 || l.k_cols <= 0) { pl.error = "mlp_chain: empty layer"; return pl; }
    if (l.ldw % 8 || l.ld_out % 8) { pl.error = "mlp_chain: leading dimensions must be multiples of 8 elements"; return pl; }
    if (!d.backward) {
      p.n_acc[i] = l.n_rows;                                  // accumulator columns = output features
      if (p.n_acc[i] % 16 || p.n_acc[i] > 448) { pl.error = "mlp_chain: layer width must be a multiple of 16, at most 448"; return pl; }
      p.n_valid[i] = l.n_rows;
      p.ones_col[i] = l.n_rows;
      p.out_cols[i] = (l.n_rows + 1 + kKB - 1) / kKB * kKB;   // features, the constant-one column, zero padding
      p.kt[i] = (l.k_cols + kKB - 1) / kKB;
      p.relu[i] = l.relu;
      p.mask[i] = nullptr; p.ld_mask[i] = 0;
    } else {
      p.n_acc[i] = (l.k_cols + 63) / 64 * 64;                 // accumulator columns = input features of the layer
      if (p.n_acc[i] > 448) { pl.error = "mlp_chain: layer input wider than 448 columns"; return pl; }
      p.n_valid[i] = l.n_valid;
      p.ones_col[i] = -1;
      p.out_cols[i] = p.n_acc[i];
      p.kt[i] = (l.n_rows + kKB - 1) / kKB;
      p.relu[i] = 0;
      p.mask[i] = reinterpret_cast<const __nv_bfloat16*>(l.mask); p.ld_mask[i] = l.ld_mask;
      if (l.mask && ((reinterpret_cast<uintptr_t>(l.mask) & 15) || l.ld_mask % 8)) { pl.error = "mlp_chain: mask must be 16-byte aligned"; return pl; }
    }
    split_columns(p.n_acc[i], split, d.backward != 0, p.n_lo[i], p.n_cnt[i]);
    for (int r = 0; r < split; ++r) {
      const int c = p.n_cnt[i][r];
      if (c < 16 || c > (split == 2 ? 256 : 448) || (split == 1 && c > 256 && c - 256 < 16)) { pl.error = "mlp_chain: a CTA's share of a layer must be 16..256 columns"; return pl; }
      p.box_rows[i][r] = d.backward ? kKB : largest_box(c);
      if (p.box_rows[i][r] == 0) { pl.error = "mlp_chain: layer width has no TMA box"; return pl; }
      stage = stage > c * kKB * 2 ? stage : c * kKB * 2;
    }
    if (p.kt[i] > kt_prev) { pl.error = "mlp_chain: a layer contracts over more columns than the previous one produced"; return pl; }
    if (p.out_cols[i] > l.ld_out + 63) { pl.error = "mlp_chain: output buffer narrower than the layer"; return pl; }
    kt_prev = p.out_cols[i] / kKB;
    kt_max = kt_max > kt_prev ? kt_max : kt_prev;
  }
  p.kt_max = kt_max;
  p.stage_bytes = (uint32_t)((stage + 1023) / 1024 * 1024);
  const size_t budget = 227 * 1024 - 512;
  const size_t a_bytes = (size_t)kt_max * kTileBytes + 1024;
  if (a_bytes + 2 * (size_t)p.stage_bytes > budget) { pl.error = "mlp_chain: tower does not fit in shared memory"; return pl; }
  int stages = (int)((budget - a_bytes) / p.stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p.stages = stages;
  pl.smem = a_bytes + (size_t)stages * p.stage_bytes;
  return pl;
}

static int choose_split(const MlpChainDesc& d) {
  if (d.split == 1 || d.split == 2) return d.split;
  static const int env = []() { const char* e = getenv("TN_MLP_SPLIT"); return e ? atoi(e) : 0; }();
  if (env == 1 || env == 2) return env;
  // a pair per stripe as soon as single CTAs would leave more than half of the GPU idle
  const int stripes = (d.M + kRows - 1) / kRows;
  return (stripes <= 148 / 2 + 32 && plan_chain(d, 2).error == nullptr) ? 2 : 1;
}

const char* mlp_chain_supported(const MlpChainDesc& d) {
  return plan_chain(d, choose_split(d)).error;
}

const char* mlp_chain(const MlpChainDesc& d, cudaStream_t stream) {
  const int split = choose_split(d);
  ChainPlan pl = plan_chain(d, split);
  if (pl.error) return pl.error;
  MlpChainParams& p = pl.p;
  ChainMaps maps;
  p.status = d.status;
  p.prof = d.prof;
  p.gate_flags = d.gate_flags; p.gate_epoch = d.gate_epoch; p.gate_world = d.gate_world; p.gate_wait_ns = d.gate_wait_ns;
  if (reinterpret_cast<uintptr_t>(d.in) & 15) return "mlp_chain: input must be 16-byte aligned";
  if (!get_tensor_map(d.in, d.M, d.in_cols, d.ld_in, kRows, &maps.in)) return "mlp_chain: cuTensorMapEncodeTiled failed (input)";
  for (int i = 0; i < d.L; ++i) {
    const MlpChainLayer& l = d.layer[i];
    if ((reinterpret_cast<uintptr_t>(l.w) | reinterpret_cast<uintptr_t>(l.out)) & 15) return "mlp_chain: operands must be 16-byte aligned";
    for (int r = 0; r < 2; ++r) {
      const int br = r < split ? p.box_rows[i][r] : p.box_rows[i][0];
      if (!get_tensor_map(l.w, l.n_rows, l.k_cols, l.ldw, br, &maps.w[i][r])) return "mlp_chain: cuTensorMapEncodeTiled failed (weights)";
    }
    if (!get_tensor_map(l.out, d.M, l.ld_out, l.ld_out, kRows, &maps.out[i])) return "mlp_chain: cuTensorMapEncodeTiled failed (output)";
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(mlp_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 256);
    if (e != cudaSuccess) return cudaGetErrorString(e);
    attr_set = true;
  }
  static const bool use_pdl = []() { const char* e = getenv("TN_PDL"); return e == nullptr || atoi(e) != 0; }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(split * ((d.M + kRows - 1) / kRows)));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (use_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (split == 2) {       // the two CTAs of a stripe form a cluster (distributed shared memory)
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 2;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, mlp_chain_kernel, maps, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace tn
