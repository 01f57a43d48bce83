// bf16 GEMM family for the dense towers (MLP forward, dgrad, wgrad and the DCN-v2 cross
// layers) written directly against the Blackwell tensor-core path:
//   * operand tiles are fetched by TMA (cp.async.bulk.tensor, no multicast) into a
//     128B-swizzled shared-memory ring guarded by mbarriers,
//   * one elected thread issues tcgen05.mma (kind::f16, bf16 in / fp32 accumulate) with
//     the accumulator tile living in tensor memory (TMEM),
//   * four epilogue warps read the accumulator back with tcgen05.ld and apply the fused
//     epilogue (bias, ReLU, ReLU-mask of the backward pass, "ones" bias column,
//     Hadamard-residual of DCN-v2, fp32 accumulate with split-K reduction).
// The reference runs these layers as Keras Dense / tf.matmul on CPU
// (examples/models/deepfm.py:43-44, examples/common/layers.py:53-59).
//
// C[M,N] = sum_k A(m,k) * B(n,k).  Each operand may be stored contraction-major
// ("K-major": [rows, k] row-major) or output-major ("MN-major": [k, rows] row-major), which
// covers forward (K,K), dgrad (K,MN) and wgrad (MN,MN) without any transposed copies.
//
// Every mbarrier wait is bounded; on expiry the CTA records an error, lets its TMA copies
// land, frees its TMEM columns and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include "gemm_tcgen05.h"
#include "tc_primitives.cuh"
#include "gemm_epilogue.cuh"

namespace tn {

using namespace tc;

namespace {

constexpr int kBM = 128;        // tile rows (UMMA M)
constexpr int kBK = 64;         // contraction elements per stage = one 128-byte swizzle row of bf16
constexpr int kUmmaK = 16;
constexpr int kABytes = kBM * kBK * 2;   // 16 KiB
constexpr int kEpiSubs = 4;               // epilogue warps per TMEM lane quarter
constexpr int kEpiWarps = 4 * kEpiSubs;
constexpr int kGemmThreads = 32 * (2 + kEpiWarps);   // warp0 TMA, warp1 MMA + TMEM owner, the rest epilogue
constexpr int kEpiBytesPerWarp = gemm_epi::kBytesPerWarp;

template <int kStages, int kHalves>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kStages];
  __shared__ __align__(8) uint64_t s_empty[kStages];
  __shared__ __align__(8) uint64_t s_accum;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort_i;
  volatile int* s_abort = &s_abort_i;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BN = p.BN;
  const uint32_t b_bytes = (uint32_t)BN * kBK * 2;
  // A CTA owns one or two 128-row accumulators that share every B tile: with two, the operand bytes per FLOP drop
  // by a third (the 128 x 256 tile is bound by the ~120 GB/s at which one SM can ingest operands).
  constexpr int halves = kHalves;
  const uint32_t a_stage = (uint32_t)halves * kABytes;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_smem = base;
  const uint32_t b_smem = base + kStages * a_stage;

  // Tile order.  Large grids walk the tiles in groups of kRasterGroup rows of tiles, column by column inside a
  // group, so that the CTAs resident at one time share a compact block of A and B tiles in L2 instead of a thin
  // stripe that streams all of B for every few rows of A.
  int tile_n = blockIdx.x, tile_m = blockIdx.y;
  if (p.raster_group > 1) {
    const int gx = gridDim.x, gy = gridDim.y;
    const int pid = blockIdx.y * gx + blockIdx.x;
    const int width = p.raster_group * gx;
    const int first_m = (pid / width) * p.raster_group;
    const int gsize = min(gy - first_m, p.raster_group);
    tile_m = first_m + (pid % width) % gsize;
    tile_n = (pid % width) / gsize;
  }
  const int n0 = tile_n * BN;
  const int m0 = tile_m * kBM * halves;
  const int kt_total = (p.K + kBK - 1) / kBK;
  const int kt0 = blockIdx.z * p.k_tiles_per_split;
  int nk = kt_total - kt0;
  if (nk > p.k_tiles_per_split) nk = p.k_tiles_per_split;

  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < BN) tmem_cols <<= 1;
  if (halves == 2) tmem_cols = 512;          // second accumulator at column 256
  unsigned long long* prof = (p.prof && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.prof : nullptr;
  if (prof && threadIdx.x == 0) prof[0] = globaltimer_ns();

  if (threadIdx.x == 0) {
    *s_abort = 0;
    for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&s_full[s]), 1); mbar_init(smem_u32(&s_empty[s]), 1); }
    mbar_init(smem_u32(&s_accum), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmA)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmB)) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  // Programmatic dependent launch: everything above (barrier init, TMEM allocation, descriptor prefetch) touches
  // no tensor data and may overlap the tail of the kernel launched before this one; from here on the previous
  // kernel's results are needed.  The kernel launched after this one may start its own set-up right away.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (prof && threadIdx.x == 0) prof[1] = globaltimer_ns();

  if (warp == 0) {
    // ------------------------------- TMA producer ---------------------------------------
    if (lane == 0) {
      bool gate_ok = true;
      if (p.gate_flags != nullptr) {
        // every owner's chunk of the weight array has landed in this GPU's replica
        const unsigned long long want = __ldcg(p.gate_epoch);
        for (int q = 0; q < p.gate_world && gate_ok; ++q) {
          const unsigned long long t0 = globaltimer_ns();
          unsigned spins = 0;
          while ((ld_acquire_sys_u64(p.gate_flags + q) >> 32) < want) {
            if (((++spins) & 63u) == 0 && globaltimer_ns() - t0 > p.gate_wait_ns) { gate_ok = false; break; }
            __nanosleep(64);
          }
          if (!gate_ok) set_status(p.status, kPeerWaitTimeout, 70, q);
        }
        asm volatile("fence.proxy.async;" ::: "memory");
        if (!gate_ok) *s_abort = 1;
      }
      for (int i = 0; i < nk && gate_ok; ++i) {
        const int s = i % kStages;
        const uint32_t ph = (uint32_t)(i / kStages) & 1u;
        if (!mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, s_abort)) { *s_abort = 1; break; }
        const uint32_t full = smem_u32(&s_full[s]);
        mbar_expect_tx(full, a_stage + b_bytes);
        const int kc = (kt0 + i) * kBK;
        const uint32_t b_dst = b_smem + s * b_bytes;
#pragma unroll
        for (int h = 0; h < halves; ++h) {
          const uint32_t a_dst = a_smem + s * a_stage + h * kABytes;
          const int mh = m0 + h * kBM;
          if (!p.a_mn) {
            tma_load_2d(a_dst, &tmA, kc, mh, full);
          } else {
            tma_load_2d(a_dst, &tmA, mh, kc, full);
            tma_load_2d(a_dst + 8192, &tmA, mh + 64, kc, full);
          }
        }
        if (!p.b_mn) {
          tma_load_2d(b_dst, &tmB, kc, n0, full);
        } else {
          for (int c = 0; c < BN / 64; ++c) tma_load_2d(b_dst + c * 8192, &tmB, n0 + 64 * c, kc, full);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -----------------------------------------
    if (lane == 0) {
      // instruction descriptor: D=f32, A=B=bf16, majors, N>>3, M>>4
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.a_mn ? 1 : 0) << 15) |
                             ((uint32_t)(p.b_mn ? 1 : 0) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u, b_kstep = p.b_mn ? 2048u : 32u;
      bool ok = true;
      for (int i = 0; i < nk && ok; ++i) {
        const int s = i % kStages;
        const uint32_t ph = (uint32_t)(i / kStages) & 1u;
        if (!mbar_wait(smem_u32(&s_full[s]), ph, s_abort)) { *s_abort = 1; ok = false; break; }
        tc_fence_after();
        if (prof && i < 8) prof[2 + i] = globaltimer_ns();
        const uint32_t a_base = a_smem + s * a_stage;
        const uint32_t b_base = b_smem + s * b_bytes;
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          const uint64_t bd = make_smem_desc(b_base + k * b_kstep, b_lbo, 1024u);
#pragma unroll
          for (int h = 0; h < halves; ++h) {
            const uint64_t ad = make_smem_desc(a_base + h * kABytes + k * a_kstep, a_lbo, 1024u);
            umma_f16(tmem + (uint32_t)(h * 256), ad, bd, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(smem_u32(&s_empty[s]));   // frees the stage once the MMAs have read it
      }
      if (ok) umma_commit(smem_u32(&s_accum));
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue (warps 2..) --------------------------------
    // kEpiSubs warps share each TMEM lane quarter and take column chunks round-robin.
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int sub = (warp - 2) >> 2;        // which of the interleaved chunk sequences
    bool ok = nk > 0;
    if (ok && !mbar_wait(smem_u32(&s_accum), 0u, s_abort)) { *s_abort = 1; ok = false; }
    tc_fence_after();
    if (prof && warp == 2 && lane == 0) prof[10] = globaltimer_ns();
    if (ok) {
      // The accumulator barrier has fired: every TMA load has landed and every MMA has read its
      // operands, so the stage ring is free.  Each epilogue warp takes 6 KiB of it as a transpose
      // buffer: TMEM gives a lane one ROW of the tile, global memory wants a warp on whole lines.
      // Blocks of 32 rows x 64 bytes go through shared memory (16-byte pieces, XOR-swizzled so both
      // the row-wise writes and the line-wise reads are bank-conflict free) and leave as 64-byte
      // row segments, eight rows per store instruction.
      uint8_t* smem_gen = smem_raw + (base - smem_u32(smem_raw));
      uint8_t* sm_out = smem_gen + (warp - 2) * kEpiBytesPerWarp;
#pragma unroll 1
      for (int half = 0; half < halves; ++half) {
        const int row_base = m0 + half * kBM + q * 32;
        const uint32_t tm_lane = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * 256);
        gemm_epi::store_rows(p, tm_lane, row_base, n0, BN, sub, kEpiSubs, lane, sm_out);
      }
    }
  }

  if (prof && warp == 2 && lane == 0) prof[11] = globaltimer_ns();
  tc_fence_before();
  __syncthreads();
  if (prof && threadIdx.x == 0) prof[12] = globaltimer_ns();
  if (*s_abort) {
    // a wait ran out: report, give copies in flight time to land, then release TMEM
    if (threadIdx.x == 0) set_status(p.status, kMbarTimeout, 30, (int)blockIdx.x);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------
// host side: tensor-map cache + launch
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

struct MapKey {
  const void* ptr; long long rows, cols, ld; int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = mix64((uint64_t)k.ptr);
    h = mix64(h ^ (uint64_t)k.rows * 0x9E3779B97F4A7C15ull);
    h = mix64(h ^ (uint64_t)k.cols * 0xC2B2AE3D27D4EB4Full);
    h = mix64(h ^ (uint64_t)k.ld ^ ((uint64_t)k.box_rows << 48));
    return (size_t)h;
  }
};

}  // namespace

// 2-D bf16 row-major tensor [rows, cols] with leading dimension `ld` elements; box = 64 x box_rows.
bool get_tensor_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}

// gemm_2sm.cu: the persistent kernel on pairs of CTAs
bool gemm_pair_supported(const GemmDesc& d, int BN, int splits);
const char* gemm_bf16_pair(const GemmDesc& d, const GemmParams& p, int raster_group, cudaStream_t stream);

const char* gemm_bf16(const GemmDesc& d, cudaStream_t stream) {
  if (d.M <= 0 || d.N <= 0 || d.K <= 0) return "gemm_bf16: empty problem";
  if ((reinterpret_cast<uintptr_t>(d.A) & 15) || (reinterpret_cast<uintptr_t>(d.B) & 15)) return "gemm_bf16: operands must be 16-byte aligned";
  if ((d.lda % 8) || (d.ldb % 8)) return "gemm_bf16: leading dimensions must be multiples of 8 elements";
  if (d.out_f32 ? (d.ldc % 4) : (d.ldc % 8)) return "gemm_bf16: ldc alignment";
  if (reinterpret_cast<uintptr_t>(d.C) & 15) return "gemm_bf16: C must be 16-byte aligned";
  if (d.mask_aux || d.had_x0 || d.had_xl) {
    if (d.out_f32) return "gemm_bf16: mask / Hadamard epilogues need a bf16 output";
    if (d.ld_aux % 8) return "gemm_bf16: ld_aux must be a multiple of 8 elements";
    if ((reinterpret_cast<uintptr_t>(d.mask_aux) | reinterpret_cast<uintptr_t>(d.had_x0) | reinterpret_cast<uintptr_t>(d.had_xl)) & 15)
      return "gemm_bf16: auxiliary operands must be 16-byte aligned";
    if (d.had_x0 && !d.had_xl) return "gemm_bf16: Hadamard epilogue needs both x0 and xl";
  }
  if (d.aux_out) {
    if (!d.had_xl || d.mask_aux) return "gemm_bf16: aux_out goes with the Hadamard / residual epilogue";
    if (reinterpret_cast<uintptr_t>(d.aux_out) & 15) return "gemm_bf16: aux_out must be 16-byte aligned";
  }

  // Tile N (multiple of 16; 64 when B is MN-major) and the split-K factor are chosen together with a small
  // cost model fitted to measurements on B200: a CTA ingests operand tiles at ~120 GB/s, the epilogue
  // costs ~22 ns per accumulator column (more for the fp32 reduce), a launch ~3 us, and CTAs run in
  // waves of 148.
  const int n_cover = d.n_store > d.N ? d.n_store : d.N;
  const int kt_total = (d.K + kBK - 1) / kBK;
  const int m_tiles = (d.M + kBM - 1) / kBM;
  const bool may_split = d.out_f32 && d.accumulate;
  if (d.split_k > 1 && !may_split) return "gemm_bf16: split-K needs an fp32 accumulate epilogue";
  int BN = d.BN, splits = d.split_k;
  // Compute-sized problems (several waves of 256 x 512 tiles, a long contraction, no split-K) go to the persistent
  // kernel on pairs of CTAs (gemm_2sm.cu); m_halves == 4 asks for it whatever the size.
  bool pair = false;
  {
    const int bn_pair = d.BN > 0 ? d.BN : 512;
    const long long tiles = (long long)((d.M + 2 * kBM - 1) / (2 * kBM)) * ((n_cover + bn_pair - 1) / bn_pair);
    const bool sized = tiles >= 2 * 74 && kt_total >= 16;
    pair = (d.m_halves == 4 || (d.m_halves == 0 && sized)) && d.split_k <= 1 && gemm_pair_supported(d, bn_pair, 1);
    if (pair) { BN = bn_pair; splits = 1; }
  }
  if (!pair) {
    const int gran = d.b_mn ? 64 : 16;
    double best_cost = 1e30;
    int best_bn = 0, best_sp = 1;
    for (int cand = (BN > 0 ? BN : gran); cand <= (BN > 0 ? BN : 256); cand += gran) {
      const int n_tiles = (n_cover + cand - 1) / cand;
      const int sp_lo = splits > 0 ? splits : 1;
      const int sp_hi = splits > 0 ? splits : (may_split ? (kt_total < 32 ? kt_total : 32) : 1);
      for (int sp = sp_lo; sp <= sp_hi; ++sp) {
        const int ktps = (kt_total + sp - 1) / sp;
        const int sp_eff = (kt_total + ktps - 1) / ktps;
        const long long ctas = (long long)m_tiles * n_tiles * sp_eff;
        const long long waves = (ctas + 147) / 148;
        const double per_cta = ktps * (128.0 + cand) * 1.07 + cand * (d.out_f32 ? 33.0 : 22.0) + 600.0;
        const double cost = waves * per_cta;
        if (cost < best_cost - 1e-9) { best_cost = cost; best_bn = cand; best_sp = sp_eff; }
      }
    }
    BN = best_bn;
    splits = best_sp;
  }
  if (!pair && (BN % 16 || BN < 16 || BN > 256 || (d.b_mn && BN % 64))) return "gemm_bf16: bad tile N";
  if (splits < 1) splits = 1;
  if (splits > kt_total) splits = kt_total;
  int ktps = (kt_total + splits - 1) / splits;
  splits = (kt_total + ktps - 1) / ktps;

  CUtensorMap tmA, tmB;
  if (!pair) {       // the pair kernel makes its own (other box sizes)
    bool ok;
    if (!d.a_mn) ok = get_tensor_map(d.A, d.M, d.K, d.lda, kBM, &tmA);          // [M, K]
    else         ok = get_tensor_map(d.A, d.K, d.M, d.lda, kBK, &tmA);          // [K, M]
    if (!ok) return "gemm_bf16: cuTensorMapEncodeTiled failed for A";
    if (!d.b_mn) ok = get_tensor_map(d.B, d.N, d.K, d.ldb, BN, &tmB);           // [N, K]
    else         ok = get_tensor_map(d.B, d.K, d.N, d.ldb, kBK, &tmB);          // [K, N]
    if (!ok) return "gemm_bf16: cuTensorMapEncodeTiled failed for B";
  }

  // 256-row tiles pay off when the problem is compute-sized: several waves of full-width tiles, no split-K
  int halves = pair ? 2 : d.m_halves;
  if (halves == 4) halves = 0;         // the pair kernel was asked for but does not take this problem
  if (halves == 0) {
    const long long tiles256 = (long long)((d.M + 2 * kBM - 1) / (2 * kBM)) * ((n_cover + BN - 1) / BN);
    // measured on 8192 x 6416 x 6416: (K,K) 1087 -> 1313 TFLOP/s, (K,MN) 1000 -> 1327, (MN,MN) 962 -> 1238
    halves = (BN >= 128 && splits == 1 && tiles256 >= 3 * 148 && kt_total >= 16) ? 2 : 1;
  }
  if (halves != 1 && halves != 2) return "gemm_bf16: m_halves must be 1 or 2";
  if (!pair && halves == 2 && BN > 256) return "gemm_bf16: bad tile N";

  GemmParams p;
  p.m_halves = halves;
  {
    static const int rg_env = []() { const char* e = getenv("TN_GEMM_RASTER_GROUP"); return e ? atoi(e) : -1; }();
    const long long tiles = (long long)((d.M + kBM * halves - 1) / (kBM * halves)) * ((n_cover + BN - 1) / BN);
    p.raster_group = rg_env >= 0 ? rg_env : ((splits == 1 && tiles >= 2 * 148) ? 16 : 1);   // 1 % on 8192 x 6416 x 6416
  }
  p.M = d.M; p.N = d.N; p.K = d.K; p.BN = BN; p.a_mn = d.a_mn; p.b_mn = d.b_mn; p.k_tiles_per_split = ktps;
  p.C = d.C; p.ldc = d.ldc; p.out_f32 = d.out_f32; p.accumulate = d.accumulate; p.relu = d.relu;
  p.mask_aux = reinterpret_cast<const __nv_bfloat16*>(d.mask_aux);
  p.had_x0 = reinterpret_cast<const __nv_bfloat16*>(d.had_x0);
  p.had_xl = reinterpret_cast<const __nv_bfloat16*>(d.had_xl);
  p.aux_out = reinterpret_cast<__nv_bfloat16*>(d.aux_out);
  p.ld_aux = d.ld_aux; p.ones_col = d.ones_col; p.n_store = n_cover; p.bias = d.bias; p.status = d.status; p.prof = d.prof;
  p.gate_flags = d.gate_flags; p.gate_epoch = d.gate_epoch; p.gate_world = d.gate_world; p.gate_wait_ns = d.gate_wait_ns;

  if (pair) return gemm_bf16_pair(d, p, p.raster_group, stream);

  dim3 grid((n_cover + BN - 1) / BN, (d.M + kBM * halves - 1) / (kBM * halves), splits);
  const size_t b_bytes = (size_t)BN * kBK * 2;
  const size_t epi_bytes = (size_t)kEpiWarps * kEpiBytesPerWarp + 1024;
  const size_t a_stage = (size_t)halves * kABytes;
  size_t smem4 = 4 * (a_stage + b_bytes) + 1024, smem3 = 3 * (a_stage + b_bytes) + 1024;
  if (smem4 < epi_bytes) smem4 = epi_bytes;
  if (smem3 < epi_bytes) smem3 = epi_bytes;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<4, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<3, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<3, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    attr_set = true;
  }
  // launched as a programmatic dependent of whatever precedes it in the stream (plain serialisation when the
  // predecessor is not a kernel or the attribute is switched off)
  static const bool use_pdl = []() { const char* e = getenv("TN_PDL"); return e == nullptr || atoi(e) != 0; }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kGemmThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 1 : 0;
  cudaError_t e;
  if (halves == 2) {
    if (smem3 > 220 * 1024) return "gemm_bf16: two-accumulator tile does not fit in shared memory";
    cfg.dynamicSmemBytes = smem3;
    e = cudaLaunchKernelEx(&cfg, gemm_bf16_tcgen05_kernel<3, 2>, tmA, tmB, p);
  } else if (smem4 <= 200 * 1024) {
    cfg.dynamicSmemBytes = smem4;
    e = cudaLaunchKernelEx(&cfg, gemm_bf16_tcgen05_kernel<4, 1>, tmA, tmB, p);
  } else {
    cfg.dynamicSmemBytes = smem3;
    e = cudaLaunchKernelEx(&cfg, gemm_bf16_tcgen05_kernel<3, 1>, tmA, tmB, p);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace tn
