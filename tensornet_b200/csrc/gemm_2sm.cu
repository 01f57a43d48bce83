// Persistent bf16 GEMM for compute-sized problems (the DCN-v2 cross layers: 8192 x 6416 x 6416) on PAIRS of SMs.
//
// Two CTAs of a thread-block cluster own one 256 x BN output tile (BN = 512, 256 or 128):
//   * each CTA loads ITS OWN operand half by TMA (its 128 rows of A, its BN/2 columns of B) into its own shared
//     memory; nothing is replicated between the two, so an SM ingests half the bytes per FLOP of a one-CTA tile of
//     the same shape;
//   * the even CTA issues tcgen05.mma.cta_group::2, which runs on both SMs' tensor cores and leaves each CTA its 128
//     rows of the accumulator in its own tensor memory;
//   * BN <= 256: the accumulator is double-buffered in TMEM (2 x BN columns), so the four epilogue warps of each CTA
//     drain tile i while the MMAs of tile i+1 run;
//   * BN = 512: two MMAs per contraction step (columns 0-255 and 256-511) share each A tile and fill all 512 TMEM
//     columns.  A 256 x 512 tile reads a quarter fewer operand bytes per FLOP than 256 x 256, and this kernel family is
//     bound by the rate at which one SM takes in operand tiles: on 8192 x 6416 x 6416 both tile shapes (and the one-CTA
//     256 x 256 tile) settle at about 72 GB/s per SM, 10.6 TB/s over the chip, with the tensor pipe 77 % busy.  The
//     epilogue is then not overlapped (8 us per tile), but the operand ring refills for the next tile while it runs.
//     Measured on that shape, forward / dgrad / wgrad: 481 / 481 / 512 us against 497 / 504 / 535 for the one-CTA
//     256 x 256 tile and 551 / 550 / 597 for the pair's 256 x 256 tile (library GEMM: 455);
//   * the pair walks the tile list (static round-robin over the clusters, same L2-friendly raster as the one-CTA
//     kernel), so barrier set-up, TMEM allocation and the pipeline fill are paid once per launch, not per tile.
// Operand layouts, epilogues and error handling are those of gemm_tcgen05.cu (the epilogue code is shared).
// The reference runs these layers as tf.matmul on CPU (examples/common/layers.py:53-59).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdlib>
#include "gemm_tcgen05.h"
#include "tc_primitives.cuh"
#include "gemm_epilogue.cuh"

namespace tn {

using namespace tc;

namespace {

constexpr int kBM = 128;        // rows per CTA (the pair's tile has 256)
constexpr int kBK = 64;
constexpr int kUmmaK = 16;
constexpr int kABytes = kBM * kBK * 2;
constexpr int kNBlockBytes = 128 * kBK * 2;   // this CTA's half (128 columns) of one 256-column block of B

struct PairTiles {
  int tiles_m, tiles_n, raster_group;
  int epi_bytes_per_warp;      // 2 KiB (transpose block only) or gemm_epi::kBytesPerWarp (plus the auxiliary operand blocks)
};

__device__ __forceinline__ void tile_of(const PairTiles& g, int t, int* tile_m, int* tile_n) {
  if (g.raster_group > 1) {
    const int width = g.raster_group * g.tiles_n;
    const int first_m = (t / width) * g.raster_group;
    const int gsize = min(g.tiles_m - first_m, g.raster_group);
    *tile_m = first_m + (t % width) % gsize;
    *tile_n = (t % width) / gsize;
  } else {
    *tile_m = t / g.tiles_n;
    *tile_n = t % g.tiles_n;
  }
}

// kNB: 256-column MMA blocks per tile (2 for BN = 512); kStages: operand ring depth; kEpiW: epilogue warps (a multiple of
// four: warp w reads TMEM lane quarter w % 4).  Threads: warp 0 TMA, warp 1 MMA + TMEM owner, then the epilogue warps.
template <int kNB, int kStages, int kEpiW>
__global__ void __launch_bounds__(32 * (2 + kEpiW), 1)
gemm_bf16_2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                     const PairTiles g) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kStages];     // used in the even CTA: both CTAs' loads of a stage have landed
  __shared__ __align__(8) uint64_t s_empty[kStages];    // in each CTA: the MMAs have read this CTA's stage
  __shared__ __align__(8) uint64_t s_acc_full[2];           // in each CTA: accumulator stage complete
  __shared__ __align__(8) uint64_t s_acc_empty[2];          // used in the even CTA: both CTAs' epilogues have drained the stage
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort_i;
  volatile int* s_abort = &s_abort_i;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: issues the MMAs
  const int BN = p.BN, BNh = BN >> 1;
  const uint32_t b_bytes = (uint32_t)BNh * kBK * 2;
  const uint32_t stage_bytes = (uint32_t)kABytes + b_bytes;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi_smem_off = kStages * stage_bytes;
  constexpr uint32_t kAcc = kNB == 1 ? 2u : 1u;        // accumulator stages in TMEM
  const int nk = (p.K + kBK - 1) / kBK;
  const int n_tiles = g.tiles_m * g.tiles_n;
  const int cid = (int)(blockIdx.x >> 1), ncl = (int)(gridDim.x >> 1);
  const uint32_t tmem_cols = BN >= 256 ? 512u : 256u;

  if (threadIdx.x == 0) {
    *s_abort = 0;
    for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&s_full[s]), 1); mbar_init(smem_u32(&s_empty[s]), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&s_acc_full[a]), 1); mbar_init(smem_u32(&s_acc_empty[a]), 2 * kEpiW); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmA)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmB)) : "memory");
  }
  if (warp == 1) {
    // the same warp of both CTAs allocates: the pair's MMA addresses the same TMEM columns in each
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the other CTA's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem = s_tmem;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) ----------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = cid; t < n_tiles && ok; t += ncl) {
        int tile_m, tile_n;
        tile_of(g, t, &tile_m, &tile_n);
        const int m0 = tile_m * 2 * kBM + (int)rank * kBM;
        const int n0 = tile_n * BN + (int)rank * (kNB == 1 ? BNh : 128);
        for (int i = 0; i < nk; ++i, ++it) {
          const int s = (int)(it % kStages);
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, s_abort)) { *s_abort = 1; ok = false; break; }
          const uint32_t full_even = map_to_cta(smem_u32(&s_full[s]), 0);
          if (rank == 0) mbar_expect_tx(smem_u32(&s_full[s]), 2u * stage_bytes);
          const int kc = i * kBK;
          const uint32_t a_dst = base + s * stage_bytes;
          const uint32_t b_dst = a_dst + kABytes;
          if (!p.a_mn) {
            tma_load_2d_pair(a_dst, &tmA, kc, m0, full_even);
          } else {
            tma_load_2d_pair(a_dst, &tmA, m0, kc, full_even);
            tma_load_2d_pair(a_dst + 8192, &tmA, m0 + 64, kc, full_even);
          }
          if (kNB == 1) {
            if (!p.b_mn) {
              tma_load_2d_pair(b_dst, &tmB, kc, n0, full_even);
            } else {
              for (int c = 0; c < BNh / 64; ++c) tma_load_2d_pair(b_dst + c * 8192, &tmB, n0 + 64 * c, kc, full_even);
            }
          } else {
            // block j of the tile covers columns 256 j .. 256 j + 255; this CTA supplies its 128 of them
#pragma unroll
            for (int j = 0; j < kNB; ++j) {
              const uint32_t bj = b_dst + j * kNBlockBytes;
              if (!p.b_mn) {
                tma_load_2d_pair(bj, &tmB, kc, n0 + 256 * j, full_even);
              } else {
                tma_load_2d_pair(bj, &tmB, n0 + 256 * j, kc, full_even);
                tma_load_2d_pair(bj + 8192, &tmB, n0 + 256 * j + 64, kc, full_even);
              }
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (even CTA) -------------------------------
    if (lane == 0 && rank == 0) {
      // instruction descriptor: D=f32, A=B=bf16, majors, N>>3, M>>4 with M = 256 over the pair
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.a_mn ? 1 : 0) << 15) |
                             ((uint32_t)(p.b_mn ? 1 : 0) << 16) | ((uint32_t)((kNB == 1 ? BN : 256) >> 3) << 17) | ((uint32_t)((2 * kBM) >> 4) << 24);
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u, b_kstep = p.b_mn ? 2048u : 32u;
      uint32_t it = 0, lt = 0;
      bool ok = true;
      // optional diagnosis by cluster 0: [0] start, [1] end of the tile loop, [2] ns spent waiting for operand stages,
      // [3] ns spent waiting for a free accumulator stage, [4] tiles walked, [5] contraction steps per tile
      unsigned long long* prof = (p.prof != nullptr && cid == 0) ? p.prof : nullptr;
      unsigned long long w_full = 0, w_acc = 0, t_mark = 0;
      if (prof) prof[0] = globaltimer_ns();
      for (int t = cid; t < n_tiles && ok; t += ncl, ++lt) {
        const uint32_t a = lt % kAcc, aph = (lt / kAcc) & 1u;
        if (prof) t_mark = globaltimer_ns();
        if (!mbar_wait_cluster(smem_u32(&s_acc_empty[a]), aph ^ 1u, s_abort)) { *s_abort = 1; ok = false; break; }
        if (prof) w_acc += globaltimer_ns() - t_mark;
        tc_fence_after();
        const uint32_t d_tmem = tmem + a * (uint32_t)BN;
        for (int i = 0; i < nk; ++i, ++it) {
          const int s = (int)(it % kStages);
          const uint32_t ph = (it / kStages) & 1u;
          if (prof) t_mark = globaltimer_ns();
          if (!mbar_wait(smem_u32(&s_full[s]), ph, s_abort)) { *s_abort = 1; ok = false; break; }
          if (prof) w_full += globaltimer_ns() - t_mark;
          tc_fence_after();
          const uint32_t a_base = base + s * stage_bytes;
          const uint32_t b_base = a_base + kABytes;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint64_t ad = make_smem_desc(a_base + k * a_kstep, a_lbo, 1024u);
#pragma unroll
            for (int j = 0; j < kNB; ++j) {
              const uint64_t bd = make_smem_desc(b_base + j * kNBlockBytes + k * b_kstep, b_lbo, 1024u);
              umma_f16_2sm(d_tmem + (uint32_t)(256 * j), ad, bd, idesc, (i > 0 || k > 0) ? 1u : 0u);
            }
          }
          // frees the stage in both CTAs once the MMAs have read it
          umma_commit_2sm(smem_u32(&s_empty[s]));
          umma_commit_2sm(map_to_cta(smem_u32(&s_empty[s]), 1));
        }
        if (ok) {
          umma_commit_2sm(smem_u32(&s_acc_full[a]));
          umma_commit_2sm(map_to_cta(smem_u32(&s_acc_full[a]), 1));
        }
      }
      if (prof) { prof[1] = globaltimer_ns(); prof[2] = w_full; prof[3] = w_acc; prof[4] = lt; prof[5] = (unsigned long long)nk; }
    }
    __syncwarp();
  } else {
    // ------------------------------- epilogue (both CTAs, kEpiW / 4 warps per TMEM lane quarter) --
    const int q = warp & 3;
    const int sub = (warp - 2) >> 2;
    uint8_t* sm_out = smem_raw + (base - smem_u32(smem_raw)) + epi_smem_off + (warp - 2) * g.epi_bytes_per_warp;
    const uint32_t acc_empty_even = map_to_cta(smem_u32(&s_acc_empty[0]), 0);
    uint32_t lt = 0;
    bool ok = true;
    for (int t = cid; t < n_tiles && ok; t += ncl, ++lt) {
      int tile_m, tile_n;
      tile_of(g, t, &tile_m, &tile_n);
      const uint32_t a = lt % kAcc, aph = (lt / kAcc) & 1u;
      if (!mbar_wait(smem_u32(&s_acc_full[a]), aph, s_abort)) { *s_abort = 1; ok = false; break; }
      tc_fence_after();
      const int row_base = tile_m * 2 * kBM + (int)rank * kBM + q * 32;
      const uint32_t tm_lane = tmem + ((uint32_t)(q * 32) << 16) + a * (uint32_t)BN;
      gemm_epi::store_rows(p, tm_lane, row_base, tile_n * BN, BN, sub, kEpiW / 4, lane, sm_out);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(acc_empty_even + a * (uint32_t)sizeof(uint64_t));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*s_abort) {
    // a wait ran out: report, give copies in flight time to land, then release TMEM
    if (threadIdx.x == 0) set_status(p.status, kMbarTimeout, 31, (int)blockIdx.x);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();          // neither CTA leaves (or frees TMEM) while the other may still signal it or run MMAs on it
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
  }
}

}  // namespace

// Whether the pair kernel takes this problem (compute-sized, plain epilogue path without split-K or weight gate).
bool gemm_pair_supported(const GemmDesc& d, int BN, int splits) {
  static const int env = []() { const char* e = getenv("TN_GEMM_2SM"); return e ? atoi(e) : 1; }();
  if (!env || splits != 1 || d.gate_flags != nullptr) return false;
  if (BN != 512 && BN != 256 && BN != 128) return false;
  if (d.split_k > 1) return false;
  return true;
}

namespace {

template <int kNB, int kStages, int kEpiW>
cudaError_t launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, const PairTiles& g, int clusters,
                        cudaStream_t stream) {
  const int BN = p.BN;
  const size_t smem = (size_t)kStages * (kABytes + (size_t)(BN / 2) * kBK * 2) + (size_t)kEpiW * g.epi_bytes_per_warp + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_2sm_kernel<kNB, kStages, kEpiW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  if (smem > 226 * 1024) return cudaErrorInvalidValue;
  static const bool use_pdl = []() { const char* e = getenv("TN_PDL"); return e == nullptr || atoi(e) != 0; }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * clusters));
  cfg.blockDim = dim3(32 * (2 + kEpiW));
  cfg.stream = stream;
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_2sm_kernel<kNB, kStages, kEpiW>, tmA, tmB, p, g);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e;
}

}  // namespace

const char* gemm_bf16_pair(const GemmDesc& d, const GemmParams& p_in, int raster_group, cudaStream_t stream) {
  GemmParams p = p_in;
  const int BN = p.BN;
  CUtensorMap tmA, tmB;
  bool ok;
  if (!d.a_mn) ok = get_tensor_map(d.A, d.M, d.K, d.lda, kBM, &tmA);          // [M, K]
  else         ok = get_tensor_map(d.A, d.K, d.M, d.lda, kBK, &tmA);          // [K, M]
  if (!ok) return "gemm_bf16: cuTensorMapEncodeTiled failed for A";
  // [N, K]: a CTA takes 128 columns of each 256-column block (half of the tile's columns when the tile has 128)
  if (!d.b_mn) ok = get_tensor_map(d.B, d.N, d.K, d.ldb, BN >= 256 ? 128 : BN / 2, &tmB);
  else         ok = get_tensor_map(d.B, d.K, d.N, d.ldb, kBK, &tmB);          // [K, N]
  if (!ok) return "gemm_bf16: cuTensorMapEncodeTiled failed for B";
  PairTiles g;
  g.tiles_m = (d.M + 2 * kBM - 1) / (2 * kBM);
  g.tiles_n = (p.n_store + BN - 1) / BN;
  g.raster_group = raster_group;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long clusters = (long long)g.tiles_m * g.tiles_n;
  if (clusters > sms / 2) clusters = sms / 2;
  if (clusters < 1) clusters = 1;
  // Epilogues that read auxiliary operands (ReLU mask, Hadamard / residual step) need 6 KiB of shared memory per
  // epilogue warp, the others 2 KiB: those afford a fourth operand stage and four more epilogue warps at BN = 512.
  const bool has_aux = d.mask_aux != nullptr || d.had_x0 != nullptr || d.had_xl != nullptr;
  g.epi_bytes_per_warp = has_aux ? gemm_epi::kBytesPerWarp : 2048;
  cudaError_t e;
  if (BN == 512) e = has_aux ? launch_pair<2, 3, 12>(tmA, tmB, p, g, (int)clusters, stream)
                             : launch_pair<2, 4, 16>(tmA, tmB, p, g, (int)clusters, stream);
  else { g.epi_bytes_per_warp = gemm_epi::kBytesPerWarp; e = launch_pair<1, 6, 4>(tmA, tmB, p, g, (int)clusters, stream); }
  return e == cudaSuccess ? nullptr : cudaGetErrorString(e);
}

}  // namespace tn
