// Device-side primitives shared by every sm_100a kernel in this library:
// error status words, time-bounded waits (grid barrier, peer flags), system-scope
// loads/stores for NVLink peer memory and vector reductions.
//
// Every wait in this library is bounded by a wall-time budget read from %globaltimer.
// When a wait gives up the kernel records {code, phase, peer} in the status words,
// skips the rest of its work and returns normally, so the CUDA context stays usable
// and the host can raise a Python exception.  Nothing here traps or asserts.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdlib>
#include "tn_hash.h"

namespace tn {

enum StatusCode : int {
  kOk = 0,
  kDedupOverflow = 1,      // per-batch dedup scratch is full
  kOwnerSegOverflow = 2,   // more unique ids for one owner than the segment capacity
  kTableFull = 3,          // hash table key array or row slab exhausted
  kGridBarrierTimeout = 4,
  kPeerWaitTimeout = 5,
  kMbarTimeout = 6,
  kKeyMissing = 7,
  kBadArgument = 8,
};

// status[0]=code (first error wins) status[1]=phase status[2]=peer/aux status[3]=aux2
__device__ __forceinline__ void set_status(int* status, int code, int phase, int aux) {
  if (atomicCAS(&status[0], 0, code) == 0) {
    status[1] = phase;
    status[2] = aux;
  }
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t) :: "memory");
  return t;
}

__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_volatile_s32(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// L1-bypassing loads for data another GPU (or another SM in this launch) has written.
__device__ __forceinline__ float4 ldcg_f4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

__device__ __forceinline__ void red_add_f32x4(float* p, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// ---------------------------------------------------------------------------------------
// Grid barrier for persistent kernels launched cooperatively (all CTAs co-resident).
// `bar[0]` counts arrivals (monotonic within a launch), `bar[1]` counts exiting CTAs, `bar[2..3]` serve
// `last_cta_arrives`; the last CTA to leave the kernel zeroes all four so the next launch starts clean.
// ---------------------------------------------------------------------------------------
struct GridSync {
  unsigned* bar;
  unsigned nblocks;
  unsigned gen;          // barriers passed so far by this CTA
  int* status;
  unsigned long long budget_ns;
  bool failed;

  // `nb`: CTAs taking part (all of the grid by default; a kernel whose CTAs split into roles gives each role its own
  // barrier words and count).
  __device__ __forceinline__ void init(unsigned* b, int* st, unsigned long long budget, unsigned nb = 0) {
    bar = b; nblocks = nb ? nb : gridDim.x; gen = 0; status = st; budget_ns = budget; failed = false;
  }

  // Returns false when the barrier timed out or an earlier phase already failed.
  // `sys_fence`: make this CTA's peer-memory stores visible system-wide first.
  __device__ __forceinline__ bool sync(int phase, bool sys_fence) {
    __shared__ int s_ok;
    // The CTA barrier orders every thread's earlier writes before thread 0's fence, and fences are
    // cumulative, so one fence per CTA publishes them all (the pattern of a cooperative grid sync).
    __syncthreads();
    if (threadIdx.x == 0) {
      if (sys_fence) __threadfence_system(); else __threadfence();
      gen += 1;
      unsigned target = gen * nblocks;
      atomicAdd(&bar[0], 1u);
      int ok = 1;
      unsigned long long t0 = globaltimer_ns();
      unsigned spins = 0;
      while (ld_acquire_gpu_u32(&bar[0]) < target) {
        if (((++spins) & 63u) == 0) {
          if (globaltimer_ns() - t0 > budget_ns) { ok = 0; break; }
          if (ld_volatile_s32(status) != 0) break;
        }
        __nanosleep(32);
      }
      if (!ok) set_status(status, kGridBarrierTimeout, phase, (int)blockIdx.x);
      if (ld_volatile_s32(status) != 0) ok = 0;
      s_ok = ok;
    }
    __syncthreads();
    bool ok = s_ok != 0;
    __syncthreads();
    if (!ok) failed = true;
    return ok;
  }

  // The same barrier in two halves: `arrive` when this CTA's part of a phase is done, `wait` (much later, typically
  // for free) before the first access that needs every CTA's part.  No other barrier of this object may be used in
  // between.  What the CTAs wrote before `arrive` is visible after `wait`.
  __device__ __forceinline__ void arrive() {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      gen += 1;
      atomicAdd(&bar[0], 1u);
    }
  }
  __device__ __forceinline__ bool wait(int phase) {
    __shared__ int s_ok2;
    if (threadIdx.x == 0) {
      const unsigned target = gen * nblocks;
      int ok = 1;
      unsigned long long t0 = globaltimer_ns();
      unsigned spins = 0;
      while (ld_acquire_gpu_u32(&bar[0]) < target) {
        if (((++spins) & 63u) == 0) {
          if (globaltimer_ns() - t0 > budget_ns) { ok = 0; break; }
          if (ld_volatile_s32(status) != 0) break;
        }
        __nanosleep(32);
      }
      if (!ok) set_status(status, kGridBarrierTimeout, phase, (int)blockIdx.x);
      if (ld_volatile_s32(status) != 0) ok = 0;
      s_ok2 = ok;
    }
    __syncthreads();
    const bool ok = s_ok2 != 0;
    __syncthreads();
    if (!ok) failed = true;
    return ok;
  }

  // Call once per CTA on every exit path.
  __device__ __forceinline__ void leave() {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      unsigned prev = atomicAdd(&bar[1], 1u);
      if (prev == nblocks - 1) {
        bar[0] = 0;
        bar[1] = 0;
        bar[2] = 0;
        bar[3] = 0;
        __threadfence();
      }
    }
  }
};

// "Last CTA out": true in exactly one CTA per launch for a given counter, namely the last whose threads all
// reached this point.  Everything the other CTAs wrote before arriving (peer memory included when `sys_fence`)
// is ordered before what the elected CTA does next, so it may publish a completion flag without a grid barrier.
__device__ __forceinline__ bool last_cta_arrives(unsigned* ctr, bool sys_fence, unsigned nb = 0) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (sys_fence) __threadfence_system(); else __threadfence();
    const unsigned prev = atomicAdd(ctr, 1u);
    const int last = prev == (nb ? nb : gridDim.x) - 1;
    if (last) { if (sys_fence) __threadfence_system(); else __threadfence(); }
    s_last = last;
  }
  __syncthreads();
  const bool r = s_last != 0;
  __syncthreads();
  return r;
}

// One thread waits until *flag (a 64-bit word another GPU release-stores) reaches `want`.
// Returns the observed word, or sets status and returns ~0 on expiry.
__device__ __forceinline__ bool wait_flag_ge(const unsigned long long* flag, unsigned long long want_hi32,
                                             unsigned long long* out, unsigned long long budget_ns, int* status,
                                             int phase, int peer) {
  unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  for (;;) {
    unsigned long long v = ld_acquire_sys_u64(flag);
    if ((v >> 32) == want_hi32) { *out = v; return true; }
    if (((++spins) & 63u) == 0) {
      if (globaltimer_ns() - t0 > budget_ns) break;
      if (ld_volatile_s32(status) != 0) return false;
    }
    __nanosleep(64);
  }
  set_status(status, kPeerWaitTimeout, phase, peer);
  return false;
}

// Programmatic dependent launch.  A kernel launched with `launch_pdl` may start while the kernel before it in
// the stream is still draining; `pdl_sync()` is the point after which it may touch data (it returns once the
// previous kernel has completed and its writes are visible) and also lets the next kernel in the stream start its
// own ramp-up.  Both instructions are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_sync() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  static const bool use_pdl = []() { const char* e = getenv("TN_PDL"); return e == nullptr || atoi(e) != 0; }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Lanes-per-row for row-wise kernels: power of two >= ceil(width/4), at most 32.
__host__ __device__ __forceinline__ int lanes_for_width(int width_floats) {
  int chunks = (width_floats + 3) / 4;
  int g = 1;
  while (g < chunks && g < 32) g <<= 1;
  return g;
}

}  // namespace tn
