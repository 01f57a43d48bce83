// unique_assign: per-batch dedup of raw signs on the GPU with virtual-index assignment and
// show / click counting, as a stand-alone op.  It is the first phase of sparse_pull_fused
// (csrc/sparse_fused.cu) exposed on its own for users that only need the mapping, and the
// counterpart of the reference's SparsePullVarInfo / SparsePushVarInfo constructors
// (core/kernels/sparse_table_ops.cc:113-137,274-297).
//
// Scratch: an open-addressing table of `scratch_cap` (power of two, >= 2 * unique ids) uint64 keys
// plus int32 values.  It must be all-ones (keys) on entry and is returned to that state.
// The virtual index of a sign is the order in which its first occurrence won the insert race,
// not the order of first occurrence in the input; only consistency between `uniq` and `inverse`
// matters to the callers.
#include "tn_device.cuh"
#include "tn_ops.h"

namespace tn {

namespace {

__device__ __forceinline__ unsigned uq_home(unsigned long long key, unsigned mask) {
  return (unsigned)mix64(key ^ 0x2545F4914F6CDD1Dull) & mask;
}

// pass 1: insert; the winner of each key takes the next virtual index (warp-aggregated counter)
__global__ void unique_insert_kernel(const long long* __restrict__ ids, int n, unsigned long long* dd_keys, int* dd_vals,
                                     unsigned mask, unsigned long long* __restrict__ uniq, int cap, int* count, int* status) {
  const int tid = blockIdx.x * blockDim.x + threadIdx.x, nth = gridDim.x * blockDim.x;
  const unsigned lane = threadIdx.x & 31;
  for (int base = tid - (int)lane; base < n; base += nth) {
    const int i = base + (int)lane;
    bool winner = false;
    unsigned hw = 0;
    unsigned long long key = 0;
    key = i < n ? canon_key((unsigned long long)ids[i]) : kEmptyKey;
    const unsigned same = __match_any_sync(0xffffffffu, key);      // one probe per warp and distinct sign
    if (i < n && (int)lane == __ffs(same) - 1) {
      unsigned h = uq_home(key, mask);
      bool done = false;
      for (unsigned probes = 0; probes <= mask; ++probes) {
        // read first: later occurrences of a hot sign find it without queueing an atomic on the same word
        unsigned long long old = __ldcg(&dd_keys[h]);
        if (old == kEmptyKey) old = atomicCAS(&dd_keys[h], kEmptyKey, key);
        if (old == kEmptyKey) { winner = true; hw = h; done = true; break; }
        if (old == key) { done = true; break; }
        h = (h + 1) & mask;
      }
      if (!done) set_status(status, kDedupOverflow, 50, 0);
    }
    __syncwarp();
    const unsigned wm = __ballot_sync(0xffffffffu, winner);
    if (wm) {
      const int leader = __ffs(wm) - 1;
      int b = 0;
      if ((int)lane == leader) b = atomicAdd(count, __popc(wm));
      b = __shfl_sync(0xffffffffu, b, leader);
      if (winner) {
        unsigned lt;
        asm("mov.u32 %0, %%lanemask_lt;" : "=r"(lt));
        const int v = b + __popc(wm & lt);
        if (v < cap) { uniq[v] = key; dd_vals[hw] = v; }
        else { dd_vals[hw] = -1; set_status(status, kOwnerSegOverflow, 50, 0); }
      }
    }
  }
}

// pass 2: inverse map and per-unique show / click counts
__global__ void unique_lookup_kernel(const long long* __restrict__ ids, int n, const unsigned long long* __restrict__ dd_keys,
                                     const int* __restrict__ dd_vals, unsigned mask, int* __restrict__ inverse,
                                     const float* __restrict__ labels, float* show, float* click) {
  const int tid = blockIdx.x * blockDim.x + threadIdx.x, nth = gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  for (int base = tid - lane; base < n; base += nth) {
    const int i = base + lane;
    const bool valid = i < n;
    const unsigned long long key = valid ? canon_key((unsigned long long)ids[i]) : kEmptyKey;
    const unsigned same = __match_any_sync(0xffffffffu, key);
    const int leader = __ffs(same) - 1;
    int v = -1;
    if (valid && lane == leader) {
      unsigned h = uq_home(key, mask);
      for (unsigned probes = 0; probes <= mask; ++probes) {
        const unsigned long long k = dd_keys[h];
        if (k == key) { v = dd_vals[h]; break; }
        if (k == kEmptyKey) break;
        h = (h + 1) & mask;
      }
    }
    v = __shfl_sync(same, v, leader);
    if (valid) inverse[i] = v;
    if (valid && v >= 0) {
      if (show && lane == leader) atomicAdd(show + v, (float)__popc(same));
      if (click && labels && labels[i] != 0.f) atomicAdd(click + v, labels[i]);
    }
  }
}

// pass 3: give the scratch back empty
__global__ void unique_clear_kernel(unsigned long long* dd_keys, unsigned cap) {
  ulonglong2* kk = reinterpret_cast<ulonglong2*>(dd_keys);
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < (cap >> 1); i += gridDim.x * blockDim.x)
    kk[i] = make_ulonglong2(kEmptyKey, kEmptyKey);
}

}  // namespace

void launch_unique_assign(const long long* ids, int n, const float* labels, unsigned long long* dd_keys, int* dd_vals,
                          unsigned scratch_cap, unsigned long long* uniq, int cap, int* inverse, float* show, float* click,
                          int* count, int* status, cudaStream_t st) {
  if (n <= 0) return;
  int blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  unique_insert_kernel<<<blocks, 256, 0, st>>>(ids, n, dd_keys, dd_vals, scratch_cap - 1, uniq, cap, count, status);
  unique_lookup_kernel<<<blocks, 256, 0, st>>>(ids, n, dd_keys, dd_vals, scratch_cap - 1, inverse, labels, show, click);
  int cb = (int)((scratch_cap / 2 + 255) / 256);
  if (cb > 148 * 8) cb = 148 * 8;
  if (cb < 1) cb = 1;
  unique_clear_kernel<<<cb, 256, 0, st>>>(dd_keys, scratch_cap);
}

}  // namespace tn
