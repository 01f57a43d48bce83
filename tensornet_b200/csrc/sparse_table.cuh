// GPU-resident hashed embedding table: open-addressing key array -> row index into a
// dense row slab.  Replaces the reference's 8 mutex-guarded unordered_maps per rank
// (core/ps/optimizer/optimizer_kernel.h:254-437) and its slab allocator
// (core/utility/allocator.h:26-129).
#pragma once
#include "tn_device.cuh"
#include "tn_types.h"

namespace tn {

constexpr unsigned long long kTagNew = 1ull << 31;
constexpr int kReqNewOwner = 1 << 31;   // this request created the row and must initialise it
constexpr int kReqNewCopy = 1 << 30;    // row was created this step by someone else: recompute init, do not read
constexpr int kReqRowMask = (1 << 30) - 1;
constexpr int kReqPending = -2;         // lost the insert race before the row index was published
constexpr int kReqNone = -1;            // no row (table full)

__device__ __forceinline__ unsigned table_home(const TableView& t, unsigned long long key) {
  return (unsigned)mix64(key) & t.cap_mask;
}

// Read-only probe.  Returns row index or -1.
__device__ __forceinline__ int table_find(const TableView& t, unsigned long long key) {
  unsigned h = table_home(t, key);
  for (unsigned probes = 0; probes <= t.cap_mask; ++probes) {
    unsigned long long k = __ldcg(&t.keys[h]);
    if (k == key) return ld_volatile_s32(&t.slots[h]);
    if (k == kEmptyKey) return -1;
    h = (h + 1) & t.cap_mask;
  }
  return -1;
}

// Row field offsets.
__device__ __forceinline__ int off_g2sum(int dim) { return dim; }
__device__ __forceinline__ int off_show(int kind, int dim) { return kind == kAdaGrad ? dim + 1 : 3 * dim; }
__device__ __forceinline__ int off_click(int dim) { return dim + 2; }           // AdaGrad only
__device__ __forceinline__ int off_noshow(int dim) { return dim + 3; }          // AdaGrad only (int32)
__device__ __forceinline__ int off_delta_show(int dim) { return 3 * dim + 1; }  // Adam / Ftrl (int32)

}  // namespace tn
