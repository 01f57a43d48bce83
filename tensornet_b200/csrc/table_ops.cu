// Maintenance kernels of the GPU hash table: bulk key insertion (checkpoint load,
// re-sharding), read-only lookup (serving, inspection) and the day-level show/click decay
// sweep (core/ps/optimizer/ada_grad_kernel.cc:191-195, ftrl_kernel.cc:124,
// core/ps/optimizer/optimizer_kernel.h:422-427).
#include "sparse_table.cuh"
#include "tn_ops.h"

namespace tn {

namespace {

// Find-or-insert without row initialisation; out_rows[i] = row index (or -1 when full).
// Keys of one call must be distinct.
__global__ void table_insert_keys_kernel(TableView t, const long long* __restrict__ keys, int n,
                                         int* __restrict__ out_rows, int* status) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const unsigned long long key = canon_key((unsigned long long)keys[i]);
    unsigned h = table_home(t, key);
    int r = -1;
    bool placed = false;
    for (unsigned probes = 0; probes <= t.cap_mask; ++probes) {
      unsigned long long k = __ldcg(&t.keys[h]);
      if (k == kEmptyKey) {
        k = atomicCAS(&t.keys[h], kEmptyKey, key);
        if (k == kEmptyKey) {
          r = atomicAdd(t.n_rows, 1);
          if (r >= t.row_cap) {
            atomicSub(t.n_rows, 1);
            t.slots[h] = -3;
            r = -1;
            set_status(status, kTableFull, 20, 0);
          } else {
            t.row_keys[r] = key;
            t.row_tag[r] = 0ull;
            t.slots[h] = r;
          }
          placed = true;
          break;
        }
      }
      if (k == key) { r = ld_volatile_s32(&t.slots[h]); placed = true; break; }
      h = (h + 1) & t.cap_mask;
    }
    if (!placed) set_status(status, kTableFull, 20, 1);
    out_rows[i] = r;
  }
}

__global__ void table_lookup_kernel(TableView t, const long long* __restrict__ keys, int n, int* __restrict__ out_rows) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    int r = table_find(t, canon_key((unsigned long long)keys[i]));
    out_rows[i] = r < 0 ? -1 : r;
  }
}

__global__ void table_decay_kernel(TableView t, int kind, float rate, int delta_days) {
  const int n = *t.n_rows;
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) {
    float* row = t.rows + (size_t)r * t.stride;
    if (kind == kAdaGrad) {
      row[t.dim + 1] *= rate;
      row[t.dim + 2] *= rate;
      reinterpret_cast<int*>(row)[t.dim + 3] += delta_days;
    } else if (kind == kFtrl) {
      row[3 * t.dim] *= rate;
    }
  }
}

}  // namespace

void launch_table_insert_keys(const TableView& t, const long long* keys, int n, int* out_rows, int* status, cudaStream_t st) {
  if (n <= 0) return;
  int blocks = (n + 255) / 256; if (blocks > 148 * 8) blocks = 148 * 8;
  table_insert_keys_kernel<<<blocks, 256, 0, st>>>(t, keys, n, out_rows, status);
}
void launch_table_lookup(const TableView& t, const long long* keys, int n, int* out_rows, cudaStream_t st) {
  if (n <= 0) return;
  int blocks = (n + 255) / 256; if (blocks > 148 * 8) blocks = 148 * 8;
  table_lookup_kernel<<<blocks, 256, 0, st>>>(t, keys, n, out_rows);
}
void launch_table_decay(const TableView& t, int kind, float rate, int delta_days, cudaStream_t st) {
  table_decay_kernel<<<148 * 4, 256, 0, st>>>(t, kind, rate, delta_days);
}

}  // namespace tn
