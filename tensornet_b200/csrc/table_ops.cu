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

// Rebuild the key array of a shard from its row slab: keys[] / slots[] arrive all-empty, every row r < n gets its
// sign (row_keys[r]) back in and points at r.  Used after the key array was replaced by a larger one and after a
// compaction moved rows (the reference's unordered_map rehashes itself, core/ps/optimizer/optimizer_kernel.h:257-270).
__global__ void table_rebuild_index_kernel(TableView t, int n, int* status) {
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x) {
    const unsigned long long key = t.row_keys[r];
    unsigned h = table_home(t, key);
    bool placed = false;
    for (unsigned probes = 0; probes <= t.cap_mask; ++probes) {
      unsigned long long k = __ldcg(&t.keys[h]);
      if (k == kEmptyKey) {
        k = atomicCAS(&t.keys[h], kEmptyKey, key);
        if (k == kEmptyKey) { t.slots[h] = r; placed = true; break; }
      }
      h = (h + 1) & t.cap_mask;
    }
    if (!placed) set_status(status, kTableFull, 21, 0);
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

// ---- checkpoint export ---------------------------------------------------------------------------
// The reference walks its eight sub-maps with one thread each and drops rows by the DeleteByShow rule while
// saving (core/ps/optimizer/optimizer_kernel.h:324-352,462-486; ada_grad_kernel.cc:197-204, ftrl_kernel.cc:126).
// Here a range of the row slab is filtered by the same rule and packed, grouped by block file, into a staging
// buffer that the host copies out in one piece: pass 1 counts the surviving rows per block, pass 2 scatters
// (sign, row) records behind per-block cursors.
__device__ __forceinline__ bool export_drop(const ExportRule& e, int kind, const float* row, int dim) {
  if (!e.enabled) return false;
  if (kind == kAdaGrad) {
    const float show = row[dim + 1];
    const int nsd = reinterpret_cast<const int*>(row)[dim + 3];
    return e.logic == 1 ? (show < e.show_threshold && nsd > e.no_show_days) : (show < e.show_threshold || nsd > e.no_show_days);
  }
  if (kind == kFtrl) return row[3 * dim] < e.show_threshold;
  return false;
}

// keep[r] = 1 unless the eviction rule drops row r (the DeleteByShow rule the reference applies while saving,
// ada_grad_kernel.cc:197-204, ftrl_kernel.cc:126; here it can also shed the rows from the live shard).
__global__ void table_keep_mask_kernel(TableView t, int kind, ExportRule rule, int n, unsigned char* keep) {
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < n; r += gridDim.x * blockDim.x)
    keep[r] = export_drop(rule, kind, t.rows + (size_t)r * t.stride, t.dim) ? 0 : 1;
}

__global__ void table_export_count_kernel(TableView t, int kind, ExportRule rule, int r0, int r1, int* counts) {
  __shared__ int s_cnt[kSparseBlockNum];
  if (threadIdx.x < kSparseBlockNum) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  for (int r = r0 + blockIdx.x * blockDim.x + threadIdx.x; r < r1; r += gridDim.x * blockDim.x) {
    const float* row = t.rows + (size_t)r * t.stride;
    if (!export_drop(rule, kind, row, t.dim)) atomicAdd(&s_cnt[block_of(t.row_keys[r])], 1);
  }
  __syncthreads();
  if (threadIdx.x < kSparseBlockNum && s_cnt[threadIdx.x]) atomicAdd(&counts[threadIdx.x], s_cnt[threadIdx.x]);
}

// counts[0..7] from pass 1; cursors[0..7] start at zero.  G lanes copy one row.
__global__ void table_export_scatter_kernel(TableView t, int kind, ExportRule rule, int r0, int r1, const int* __restrict__ counts,
                                            int* cursors, unsigned long long* out_keys, float* out_rows, int rf, int G) {
  const int lane = threadIdx.x % G;
  const int gid = (blockIdx.x * blockDim.x + threadIdx.x) / G, ngroups = gridDim.x * blockDim.x / G;
  const unsigned wl = threadIdx.x & 31;
  const unsigned gmask = G >= 32 ? 0xffffffffu : (((1u << G) - 1u) << (wl & ~(unsigned)(G - 1)));   // a group decides as one
  for (int r = r0 + gid; r < r1; r += ngroups) {
    const float* row = t.rows + (size_t)r * t.stride;
    if (export_drop(rule, kind, row, t.dim)) continue;
    const unsigned long long key = t.row_keys[r];
    const int b = block_of(key);
    int pos = 0;
    if (lane == 0) {
      int base = 0;
      for (int k = 0; k < b; ++k) base += counts[k];
      pos = base + atomicAdd(&cursors[b], 1);
      out_keys[pos] = key;
    }
    pos = __shfl_sync(gmask, pos, (int)wl - lane);
    float* dst = out_rows + (size_t)pos * rf;
    for (int e = lane; e < rf; e += G) dst[e] = row[e];
  }
}

}  // namespace

void launch_table_export(const TableView& t, int kind, const ExportRule& rule, int r0, int r1, int* counts, int* cursors,
                         unsigned long long* out_keys, float* out_rows, int rf, cudaStream_t st) {
  if (r1 <= r0) return;
  const int n = r1 - r0;
  int blocks = (n + 255) / 256; if (blocks > 148 * 8) blocks = 148 * 8;
  table_export_count_kernel<<<blocks, 256, 0, st>>>(t, kind, rule, r0, r1, counts);
  int G = 1;
  while (G < rf && G < 32) G <<= 1;
  long long threads = (long long)n * G;
  blocks = (int)((threads + 255) / 256); if (blocks > 148 * 8) blocks = 148 * 8;
  table_export_scatter_kernel<<<blocks, 256, 0, st>>>(t, kind, rule, r0, r1, counts, cursors, out_keys, out_rows, rf, G);
}

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
void launch_table_rebuild_index(const TableView& t, int n, int* status, cudaStream_t st) {
  if (n <= 0) return;
  int blocks = (n + 255) / 256; if (blocks > 148 * 8) blocks = 148 * 8;
  table_rebuild_index_kernel<<<blocks, 256, 0, st>>>(t, n, status);
}
void launch_table_keep_mask(const TableView& t, int kind, const ExportRule& rule, int n, unsigned char* keep, cudaStream_t st) {
  if (n <= 0) return;
  int blocks = (n + 255) / 256; if (blocks > 148 * 8) blocks = 148 * 8;
  table_keep_mask_kernel<<<blocks, 256, 0, st>>>(t, kind, rule, n, keep);
}
void launch_table_decay(const TableView& t, int kind, float rate, int delta_days, cudaStream_t st) {
  table_decay_kernel<<<148 * 4, 256, 0, st>>>(t, kind, rate, delta_days);
}

}  // namespace tn
