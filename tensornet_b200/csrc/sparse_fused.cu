// Fused sparse pull and push: the per-batch id dedup / virtual-index assignment, the
// all-to-all exchange with the owning GPUs over NVLink peer memory, the owner-side hash
// probe (insert on miss) and the optimizer update each run as ONE persistent cooperative
// kernel per direction.  Peer traffic is plain ld/st to symmetric-heap addresses with
// release/acquire flags at system scope; no collective library is involved.
//
// What these kernels replace in the reference:
//   pull : SparsePullVarInfo dedup + per-shard RPC fan-out + SparseTable::Pull + scatter back
//          (core/kernels/sparse_table_ops.cc:113-270, core/ps/table/sparse_table.cc:52-66)
//   push : SparsePushVarInfo show/click counting + per-shard RPC + SparseTable::Push + Value::Apply
//          (core/kernels/sparse_table_ops.cc:274-373, core/ps/table/sparse_table.cc:68-83,
//           core/ps/optimizer/{ada_grad,adam,ftrl}_kernel.cc)
//
// Semantics that differ on purpose: the step is synchronous, and gradients of one sign
// arriving from several GPUs (or several columns) are summed and applied once.
//
// Counters that every thread would otherwise hit (per-owner unique counts, the row slab
// bump pointer, the owner-unique index) are advanced once per warp: lanes that need a slot
// are found with a ballot, one lane adds the population count and the others take their
// rank inside the ballot.
#include "sparse_table.cuh"
#include "dense_step.cuh"

namespace tn {

namespace {

constexpr int kThreads = 1024;
constexpr int kRiderUnroll = 2;      // 16-byte reductions in flight per thread of the CTAs that carry the dense step
enum SigKind { kSigPullReq = 0, kSigPullDone = 1, kSigPushReq = 2, kSigPushDone = 3 };
__device__ __forceinline__ unsigned long long* sig_word(unsigned long long* base, int kind, int src) {
  return base + kind * kMaxWorld + src;
}

__device__ __forceinline__ unsigned group_mask(int G) {
  if (G >= 32) return 0xffffffffu;
  unsigned lane = threadIdx.x & 31;
  return ((1u << G) - 1u) << (lane & ~(unsigned)(G - 1));
}
__device__ __forceinline__ unsigned lanemask_lt() {
  unsigned m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// Warp-aggregated "counter += 1 for every lane in `mask`"; returns this lane's old value.
// Must be called by all 32 lanes; lanes outside `mask` get an unspecified value.
__device__ __forceinline__ int warp_alloc(int* counter, unsigned mask) {
  if (mask == 0) return 0;
  const unsigned lane = threadIdx.x & 31;
  const int leader = __ffs(mask) - 1;
  int base = 0;
  if ((int)lane == leader) base = atomicAdd(counter, __popc(mask));
  base = __shfl_sync(0xffffffffu, base, leader);
  return base + __popc(mask & lanemask_lt());
}

// Default value of stored-row element `e` (e < stride) for a brand-new row.
__device__ __forceinline__ float new_row_elem(const SparseOptParams& o, unsigned long long key, int e, int dim) {
  if (e < dim) return o.zero_init ? 0.f : init_weight(o.seed, key, e, dim, o.initial_scale);
  if (o.kind == kAdaGrad && e == dim) return o.initial_g2sum;
  return 0.f;  // slots, show, click; int fields are bit-zero
}

// A group's lanes ask L2 for the 128-byte lines of a row the group will touch in its next loop iteration,
// so the HBM latency of iteration k+1 overlaps the arithmetic and stores of iteration k.
__device__ __forceinline__ void prefetch_row_l2(const float* row, int n_floats, int lane, int G) {
  for (int l = lane; l * 32 < n_floats; l += G) asm volatile("prefetch.global.L2 [%0];" ::"l"(row + 32 * l));
}

__device__ __forceinline__ void prof_mark(const SparseCommView& c, int slot) {
  if (c.prof != nullptr && blockIdx.x == 0 && threadIdx.x == 0) c.prof[slot] = globaltimer_ns();
}

// One requested row, handled by a group of G lanes: initialise a brand-new row (owner) or recompute its initial
// value (other requesters of the same step), or read the stored row; write the pulled row (w[dim], the two CVM
// columns when enabled, zero padding) to `dst`, which is either the requester's matrix itself or a shared-memory
// tile that is written out afterwards.  `rr` is the resolved request word of the probe.
__device__ __forceinline__ void pull_return_row(const PullArgs& a, const TableView& t, int rr, unsigned long long key,
                                                float* dst, int gl, int G) {
  const SparseCommView& c = a.c;
  const SparseOptParams& o = a.opt;
  const int dim = t.dim, stride = t.stride;
  const int uchunks = c.ustride >> 2, rchunks = stride >> 2;
  if (rr == kReqNone) {
    for (int ch = gl; ch < uchunks; ch += G) *reinterpret_cast<float4*>(dst + 4 * ch) = make_float4(0.f, 0.f, 0.f, 0.f);
    return;
  }
  const int r = rr & kReqRowMask;
  float* row = t.rows + (size_t)r * stride;
  if (rr & (kReqNewOwner | kReqNewCopy)) {
    const bool write_row = (rr & kReqNewOwner) != 0;
    const int nch = write_row ? max(rchunks, uchunks) : uchunks;
    for (int ch = gl; ch < nch; ch += G) {
      float4 v;
      v.x = new_row_elem(o, key, 4 * ch + 0, dim);
      v.y = new_row_elem(o, key, 4 * ch + 1, dim);
      v.z = new_row_elem(o, key, 4 * ch + 2, dim);
      v.w = new_row_elem(o, key, 4 * ch + 3, dim);
      if (write_row && ch < rchunks) *reinterpret_cast<float4*>(row + 4 * ch) = v;
      if (ch < uchunks) {
        // pulled row = w[dim] (+ two zero CVM columns for a new row), zero padding
        float4 u;
        u.x = 4 * ch + 0 < dim ? v.x : 0.f;
        u.y = 4 * ch + 1 < dim ? v.y : 0.f;
        u.z = 4 * ch + 2 < dim ? v.z : 0.f;
        u.w = 4 * ch + 3 < dim ? v.w : 0.f;
        *reinterpret_cast<float4*>(dst + 4 * ch) = u;
      }
    }
    return;
  }
  float show = 0.f, click = 0.f;
  if (t.use_cvm && o.kind == kAdaGrad) { show = row[dim + 1]; click = row[dim + 2]; }
  // up to four 16-byte loads in flight per lane (G >= ceil(uchunks / 4)), then the stores
  float4 buf[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int ch = gl + k * G;
    if (ch < uchunks) buf[k] = *reinterpret_cast<const float4*>(row + 4 * ch);   // stride >= ustride by layout
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int ch = gl + k * G;
    if (ch >= uchunks) continue;
    float4 v = buf[k];
    if (4 * ch + 4 > dim) {
      float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        int idx = 4 * ch + kk;
        if (idx >= dim) {
          float x = 0.f;
          if (t.use_cvm && o.kind == kAdaGrad) {
            if (idx == dim) x = show;
            else if (idx == dim + 1) x = logf(click + 1.f) - logf(show + 1.f);
          }
          e[kk] = x;
        }
      }
      v = make_float4(e[0], e[1], e[2], e[3]);
    }
    *reinterpret_cast<float4*>(dst + 4 * ch) = v;
  }
}

}  // namespace

// =======================================================================================
// sparse_pull_fused
// =======================================================================================
// kTiled: the staged row return (PullArgs::tile_rows > 0); one instantiation per form keeps the other form's code and
// registers out of the loop.
template <bool kTiled>
__global__ void __launch_bounds__(kThreads, 1) sparse_pull_fused_kernel(const __grid_constant__ PullArgs a) {
  const SparseCommView& c = a.c;
  // The table's arrays are read through a descriptor in device memory when the caller has one: the shard can then
  // grow (new key array, longer row slab) between two launches of an already captured CUDA graph.
  __shared__ TableView s_tbl;
  if (threadIdx.x == 0) s_tbl = a.tbl_dev != nullptr ? *a.tbl_dev : a.tbl;
  __syncthreads();
  const TableView& t = s_tbl;
  GridSync gs;
  gs.init(c.bar, c.status, c.wait_ns);
  __shared__ unsigned long long s_flag;
  __shared__ int s_n[kMaxWorld];
  __shared__ int s_pre[kMaxWorld + 1];

  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  const int nth = gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  const int W = c.world, R = c.rank, capo = c.capo;
  const unsigned long long epoch = __ldcg(c.epoch) + 1ull;
  const int dim = t.dim;
  const bool need_ou = a.training && W > 1;

  const bool front_done = a.front_done != 0;     // dedup, id dispatch and inverse map already ran (pull_front_*)
  if (tid == 0 && !front_done) *c.ocount = 0;    // (with the front ahead, the push of the previous step re-armed it)
  prof_mark(c, 0);

  if (front_done) {
    // show / click counts of the batch into the gradient records (the front runs while the previous step's records
    // are still in use, so it leaves them alone)
    if (a.training) {
      for (int base = tid - lane; base < a.n_ids; base += nth) {
        const int i = base + lane;
        const bool valid = i < a.n_ids;
        const int v = valid ? a.inverse[i] : -1;
        const unsigned same = __match_any_sync(0xffffffffu, (valid && v >= 0) ? v : -2 - lane);
        if (valid && v >= 0) {
          float* rec = c.cnts + 2 * (size_t)v;
          if (lane == __ffs(same) - 1) atomicAdd(rec, (float)__popc(same));
          if (a.labels != nullptr) {
            float y = a.label_mod > 0 ? a.labels[i % a.label_mod] : a.labels[i];
            if (y != 0.f) atomicAdd(rec + 1, y);
          }
        }
      }
    }
    prof_mark(c, 1);
    prof_mark(c, 2);
  } else {
  // ---- phase A: dedup; first occurrence of a sign allocates a slot in its owner's segment --------
  for (int base = tid - lane; base < a.n_ids; base += nth) {
    const int i = base + lane;
    bool winner = false;
    unsigned hw = 0;
    unsigned long long key = 0;
    if (i < a.n_ids) key = canon_key((unsigned long long)a.ids[i]);
    else key = kEmptyKey;
    // lanes of the warp that carry the same sign elect one representative: a hot sign costs one probe per warp
    const unsigned same = __match_any_sync(0xffffffffu, key);
    if (i < a.n_ids && lane == __ffs(same) - 1) {
      unsigned h = (unsigned)mix64(key ^ 0x2545F4914F6CDD1Dull) & c.dd_mask;
      bool done = false;
      for (unsigned probes = 0; probes <= c.dd_mask; ++probes) {
        // read first: later occurrences of a hot sign find it without queueing an atomic on the same word
        unsigned long long old = __ldcg(&c.dd_keys[h]);
        if (old == kEmptyKey) old = atomicCAS(&c.dd_keys[h], kEmptyKey, key);
        if (old == kEmptyKey) { winner = true; hw = h; done = true; break; }
        if (old == key) { done = true; break; }
        h = (h + 1) & c.dd_mask;
      }
      if (!done) set_status(c.status, kDedupOverflow, 1, 0);
    }
    __syncwarp();
    int owner = 0, pos = 0;
    if (W == 1) {
      pos = warp_alloc(&c.cnt[0], __ballot_sync(0xffffffffu, winner));
    } else {
      owner = winner ? owner_of(key, W) : -1;
      const unsigned peers = __match_any_sync(0xffffffffu, owner);
      if (winner) {
        const int leader = __ffs(peers) - 1;
        int b = 0;
        if (lane == leader) b = atomicAdd(&c.cnt[owner], __popc(peers));
        b = __shfl_sync(peers, b, leader);
        pos = b + __popc(peers & lanemask_lt());
      }
    }
    if (winner) {
      if (pos >= capo) {
        set_status(c.status, kOwnerSegOverflow, 1, owner);
        c.dd_vals[hw] = -1;
      } else {
        c.stage_ids[owner * capo + pos] = key;
        c.dd_vals[hw] = owner * capo + pos;
      }
    }
  }
  if (!gs.sync(1, false)) goto done;
  prof_mark(c, 1);

  // ---- phase A2: ship id segments to the owners (first, so that the link latency and the owners' wait overlap
  // the rest of this phase), then inverse map and show/click counts ---------------------------------------
  if (W > 1) {
    // coalesced 16-byte peer stores of each owner's id segment
    for (int p = 0; p < W; ++p) {
      if (p == R) continue;
      int n = __ldcg(&c.cnt[p]);
      if (n > capo) n = capo;
      const ulonglong2* src = reinterpret_cast<const ulonglong2*>(c.stage_ids + (size_t)p * capo);
      ulonglong2* dst = reinterpret_cast<ulonglong2*>(c.inbox_ids[p] + (size_t)R * capo);
      int n2 = (n + 1) >> 1;
      for (int j = tid; j < n2; j += nth) dst[j] = __ldcg(&src[j]);
    }
    // no grid barrier: the CTA that finishes shipping last tells the owners their segments are complete, while
    // the others already probe the local segment (which only needs phase A, and that is behind barrier 1)
    if (last_cta_arrives(&c.bar[2], true) && threadIdx.x < W && threadIdx.x != R) {
      int p = threadIdx.x;
      int n = min(__ldcg(&c.cnt[p]), capo);
      st_release_sys_u64(sig_word(c.sig[p], kSigPullReq, R), (epoch << 32) | (unsigned long long)n);
    }
  }
  for (int base = tid - lane; base < a.n_ids; base += nth) {
    const int i = base + lane;
    const bool valid = i < a.n_ids;
    const unsigned long long key = valid ? canon_key((unsigned long long)a.ids[i]) : kEmptyKey;
    const unsigned same = __match_any_sync(0xffffffffu, key);
    const int leader = __ffs(same) - 1;
    int v = -1;
    if (valid && lane == leader) {
      unsigned h = (unsigned)mix64(key ^ 0x2545F4914F6CDD1Dull) & c.dd_mask;
      for (unsigned probes = 0; probes <= c.dd_mask; ++probes) {
        unsigned long long k = __ldcg(&c.dd_keys[h]);
        if (k == key) { v = __ldcg(&c.dd_vals[h]); break; }
        if (k == kEmptyKey) break;
        h = (h + 1) & c.dd_mask;
      }
    }
    v = __shfl_sync(same, v, leader);
    if (valid) a.inverse[i] = v;
    if (a.training && valid && v >= 0) {
      float* rec = c.cnts + 2 * (size_t)v;                             // compact (show, click) pair: stays in L2
      if (lane == leader) atomicAdd(rec, (float)__popc(same));      // show: occurrences, one add per warp and sign
      if (a.labels != nullptr) {
        float y = a.label_mod > 0 ? a.labels[i % a.label_mod] : a.labels[i];
        if (y != 0.f) atomicAdd(rec + 1, y);
      }
    }
  }
  gs.arrive();       // this CTA no longer reads the dedup scratch; phase C waits for all of them before clearing it
  prof_mark(c, 2);
  }

  // ---- phase B: as owner, probe / insert every requested sign and return its row ----------------------
  // A warp takes 32 requests at a time: every lane probes (or inserts) one sign, then the warp's lane groups
  // return the 32 rows.  No grid barrier separates probing from the row return, so the row stores of one warp
  // cross NVLink while other warps still wait on their probes.  Two passes: this GPU's own segment first
  // (nothing to wait for), then the segments of all other senders as ONE flat space of units, so that with many
  // GPUs no warp idles on a short per-sender segment.  A unit is one shared-memory tile of the staged return
  // (tile_rows consecutive requests of one sender) or, without staging, a single request.
  // s_pre[k] = units of the senders that precede the k-th sender of the pass.
  {
    const int G = a.lanes;
    const int gl = threadIdx.x % G, sub = lane / G, rpp = 32 / G;
    const int ustride = c.ustride, uchunks = ustride >> 2;
    const int TR = kTiled ? a.tile_rows : 0;
    const int urows = kTiled ? TR : 1;
    const int upw = 32 / urows;                        // units per warp step
    extern __shared__ float4 s_tiles[];
    float* tile = reinterpret_cast<float*>(s_tiles) + (size_t)(threadIdx.x >> 5) * TR * ustride;
    const int n_warps = nth >> 5;
    for (int part = 0; part < (W > 1 ? 2 : 1); ++part) {
      __syncthreads();
      if (part == 0 && threadIdx.x == 0) {
        const int v = min(__ldcg(&c.cnt[R]), capo);
        s_n[R] = v;
        if (blockIdx.x == 0) c.req_n[R] = v;
        s_pre[0] = 0;
        s_pre[1] = (v + urows - 1) / urows;
        s_flag = (unsigned long long)s_pre[1];
      }
      if (part == 1 && threadIdx.x < 32) {
        // one lane per sender: the W-1 flags are polled side by side, the counts they carry are turned into the
        // flat unit space with a warp scan
        const int k = threadIdx.x;
        const int sk = (R + 1 + k) % W;
        unsigned long long f = 0;
        bool ok = true;
        if (k + 1 < W) ok = wait_flag_ge(sig_word(c.sig[R], kSigPullReq, sk), epoch, &f, c.wait_ns, c.status, 3, sk);
        const bool all_ok = __all_sync(0xffffffffu, ok);
        const int n_k = (k + 1 < W && all_ok) ? (int)(f & 0xffffffffull) : 0;
        int incl = (n_k + urows - 1) / urows;
#pragma unroll
        for (int o = 1; o < kMaxWorld; o <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, incl, o);
          if (k >= o) incl += up;
        }
        if (k + 1 < W) {
          s_n[sk] = n_k;
          if (blockIdx.x == 0) c.req_n[sk] = n_k;
          s_pre[k + 1] = incl;
        }
        if (k == 0) s_pre[0] = 0;
        const int total = __shfl_sync(0xffffffffu, incl, W - 2);
        if (k == 0) s_flag = all_ok ? (unsigned long long)total : ~0ull;
      }
      __syncthreads();
      if (s_flag == ~0ull) { gs.failed = true; break; }
      const int n_units = (int)(s_flag & 0xffffffffull);
      const int first = part == 0 ? R : R + 1;
      // units per warp step: all 32 lanes probe when there is enough work for every warp, fewer when a small batch
      // would otherwise leave most warps idle while a few return 32 rows one after the other
      int su = min(upw, (n_units + n_warps - 1) / n_warps);
      if (!kTiled) su = min(32, (su + rpp - 1) / rpp * rpp);
      if (su < 1) su = 1;
      for (int wu = (tid >> 5) * su; wu < n_units; wu += n_warps * su) {
        // -- probe: one request per lane
        const int lu = lane / urows;
        const int u = wu + lu;
        int s = R, j = 0;
        bool valid = false;
        if (lu < su && u < n_units) {
          int k = 0;
          while (u >= s_pre[k + 1]) ++k;
          s = (first + k) % W;
          j = (u - s_pre[k]) * urows + lane % urows;
          valid = j < s_n[s];
        }
        const unsigned long long* src = (s == R) ? c.stage_ids + (size_t)R * capo : c.inbox_ids[R] + (size_t)s * capo;
        int rr = kReqNone, ou = -1;
        bool is_new = false, need_claim = false;
        unsigned hnew = 0;
        int r_exist = -1;
        unsigned long long tag_seen = 0, key = 0;
        if (valid) {
          key = __ldcg(&src[j]);
          unsigned h = table_home(t, key);
          bool placed = false;
          for (unsigned probes = 0; probes <= t.cap_mask; ++probes) {
            unsigned long long k = __ldcg(&t.keys[h]);
            if (k == kEmptyKey) {
              if (a.lookup_only) { placed = true; break; }        // read-only table (serving): an unknown sign pulls zeros
              k = atomicCAS(&t.keys[h], kEmptyKey, key);
              if (k == kEmptyKey) { is_new = true; hnew = h; placed = true; break; }
            }
            if (k == key) {
              const int r = ld_volatile_s32(&t.slots[h]);
              if (r == -1) {          // inserter has not published the row yet: resolved below, after this warp's own inserts
                rr = kReqPending;
                ou = (int)h;
              } else if (r >= 0) {
                rr = r;
                if (W > 1) {
                  const unsigned long long tg = *((volatile unsigned long long*)&t.row_tag[r]);
                  if ((tg >> 32) == epoch) {
                    if (tg & kTagNew) rr = r | kReqNewCopy;
                    if (need_ou) ou = (int)(tg & 0x7fffffffull);
                  } else if (need_ou) {
                    need_claim = true; r_exist = r; tag_seen = tg;
                  }
                }
              }
              placed = true;
              break;
            }
            h = (h + 1) & t.cap_mask;
          }
          if (!placed) set_status(c.status, kTableFull, 3, s);
        }
        __syncwarp();
        const unsigned nm = __ballot_sync(0xffffffffu, is_new);
        const unsigned cm = __ballot_sync(0xffffffffu, need_claim);
        const int r_new = warp_alloc(t.n_rows, nm);
        int my_ou = -1;
        if (need_ou) my_ou = warp_alloc(c.ocount, nm | cm);
        if (is_new) {
          if (r_new >= t.row_cap) {
            atomicSub(t.n_rows, 1);
            set_status(c.status, kTableFull, 3, s);
            *((volatile int*)&t.slots[hnew]) = -3;
            if (need_ou) c.ou_row[my_ou] = -1;
          } else {
            t.row_keys[r_new] = key;
            unsigned long long tag = (epoch << 32) | kTagNew;
            if (need_ou) { c.ou_row[my_ou] = r_new; tag |= (unsigned long long)my_ou; ou = my_ou; }
            t.row_tag[r_new] = tag;
            __threadfence();
            *((volatile int*)&t.slots[hnew]) = r_new;
            rr = r_new | kReqNewOwner;
          }
        } else if (need_claim) {
          const unsigned long long old = atomicCAS(&t.row_tag[r_exist], tag_seen, (epoch << 32) | (unsigned long long)my_ou);
          if (old == tag_seen) {
            c.ou_row[my_ou] = r_exist;
            ou = my_ou;
          } else {                     // another sender claimed the row first: my index stays a hole
            c.ou_row[my_ou] = -1;
            ou = (int)(old & 0x7fffffffull);
          }
        }
        __syncwarp();
        if (rr == kReqPending) {
          // Another thread won the insert of this sign in this very step and publishes the row index a few
          // instructions after its CAS (a lane of this warp has done so above); wait for it, with a limit.
          const int h = ou;
          int r = ld_volatile_s32(&t.slots[h]);
          const unsigned long long t0 = globaltimer_ns();
          while (r == -1) {
            if (globaltimer_ns() - t0 > c.wait_ns) { set_status(c.status, kGridBarrierTimeout, 4, s); break; }
            r = ld_volatile_s32(&t.slots[h]);
          }
          __threadfence();
          rr = kReqNone;
          ou = -1;
          if (r >= 0) {
            const unsigned long long tg = *((volatile unsigned long long*)&t.row_tag[r]);
            const bool fresh = (tg >> 32) == epoch && (tg & kTagNew);
            rr = fresh ? (r | kReqNewCopy) : r;
            if (need_ou) ou = (int)(tg & 0x7fffffffull);
          }
        }
        if (valid) {
          const int q = s * capo + j;
          c.req_row[q] = rr;
          c.req_ou[q] = ou;
        }
        __syncwarp();
        // -- return: groups of G lanes take the warp's rows in turn
        const unsigned vmask = __ballot_sync(0xffffffffu, valid);
        if (kTiled) {
          // Staged return: the warp gathers the rows of a tile into shared memory and then writes the tile out as
          // one contiguous run of full 128-byte lines (16 bytes per lane, 512 per instruction).  Row-by-row stores
          // of short rows (80 bytes for dim 16 + linear) reach a peer as partial lines and lose about a third of
          // the NVLink write rate; the local case gains too.
          for (int ti = 0; ti < su; ++ti) {
            const unsigned tmask = (vmask >> (ti * TR)) & (TR >= 32 ? 0xffffffffu : ((1u << TR) - 1u));
            if (tmask == 0) continue;
            const int nrows = __popc(tmask);            // the valid requests of a tile are its first ones
            const int s_t = __shfl_sync(0xffffffffu, s, ti * TR), j0 = __shfl_sync(0xffffffffu, j, ti * TR);
            for (int p0 = 0; p0 < TR; p0 += rpp) {
              const int jr = p0 + sub;
              const int from = (ti * TR + jr) & 31;
              const int rr_s = __shfl_sync(0xffffffffu, rr, from);
              const unsigned long long key_s = __shfl_sync(0xffffffffu, key, from);
              if (jr < nrows) pull_return_row(a, t, rr_s, key_s, tile + (size_t)jr * ustride, gl, G);
            }
            __syncwarp();
            float4* d4 = reinterpret_cast<float4*>(c.U[s_t] + ((size_t)R * capo + j0) * ustride);
            const float4* t4 = reinterpret_cast<const float4*>(tile);
            const int n4 = nrows * uchunks;
            for (int i = lane; i < n4; i += 32) d4[i] = t4[i];
            __syncwarp();
          }
        } else {
          for (int p0 = 0; p0 < su; p0 += rpp) {
            const int from = p0 + sub;
            const int rr_s = __shfl_sync(0xffffffffu, rr, from);
            const unsigned long long key_s = __shfl_sync(0xffffffffu, key, from);
            const int s_s = __shfl_sync(0xffffffffu, s, from), j_s = __shfl_sync(0xffffffffu, j, from);
            if ((vmask >> from) & 1u)
              pull_return_row(a, t, rr_s, key_s, c.U[s_s] + ((size_t)R * capo + j_s) * ustride, gl, G);
          }
        }
      }
      if (part == 0) prof_mark(c, 3);
    }
  }
  if (gs.failed) goto done;
  if (c.prof != nullptr && threadIdx.x == 0) atomicMax(&c.prof[6], globaltimer_ns());   // slowest CTA's end of the row return
  prof_mark(c, 4);

  // ---- phase C: tell the requesters their rows have landed; clear the dedup scratch while the flags travel -----
  {
    // The CTA that returns its rows last saves the per-owner counts of this step for pooling / push and re-arms
    // them, and tells every requester that its matrix is complete; CTA 0 then keeps the kernel alive until the
    // same word has arrived from every owner.
    const bool last = last_cta_arrives(&c.bar[3], W > 1);
    if (last && threadIdx.x < W) {
      c.cnt_saved[threadIdx.x] = min(c.cnt[threadIdx.x], capo);
      c.cnt[threadIdx.x] = 0;
      if (threadIdx.x != R) st_release_sys_u64(sig_word(c.sig[threadIdx.x], kSigPullDone, R), epoch << 32);
    }
    if (!front_done) {
      if (!gs.wait(4)) goto done;      // every CTA has finished its inverse map (it arrived before phase B)
      ulonglong2* kk = reinterpret_cast<ulonglong2*>(c.dd_keys);
      const int n2 = (int)((c.dd_mask + 1u) >> 1);
      for (int i = tid; i < n2; i += nth) kk[i] = make_ulonglong2(kEmptyKey, kEmptyKey);
    }
    if (W > 1 && blockIdx.x == 0 && threadIdx.x < W && threadIdx.x != R) {
      unsigned long long v;
      wait_flag_ge(sig_word(c.sig[R], kSigPullDone, threadIdx.x), epoch, &v, c.wait_ns, c.status, 6, threadIdx.x);
    }
    __syncthreads();
  }
  if (tid == 0) *c.epoch = epoch;
  prof_mark(c, 5);

done:
  gs.leave();
}

// =======================================================================================
// pull front: phases A and A2 of the pull (without the show / click counts) as two ordinary kernels.  They need
// only the ids of a batch, so they can run on a second stream while the previous step's forward and backward
// passes run; their CTAs are small and fit beside the GEMM CTAs.  `c.bar[4]` counts the CTAs of the second kernel
// (the cooperative kernels of the same link use bar[0..3] and may run at the same time).
// =======================================================================================
constexpr int kFrontThreads = 256;

__global__ void __launch_bounds__(kFrontThreads) pull_front_dedup_kernel(const __grid_constant__ PullArgs a) {
  const SparseCommView& c = a.c;
  // one read per CTA: all its threads take the same way out (a CTA barrier follows in the shipping kernel)
  __shared__ int s_bad;
  if (threadIdx.x == 0) s_bad = ld_volatile_s32(c.status);
  __syncthreads();
  if (s_bad != 0) return;
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  const int nth = gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  const int W = c.world, capo = c.capo;
  if (c.prof != nullptr && tid == 0) c.prof[16] = globaltimer_ns();
  for (int base = tid - lane; base < a.n_ids; base += nth) {
    const int i = base + lane;
    bool winner = false;
    unsigned hw = 0;
    unsigned long long key = kEmptyKey;
    if (i < a.n_ids) key = canon_key((unsigned long long)a.ids[i]);
    const unsigned same = __match_any_sync(0xffffffffu, key);
    if (i < a.n_ids && lane == __ffs(same) - 1) {
      unsigned h = (unsigned)mix64(key ^ 0x2545F4914F6CDD1Dull) & c.dd_mask;
      bool done = false;
      for (unsigned probes = 0; probes <= c.dd_mask; ++probes) {
        unsigned long long old = __ldcg(&c.dd_keys[h]);
        if (old == kEmptyKey) old = atomicCAS(&c.dd_keys[h], kEmptyKey, key);
        if (old == kEmptyKey) { winner = true; hw = h; done = true; break; }
        if (old == key) { done = true; break; }
        h = (h + 1) & c.dd_mask;
      }
      if (!done) set_status(c.status, kDedupOverflow, 1, 0);
    }
    __syncwarp();
    int owner = 0, pos = 0;
    if (W == 1) {
      pos = warp_alloc(&c.cnt[0], __ballot_sync(0xffffffffu, winner));
    } else {
      owner = winner ? owner_of(key, W) : -1;
      const unsigned peers = __match_any_sync(0xffffffffu, owner);
      if (winner) {
        const int leader = __ffs(peers) - 1;
        int b = 0;
        if (lane == leader) b = atomicAdd(&c.cnt[owner], __popc(peers));
        b = __shfl_sync(peers, b, leader);
        pos = b + __popc(peers & lanemask_lt());
      }
    }
    if (winner) {
      if (pos >= capo) {
        set_status(c.status, kOwnerSegOverflow, 1, owner);
        c.dd_vals[hw] = -1;
      } else {
        c.stage_ids[owner * capo + pos] = key;
        c.dd_vals[hw] = owner * capo + pos;
      }
    }
  }
  if (c.prof != nullptr && threadIdx.x == 0) atomicMax(&c.prof[17], globaltimer_ns());      // last CTA's end
}

__global__ void __launch_bounds__(kFrontThreads) pull_front_ship_kernel(const __grid_constant__ PullArgs a) {
  const SparseCommView& c = a.c;
  // one read per CTA: all its threads take the same way out (a CTA barrier follows in the shipping kernel)
  __shared__ int s_bad;
  if (threadIdx.x == 0) s_bad = ld_volatile_s32(c.status);
  __syncthreads();
  if (s_bad != 0) return;
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  const int nth = gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  const int W = c.world, R = c.rank, capo = c.capo;
  const unsigned long long epoch = __ldcg(c.epoch) + 1ull;
  if (W > 1) {
    for (int p = 0; p < W; ++p) {
      if (p == R) continue;
      int n = __ldcg(&c.cnt[p]);
      if (n > capo) n = capo;
      const ulonglong2* src = reinterpret_cast<const ulonglong2*>(c.stage_ids + (size_t)p * capo);
      ulonglong2* dst = reinterpret_cast<ulonglong2*>(c.inbox_ids[p] + (size_t)R * capo);
      const int n2 = (n + 1) >> 1;
      for (int j = tid; j < n2; j += nth) dst[j] = __ldcg(&src[j]);
    }
    // the CTA that finishes shipping last tells the owners their segments are complete and re-arms the counter
    if (last_cta_arrives(&c.bar[4], true)) {
      if (threadIdx.x < W && threadIdx.x != R) {
        const int p = threadIdx.x;
        const int n = min(__ldcg(&c.cnt[p]), capo);
        st_release_sys_u64(sig_word(c.sig[p], kSigPullReq, R), (epoch << 32) | (unsigned long long)n);
      }
      if (threadIdx.x == 0) c.bar[4] = 0;
    }
  }
  for (int base = tid - lane; base < a.n_ids; base += nth) {
    const int i = base + lane;
    const bool valid = i < a.n_ids;
    const unsigned long long key = valid ? canon_key((unsigned long long)a.ids[i]) : kEmptyKey;
    const unsigned same = __match_any_sync(0xffffffffu, key);
    const int leader = __ffs(same) - 1;
    int v = -1;
    if (valid && lane == leader) {
      unsigned h = (unsigned)mix64(key ^ 0x2545F4914F6CDD1Dull) & c.dd_mask;
      for (unsigned probes = 0; probes <= c.dd_mask; ++probes) {
        unsigned long long k = __ldcg(&c.dd_keys[h]);
        if (k == key) { v = __ldcg(&c.dd_vals[h]); break; }
        if (k == kEmptyKey) break;
        h = (h + 1) & c.dd_mask;
      }
    }
    v = __shfl_sync(same, v, leader);
    if (valid) a.inverse[i] = v;
  }
  if (c.prof != nullptr && threadIdx.x == 0) atomicMax(&c.prof[18], globaltimer_ns());      // last CTA's end
}

// =======================================================================================
// sparse_push_fused
// =======================================================================================
namespace {

// The row updates run at 1024 threads per SM with a dozen memory operations per element group; IEEE division and
// square root (software sequences of 10-20 instructions each) then cost as much issue time as the memory
// round trips.  The approximate forms are good to 2 ulp, far inside the parity tolerance with the CPU restatement.
__device__ __forceinline__ float fast_sqrt(float x) {
  float y;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_div(float a, float b) { return __fdividef(a, b); }

// One optimizer step on one row by a group of G lanes.  `g` points at the gradient (dim floats), bshow / bclick
// are the batch's show and click counts of the sign.   Math as in the reference's Sparse*Value::Apply.
// VEC: dim is a multiple of 4, every lane works on float4 chunks.
template <bool VEC>
__device__ __forceinline__ void apply_row(const SparseOptParams& o, float* row, const float* g, float bshow, float bclick,
                                          int dim, int lane, int G, unsigned gmask) {
  if (o.kind == kAdaGrad) {
    if (VEC && (dim >> 2) <= 2 * G) {
      // Every load of the row is issued before the first use, so a row costs one memory round trip instead of
      // three (gradient -> squared norm -> accumulator -> weights): up to two float4 chunks per lane.
      const int nch = dim >> 2;
      const int c0 = lane, c1 = lane + G;
      float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0, w0 = x0, w1 = x0;
      if (c0 < nch) { x0 = *reinterpret_cast<const float4*>(g + 4 * c0); w0 = *reinterpret_cast<const float4*>(row + 4 * c0); }
      if (c1 < nch) { x1 = *reinterpret_cast<const float4*>(g + 4 * c1); w1 = *reinterpret_cast<const float4*>(row + 4 * c1); }
      const float g2old = row[dim];
      float ss = x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w;
      ss += x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w;
      for (int off = G >> 1; off > 0; off >>= 1) ss += __shfl_xor_sync(gmask, ss, off);
      const float g2 = g2old + ss / (float)dim;
      const float scale = fast_div(o.lr, o.eps + fast_sqrt(g2));
      if (c0 < nch) {
        w0.x -= scale * x0.x; w0.y -= scale * x0.y; w0.z -= scale * x0.z; w0.w -= scale * x0.w;
        *reinterpret_cast<float4*>(row + 4 * c0) = w0;
      }
      if (c1 < nch) {
        w1.x -= scale * x1.x; w1.y -= scale * x1.y; w1.z -= scale * x1.z; w1.w -= scale * x1.w;
        *reinterpret_cast<float4*>(row + 4 * c1) = w1;
      }
      __syncwarp(gmask);
      if (lane == 0) {
        row[dim] = g2;
        row[dim + 1] += bshow;
        row[dim + 2] += bclick;
        reinterpret_cast<int*>(row)[dim + 3] = 0;
      }
      return;
    }
    float ss = 0.f;
    if (VEC) {
      for (int ch = lane; ch < (dim >> 2); ch += G) {
        const float4 x = *reinterpret_cast<const float4*>(g + 4 * ch);
        ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
      }
    } else {
      for (int e = lane; e < dim; e += G) { float x = g[e]; ss += x * x; }
    }
    for (int off = G >> 1; off > 0; off >>= 1) ss += __shfl_xor_sync(gmask, ss, off);
    const float g2 = row[dim] + ss / (float)dim;
    const float scale = o.lr / (o.eps + sqrtf(g2));
    if (VEC) {
      for (int ch = lane; ch < (dim >> 2); ch += G) {
        const float4 x = *reinterpret_cast<const float4*>(g + 4 * ch);
        float4 w = *reinterpret_cast<float4*>(row + 4 * ch);
        w.x -= scale * x.x; w.y -= scale * x.y; w.z -= scale * x.z; w.w -= scale * x.w;
        *reinterpret_cast<float4*>(row + 4 * ch) = w;
      }
    } else {
      for (int e = lane; e < dim; e += G) row[e] -= scale * g[e];
    }
    __syncwarp(gmask);
    if (lane == 0) {
      row[dim] = g2;
      row[dim + 1] += bshow;
      row[dim + 2] += bclick;
      reinterpret_cast<int*>(row)[dim + 3] = 0;
    }
  } else if (o.kind == kAdam) {
    float* m = row + dim;
    float* v = row + 2 * dim;
    const float c1 = 1.f - o.beta1, c2 = 1.f - o.beta2;
    if (VEC) {
      for (int ch = lane; ch < (dim >> 2); ch += G) {
        const float4 x = *reinterpret_cast<const float4*>(g + 4 * ch);
        float4 mm = *reinterpret_cast<float4*>(m + 4 * ch), vv = *reinterpret_cast<float4*>(v + 4 * ch);
        float4 w = *reinterpret_cast<float4*>(row + 4 * ch);
#define TN_SADAM(cmp) \
        mm.cmp = o.beta1 * mm.cmp + c1 * x.cmp; vv.cmp = o.beta2 * vv.cmp + c2 * x.cmp * x.cmp; \
        w.cmp -= fast_div(o.lr * mm.cmp, o.eps + fast_sqrt(vv.cmp));
        TN_SADAM(x) TN_SADAM(y) TN_SADAM(z) TN_SADAM(w)
#undef TN_SADAM
        *reinterpret_cast<float4*>(m + 4 * ch) = mm;
        *reinterpret_cast<float4*>(v + 4 * ch) = vv;
        *reinterpret_cast<float4*>(row + 4 * ch) = w;
      }
    } else {
      for (int e = lane; e < dim; e += G) {
        float x = g[e];
        float mm = o.beta1 * m[e] + c1 * x;
        float vv = o.beta2 * v[e] + c2 * x * x;
        m[e] = mm; v[e] = vv;
        row[e] -= o.lr * mm / (o.eps + sqrtf(vv));
      }
    }
    if (lane == 0) reinterpret_cast<int*>(row)[3 * dim + 1] += (int)bshow;
  } else {
    float* z = row + dim;
    float* n = row + 2 * dim;
    if (VEC) {
      // all four 16-byte loads of a chunk are issued before the arithmetic; approximate sqrt / division as in the
      // other two optimizers (three square roots and a division per element otherwise dominate the update)
      for (int ch = lane; ch < (dim >> 2); ch += G) {
        const float4 x = *reinterpret_cast<const float4*>(g + 4 * ch);
        float4 zz = *reinterpret_cast<float4*>(z + 4 * ch), nn = *reinterpret_cast<float4*>(n + 4 * ch);
        float4 w = *reinterpret_cast<float4*>(row + 4 * ch);
#define TN_SFTRL(cmp) { \
        const float g2 = x.cmp * x.cmp; \
        const float sn = fast_sqrt(nn.cmp + g2); \
        zz.cmp += x.cmp - o.lr * (sn - fast_sqrt(nn.cmp)) * w.cmp; \
        nn.cmp += g2; \
        const float shr = zz.cmp > 0.f ? zz.cmp - o.lambda1 : zz.cmp + o.lambda1; \
        w.cmp = fabsf(zz.cmp) > o.lambda1 ? -fast_div(shr, (o.ftrl_beta + sn) * o.lr + o.lambda2) : 0.f; }
        TN_SFTRL(x) TN_SFTRL(y) TN_SFTRL(z) TN_SFTRL(w)
#undef TN_SFTRL
        *reinterpret_cast<float4*>(z + 4 * ch) = zz;
        *reinterpret_cast<float4*>(n + 4 * ch) = nn;
        *reinterpret_cast<float4*>(row + 4 * ch) = w;
      }
    } else {
    for (int e = lane; e < dim; e += G) {
      float x = g[e], w = row[e], nn = n[e];
      float g2 = x * x;
      float zz = z[e] + x - o.lr * (sqrtf(nn + g2) - sqrtf(nn)) * w;
      nn += g2;
      float nw = 0.f;
      if (fabsf(zz) > o.lambda1) {
        nw = -1.f / ((o.ftrl_beta + sqrtf(nn)) * o.lr + o.lambda2);
        nw *= zz > 0.f ? zz - o.lambda1 : zz + o.lambda1;
      }
      z[e] = zz; n[e] = nn; row[e] = nw;
    }
    }
    if (lane == 0) reinterpret_cast<int*>(row)[3 * dim + 1] += (int)bshow;
  }
}

}  // namespace

// `dense_ctas` > 0: the last `dense_ctas` CTAs of the grid run the dense step `d` of the same training step (reduce-
// scatter of the flat gradient, optimizer on the owned chunk, all-gather of the new weights) while the others push.
// Both exchanges wait on the same peers at the same point of the step, so side by side they cost one wait instead
// of two; the dense CTAs use the dense table's own barrier and flag words.
__global__ void __launch_bounds__(kThreads, 1) sparse_push_fused_kernel(const __grid_constant__ PushArgs a,
                                                                        const __grid_constant__ DenseStepArgs d,
                                                                        const int dense_ctas) {
  const int nb = (int)gridDim.x - dense_ctas;      // CTAs of the push proper
  if ((int)blockIdx.x >= nb) {
    dense::fused_step<kRiderUnroll>(d, (int)blockIdx.x - nb, dense_ctas);   // two loads in flight: fits the 64-register budget of 1024 threads
    return;
  }
  const SparseCommView& c = a.c;
  __shared__ TableView s_tbl;
  if (threadIdx.x == 0) s_tbl = a.tbl_dev != nullptr ? *a.tbl_dev : a.tbl;
  __syncthreads();
  const TableView& t = s_tbl;
  GridSync gs;
  gs.init(c.bar, c.status, c.wait_ns, (unsigned)nb);
  __shared__ unsigned long long s_flag;
  __shared__ int s_pre[kMaxWorld + 1];

  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  const int nth = nb * blockDim.x;
  const int W = c.world, R = c.rank, capo = c.capo;
  const unsigned long long epoch = __ldcg(c.epoch);
  const int dim = t.dim, gstride = c.gstride, gch = gstride >> 2;
  const int G = a.lanes;
  const int lane = threadIdx.x % G;
  const int gid = tid / G, ngroups = nth / G;
  const unsigned gmask = group_mask(G);
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool vec = (dim & 3) == 0;

  prof_mark(c, 8);
  if (W == 1) {
    // single GPU: every unique sign of the batch maps to exactly one row; update in place
    const int n = __ldcg(&c.cnt_saved[0]);
    for (int j = gid; j < n; j += ngroups) {
      int rr = __ldcg(&c.req_row[j]);
      if (j + ngroups < n) {
        const int r2 = __ldcg(&c.req_row[j + ngroups]);
        if (r2 != kReqNone && r2 != kReqPending) prefetch_row_l2(t.rows + (size_t)(r2 & kReqRowMask) * t.stride, t.stride, lane, G);
      }
      float* g = c.gU + (size_t)j * gstride;
      float* cn = c.cnts + 2 * (size_t)j;
      if (rr != kReqNone && rr != kReqPending) {
        float* row = t.rows + (size_t)(rr & kReqRowMask) * t.stride;
        const float bshow = cn[0], bclick = cn[1];
        if (vec) apply_row<true>(a.opt, row, g, bshow, bclick, dim, lane, G, gmask);
        else apply_row<false>(a.opt, row, g, bshow, bclick, dim, lane, G, gmask);
      }
      __syncwarp(gmask);
      for (int ch = lane; ch < gch; ch += G) *reinterpret_cast<float4*>(g + 4 * ch) = zero4;
      if (lane == 0) { cn[0] = 0.f; cn[1] = 0.f; }
    }
    goto done;
  }

  // ---- phase A: tell every owner that this GPU's gradient records are complete.  They are: the backward pass that
  // wrote them precedes this kernel in the stream.  The records stay where they are; each owner READS its segment of
  // every GPU's records over NVLink and sums as it reads.  (Shipping them into inboxes first cost a pass of peer
  // stores, a system-wide fence to drain it and a second pass to sum: 36 us of a 72 us push on eight GPUs.)
  if (blockIdx.x == 0 && threadIdx.x < W && threadIdx.x != R)
    st_release_sys_u64(sig_word(c.sig[threadIdx.x], kSigPushReq, R), epoch << 32);
  prof_mark(c, 9);
  prof_mark(c, 10);

  // ---- phase B: as owner, sum records of equal sign coming from different GPUs --------------------
  // own records first (nothing to wait for)
  {
    const int n_s = __ldcg(&c.req_n[R]);
    const float* src = c.gU + (size_t)R * capo * gstride;
    const int total = n_s * gch;
    for (int i = tid; i < total; i += nth) {
      const int j = i / gch, ch = i - j * gch;
      const int ou = __ldcg(&c.req_ou[R * capo + j]);
      if (ou < 0) continue;
      red_add_f32x4(c.acc + (size_t)ou * gstride + 4 * ch, ldcg_f4(src + 4 * (size_t)i));
    }
    const float2* csrc = reinterpret_cast<const float2*>(c.cnts) + (size_t)R * capo;
    for (int j = tid; j < n_s; j += nth) {
      const int ou = __ldcg(&c.req_ou[R * capo + j]);
      if (ou < 0) continue;
      const float2 sc = __ldcg(&csrc[j]);
      float* g = c.acc + (size_t)ou * gstride + dim;          // the record's show / click slots
      atomicAdd(g, sc.x);
      if (sc.y != 0.f) atomicAdd(g + 1, sc.y);
    }
  }
  prof_mark(c, 14);
  // then everybody else's, as one flat index space over the senders so that no thread idles on a short segment
  {
    __syncthreads();
    if (threadIdx.x < 32) {       // one lane per sender polls its flag; a warp scan lays the segments end to end
      const int k = threadIdx.x;
      const int sk = (R + 1 + k) % W;
      unsigned long long v;
      bool ok = true;
      if (k + 1 < W) ok = wait_flag_ge(sig_word(c.sig[R], kSigPushReq, sk), epoch, &v, c.wait_ns, c.status, 12, sk);
      const bool all_ok = __all_sync(0xffffffffu, ok);
      int incl = (k + 1 < W) ? __ldcg(&c.req_n[sk]) : 0;
#pragma unroll
      for (int o = 1; o < kMaxWorld; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (k >= o) incl += up;
      }
      if (k + 1 < W) s_pre[k + 1] = incl;
      if (k == 0) { s_pre[0] = 0; s_flag = all_ok ? 0ull : ~0ull; }
    }
    __syncthreads();
    prof_mark(c, 15);
    if (s_flag == ~0ull) { gs.failed = true; }
    else {
      const int n_all = s_pre[W - 1];
      const int total = n_all * gch;
      for (int i = tid; i < total; i += nth) {
        const int jj = i / gch, ch = i - jj * gch;
        int k = 0;
        while (jj >= s_pre[k + 1]) ++k;
        const int sk = (R + 1 + k) % W, j = jj - s_pre[k];
        const int ou = __ldcg(&c.req_ou[sk * capo + j]);
        if (ou < 0) continue;
        // sender sk keeps the records it owes this GPU in segment R of its gradient matrix
        const float4 v = ldcg_f4(c.gU_peer[sk] + ((size_t)R * capo + j) * gstride + 4 * ch);
        red_add_f32x4(c.acc + (size_t)ou * gstride + 4 * ch, v);
      }
      for (int jj = tid; jj < n_all; jj += nth) {
        int k = 0;
        while (jj >= s_pre[k + 1]) ++k;
        const int sk = (R + 1 + k) % W, j = jj - s_pre[k];
        const int ou = __ldcg(&c.req_ou[sk * capo + j]);
        if (ou < 0) continue;
        const float2 sc = __ldcg(reinterpret_cast<const float2*>(c.cnts_peer[sk]) + (size_t)R * capo + j);
        float* g = c.acc + (size_t)ou * gstride + dim;
        atomicAdd(g, sc.x);
        if (sc.y != 0.f) atomicAdd(g + 1, sc.y);
      }
    }
  }
  if (gs.failed) goto done;
  prof_mark(c, 11);
  // every value read from a peer has been consumed once all CTAs are here: the senders may clear their records
  if (last_cta_arrives(&c.bar[2], false, (unsigned)nb) && threadIdx.x < W && threadIdx.x != R)
    st_release_sys_u64(sig_word(c.sig[threadIdx.x], kSigPushDone, R), epoch << 32);
  if (!gs.sync(13, false)) goto done;
  prof_mark(c, 12);

  // ---- phase C: one optimizer update per touched row ----------------------------------------------
  {
    const int n_ou = __ldcg(c.ocount);
    for (int ou = gid; ou < n_ou; ou += ngroups) {
      const int r = __ldcg(&c.ou_row[ou]);
      if (ou + ngroups < n_ou) {
        const int r2 = __ldcg(&c.ou_row[ou + ngroups]);
        if (r2 >= 0) prefetch_row_l2(t.rows + (size_t)r2 * t.stride, t.stride, lane, G);
      }
      float* g = c.acc + (size_t)ou * gstride;
      if (r >= 0) {
        float* row = t.rows + (size_t)r * t.stride;
        const float bshow = g[dim], bclick = g[dim + 1];
        if (vec) apply_row<true>(a.opt, row, g, bshow, bclick, dim, lane, G, gmask);
        else apply_row<false>(a.opt, row, g, bshow, bclick, dim, lane, G, gmask);
      }
      __syncwarp(gmask);
      for (int ch = lane; ch < gch; ch += G) *reinterpret_cast<float4*>(g + 4 * ch) = zero4;
    }
  }
  prof_mark(c, 13);
  // every CTA is past its row updates: re-arm the owner-unique counter for a pull whose front ran ahead
  if (last_cta_arrives(&c.bar[3], false, (unsigned)nb) && threadIdx.x == 0) *c.ocount = 0;

  // ---- tail: once every owner has read this GPU's records, clear them for the next backward pass (the owners' reads
  // finished while this GPU updated its rows, so the wait is short)
  {
    __syncthreads();
    if (threadIdx.x < 32) {
      const int p = threadIdx.x;
      unsigned long long v;
      bool ok = true;
      if (p < W && p != R) ok = wait_flag_ge(sig_word(c.sig[R], kSigPushDone, p), epoch, &v, c.wait_ns, c.status, 16, p);
      const bool all_ok = __all_sync(0xffffffffu, ok);
      if (threadIdx.x == 0) s_flag = all_ok ? 0ull : ~0ull;
    }
    __syncthreads();
    if (s_flag == ~0ull) { gs.failed = true; goto done; }
    for (int p = 0; p < W; ++p) {
      const int n = __ldcg(&c.cnt_saved[p]);
      float4* g4 = reinterpret_cast<float4*>(c.gU + (size_t)p * capo * gstride);
      const int total = n * gch;
      for (int i = tid; i < total; i += nth) g4[i] = zero4;
      float2* c2 = reinterpret_cast<float2*>(c.cnts) + (size_t)p * capo;
      for (int j = tid; j < n; j += nth) c2[j] = make_float2(0.f, 0.f);
    }
  }

done:
  gs.leave();
}

// =======================================================================================
// host launchers
// =======================================================================================
static int coop_grid(const void* fn, int device) {
  int per_sm = 0, sms = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kThreads, 0);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 1) per_sm = 1;
  return per_sm * sms;
}

cudaError_t launch_sparse_pull(const PullArgs& args, int work_items, cudaStream_t stream) {
  int dev = 0;
  cudaGetDevice(&dev);
  const bool tiled = args.tile_rows > 0;
  const void* fn = tiled ? (const void*)sparse_pull_fused_kernel<true> : (const void*)sparse_pull_fused_kernel<false>;
  static int grid_max[64][2] = {{0}};
  if (grid_max[dev][tiled] == 0) grid_max[dev][tiled] = coop_grid(fn, dev);
  int grid = (work_items + kThreads - 1) / kThreads;
  if (grid < 1) grid = 1;
  if (grid > grid_max[dev][tiled]) grid = grid_max[dev][tiled];
  const size_t smem = (size_t)args.tile_rows * args.c.ustride * sizeof(float) * (kThreads / 32);
  static bool attr_set[64] = {false};
  // static + dynamic shared memory beyond 48 KiB needs the opt-in; a 48 KiB tile buffer alone already crosses it
  if (smem > 32 * 1024 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  void* params[] = {(void*)&args};
  return cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kThreads), params, smem, stream);
}

cudaError_t launch_sparse_pull_front(const PullArgs& args, cudaStream_t stream) {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = (args.n_ids + kFrontThreads - 1) / kFrontThreads;
  if (grid < 1) grid = 1;
  if (grid > 4 * sms) grid = 4 * sms;
  pull_front_dedup_kernel<<<grid, kFrontThreads, 0, stream>>>(args);
  pull_front_ship_kernel<<<grid, kFrontThreads, 0, stream>>>(args);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // the inverse map is complete: the dedup scratch goes back to all-empty (kEmptyKey is all ones)
  return cudaMemsetAsync(args.c.dd_keys, 0xFF, ((size_t)args.c.dd_mask + 1u) * sizeof(unsigned long long), stream);
}

// `max_ctas` > 0 caps the grid below the SM count, leaving whole SMs to a kernel running on another stream.
// `dense` != null (several GPUs only): the dense step rides on `dense_ctas` extra CTAs of the same cooperative grid.
cudaError_t launch_sparse_push(const PushArgs& args, int work_items, int max_ctas, const DenseStepArgs* dense, cudaStream_t stream) {
  int dev = 0;
  cudaGetDevice(&dev);
  static int grid_max[64] = {0};
  if (grid_max[dev] == 0) grid_max[dev] = coop_grid((const void*)sparse_push_fused_kernel, dev);
  int grid = (work_items + kThreads - 1) / kThreads;
  if (grid < 1) grid = 1;
  int dense_ctas = 0;
  DenseStepArgs d{};
  if (dense != nullptr) {
    if (dense->world < 2 || dense->n % 4 || dense->chunk % 4) return cudaErrorInvalidValue;
    d = *dense;
    // one pass of the owned chunk: 1024 threads x kDenseUnroll 16-byte groups per CTA, at most 16 CTAs
    const long long per_cta = (long long)kThreads * kRiderUnroll * 4;
    dense_ctas = (int)((d.chunk + per_cta - 1) / per_cta);
    if (dense_ctas < 1) dense_ctas = 1;
    if (dense_ctas > 16) dense_ctas = 16;
  }
  const int room = grid_max[dev] - dense_ctas;
  if (grid > room) grid = room;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid < 1) return cudaErrorInvalidValue;
  grid += dense_ctas;
  void* params[] = {(void*)&args, (void*)&d, (void*)&dense_ctas};
  return cudaLaunchCooperativeKernel((const void*)sparse_push_fused_kernel, dim3(grid), dim3(kThreads), params, 0, stream);
}

}  // namespace tn
