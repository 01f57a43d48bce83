"""Runtime knobs of the framework, overridable by ``TN_*`` environment variables.

The reference has no flag system: its sizes are compile-time constants
(core/ps/optimizer/optimizer_kernel.h:42-43,257-266, core/ps/ps_cluster.cc:78-79).
Here they are one dataclass so a job can size the GPU tables for its data.
"""
from __future__ import annotations

import dataclasses
import os


def _env(name: str, default, cast):
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    if cast is bool:
        return v.lower() not in ("0", "false", "no", "off")
    return cast(v)


@dataclasses.dataclass
class Config:
    #: rows each GPU's shard of a sparse table can hold (row slab capacity)
    table_rows_per_gpu: int = 1 << 22
    #: key-array load factor target; the key array is the next power of two >= rows / load_factor
    table_load_factor: float = 0.5
    #: head-room factor of one (sender, owner) segment over the even split unique/world
    owner_segment_slack: float = 1.3
    #: several GPUs: an exchange segment holds a whole batch (any spread of signs over the owners is accepted) as long
    #: as one layer's exchange buffers stay below this many MiB per GPU; beyond it segments are sized by the slack above
    segment_worst_case_mb: int = 1024
    #: enlarge a shard (row slab x2, key array re-filled) when a status poll finds it this full; 0 = never
    table_grow_at: float = 0.85
    #: wall-time budget of every device-side wait, in seconds
    wait_budget_s: float = 5.0
    #: seed of the deterministic row initialiser
    seed: int = 0x7E50A
    #: NVSwitch multicast (multimem) in the dense path when the mapping exists: 1 = always, 0 = never, -1 = from 4 GPUs up
    #: (two GPUs, 130 M parameters: 1 065 us with plain peer loads / stores against 1 778 us through the switch)
    use_multimem: int = -1
    gate_first_gemm: bool = True   # multi-GPU: first MLP GEMM waits for the dense all-gather (no closing barrier)
    #: pull returns rows through shared-memory tiles: -1 = only with several GPUs, 0 = never, 1 = always
    staged_row_return: int = -1
    #: multi-GPU: run the dense step beside the sparse push on a second stream, each on its own share of the SMs.
    #: -1 = only for dense arrays above 4 M elements (smaller ones ride on the push kernel, see below; measured at
    #: 2 GPUs on the DeepFM step, side by side was 2 % slower than back to back), 0 = never, 1 = always
    overlap_dense_push: int = -1
    overlap_dense_sms: int = 40    # SMs the push leaves to a large dense step
    nvtx_phases: bool = False      # NVTX ranges around the phases of an eager training step
    #: replayed steps stage their inputs and read their loss back through one native call each instead of Python-level
    #: stream / event / copy calls
    native_step_path: bool = True
    #: when the caller names the batch of the following step (`fit` does), its dedup and id dispatch run on a second
    #: stream under the current step's forward / backward, and the pull of that step only probes and returns rows.
    #: -1 = on one GPU only; 1 = also on several GPUs, where the caller then guarantees that all ranks change batch
    #: shape (a shorter last batch) at the same step: a rank cannot leave the two-step pull protocol alone; 0 = never
    pull_front_ahead: int = -1
    #: several GPUs: bind each process to the CPU cores closest to its GPU (NVML's affinity mask) before it allocates
    #: page-locked buffers
    bind_cpu_affinity: bool = True
    #: multi-GPU, dense arrays up to 4 M elements: the dense step runs on a few CTAs of the last sparse push kernel of
    #: the step instead of in a kernel of its own behind it
    dense_rides_push: bool = True
    #: multi-GPU: cap on the dense kernel's grid for small arrays (cheaper grid barriers); 0 = fill the GPU
    dense_small_grid: int = 0
    #: rows per streamed piece when a GPU shard is saved (bounds the pinned host staging buffer)
    checkpoint_chunk_rows: int = 1 << 22
    #: rows per piece when a shard is read back (eight block files are read side by side, each one piece at a time)
    checkpoint_load_chunk_rows: int = 1 << 18
    #: check the guard words behind the shared-memory regions after every training pass as well (they are always
    #: checked before a checkpoint is written and when a step-log window closes); costs a few small kernels and a sync
    verify_guards_each_pass: bool = False
    #: run MLP towers that fit as one kernel per direction (activations stay in shared memory between the layers).
    #: Off by default: with one 128-row stripe per CTA only 64 of the 148 SMs work on a batch of 8192 and the weight
    #: ring holds two tiles, so the DeepFM step measures 0.277 ms with it against 0.258 ms layer by layer.
    fused_mlp: bool = False
    #: capture the train step in a CUDA graph
    cuda_graph: bool = True
    #: training looks at the device status words every this many steps (asynchronously, no stall)
    status_poll_steps: int = 16
    #: force the CPU oracle path even when a GPU is visible
    force_cpu: bool = False

    @classmethod
    def from_env(cls) -> "Config":
        c = cls()
        c.table_rows_per_gpu = _env("TN_TABLE_ROWS", c.table_rows_per_gpu, int)
        c.table_load_factor = _env("TN_TABLE_LOAD_FACTOR", c.table_load_factor, float)
        c.owner_segment_slack = _env("TN_SEGMENT_SLACK", c.owner_segment_slack, float)
        c.segment_worst_case_mb = _env("TN_SEGMENT_WORST_CASE_MB", c.segment_worst_case_mb, int)
        c.table_grow_at = _env("TN_TABLE_GROW_AT", c.table_grow_at, float)
        c.wait_budget_s = _env("TN_WAIT_BUDGET_S", c.wait_budget_s, float)
        c.seed = _env("TN_SEED", c.seed, int)
        c.use_multimem = _env("TN_USE_MULTIMEM", c.use_multimem, int)
        c.gate_first_gemm = _env("TN_GATE_FIRST_GEMM", c.gate_first_gemm, bool)
        c.staged_row_return = _env("TN_STAGED_RETURN", c.staged_row_return, int)
        c.dense_small_grid = _env("TN_DENSE_SMALL_GRID", c.dense_small_grid, int)
        c.overlap_dense_push = _env("TN_OVERLAP_DENSE_PUSH", c.overlap_dense_push, int)
        c.overlap_dense_sms = _env("TN_OVERLAP_DENSE_SMS", c.overlap_dense_sms, int)
        c.nvtx_phases = _env("TN_NVTX_PHASES", c.nvtx_phases, bool)
        c.native_step_path = _env("TN_NATIVE_STEP_PATH", c.native_step_path, bool)
        c.pull_front_ahead = _env("TN_PULL_FRONT_AHEAD", c.pull_front_ahead, int)
        c.bind_cpu_affinity = _env("TN_BIND_CPU_AFFINITY", c.bind_cpu_affinity, bool)
        c.dense_rides_push = _env("TN_DENSE_RIDES_PUSH", c.dense_rides_push, bool)
        c.checkpoint_chunk_rows = _env("TN_CKPT_CHUNK_ROWS", c.checkpoint_chunk_rows, int)
        c.checkpoint_load_chunk_rows = _env("TN_CKPT_LOAD_CHUNK_ROWS", c.checkpoint_load_chunk_rows, int)
        c.verify_guards_each_pass = _env("TN_VERIFY_GUARDS", c.verify_guards_each_pass, bool)
        c.fused_mlp = _env("TN_FUSED_MLP", c.fused_mlp, bool)
        c.cuda_graph = _env("TN_CUDA_GRAPH", c.cuda_graph, bool)
        c.status_poll_steps = _env("TN_STATUS_POLL_STEPS", c.status_poll_steps, int)
        c.force_cpu = _env("TN_FORCE_CPU", c.force_cpu, bool)
        return c


config = Config.from_env()
