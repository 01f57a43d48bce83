"""Process-wide runtime: device binding, process groups, status words.

Replaces the reference's PsCluster / MpiManager bootstrap
(core/ps/ps_cluster.cc:33-67, core/utility/mpi_manager.cc:46-97): one process per GPU
started by ``torchrun``; ``torch.distributed`` carries the control plane (gloo for host
barriers and object exchange, NCCL for symmetric-memory rendezvous and the baseline
collectives); the data plane is peer memory written by this library's own kernels.
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist

from .config import config

STATUS_NAMES = {
    0: "ok",
    1: "per-batch dedup scratch overflow",
    2: "owner segment overflow (raise bucket_size or TN_SEGMENT_SLACK)",
    3: "sparse table full (raise TN_TABLE_ROWS)",
    4: "grid barrier timed out",
    5: "wait on a peer GPU timed out",
    6: "tensor-core pipeline wait timed out",
    7: "sign missing from the table",
    8: "bad argument",
}


class DeviceError(RuntimeError):
    """A kernel recorded an error in the status words."""

    def __init__(self, code: int, phase: int, aux: int):
        self.code, self.phase, self.aux = code, phase, aux
        super().__init__(f"device status {code} ({STATUS_NAMES.get(code, '?')}), phase {phase}, peer/aux {aux}")


def _bind_cpus_near(device_index: int) -> None:
    """Keep this process on the CPU cores the driver names as closest to its GPU (the same socket), before it
    allocates page-locked memory: with one process per GPU and no binding, the input batches of half the GPUs of a
    two-socket machine cross the socket interconnect on their way to the device.  Changes only this process's CPU
    affinity; does nothing when the information is not available or the allowed set would become empty."""
    try:
        import pynvml

        pynvml.nvmlInit()
        try:          # CUDA_VISIBLE_DEVICES renumbers the devices; the UUID names the same GPU to NVML
            uuid = "GPU-" + str(torch.cuda.get_device_properties(int(device_index)).uuid)
            h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if hasattr(pynvml, "c_nvmlDevice_t") else uuid)
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(int(device_index))
        n_cpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (n_cpu + 63) // 64)
        near = {64 * w + b for w, bits in enumerate(words) for b in range(64) if (int(bits) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        keep = near & allowed
        if keep and keep != allowed:
            os.sched_setaffinity(0, keep)
    except Exception:
        pass


class Runtime:
    def __init__(self):
        self.initialized = False
        self.rank = 0
        self.world = 1
        self.local_rank = 0
        self.device = torch.device("cpu")
        self.on_gpu = False
        self.host_group = None      # gloo group: barriers, object exchange
        self.peer_synced_pushes = 0  # multi-GPU sparse pushes launched so far (each one waits for all peers)
        self.device_group = None    # nccl group: symmetric memory rendezvous, baseline collectives
        self._status = None
        self._owns_pg = False
        self.failed = False          # a device error was raised and recover() has not run since

    # ------------------------------------------------------------------
    def init(self) -> bool:
        if self.initialized:
            return True
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", str(self.rank)))
        self.on_gpu = torch.cuda.is_available() and not config.force_cpu
        if self.on_gpu:
            self.device = torch.device("cuda", self.local_rank % torch.cuda.device_count())
            torch.cuda.set_device(self.device)
            if self.world > 1 and config.bind_cpu_affinity:
                _bind_cpus_near(self.device.index)
        else:
            self.device = torch.device("cpu")
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29511")
            timeout = datetime.timedelta(seconds=int(os.environ.get("TN_PG_TIMEOUT_S", "600")))
            if not dist.is_initialized():
                backend = "nccl" if self.on_gpu else "gloo"
                kwargs = {}
                if self.on_gpu:
                    kwargs["device_id"] = self.device
                dist.init_process_group(backend, rank=self.rank, world_size=self.world, timeout=timeout, **kwargs)
                self._owns_pg = True
            if self.on_gpu:
                self.device_group = dist.group.WORLD
                self.host_group = dist.new_group(backend="gloo", timeout=timeout)
            else:
                self.host_group = dist.group.WORLD
        if self.on_gpu:
            self._status = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.initialized = True
        return True

    def shutdown(self):
        if self._owns_pg and dist.is_initialized():
            dist.destroy_process_group()
        self.__init__()

    # ------------------------------------------------------------------
    @property
    def status(self) -> torch.Tensor:
        if self._status is None:
            self._status = torch.zeros(8, dtype=torch.int32, device=self.device)
        return self._status

    def check_status(self):
        """Raise DeviceError if any kernel reported a problem (synchronises the stream)."""
        if not self.on_gpu:
            return
        s = self.status.tolist()
        if s[0] != 0:
            self.raise_status(s[0], s[1], s[2])

    def raise_status(self, code: int, phase: int, aux: int):
        """A kernel reported ``code``.  Until :func:`tensornet_b200.core.recover` has run, every fused kernel skips
        its work (they all test the status word first), so nothing is half-applied behind the error; the runtime is
        marked failed and says so in the exception."""
        self.failed = True
        raise DeviceError(code, phase, aux)

    @property
    def wait_ns(self) -> int:
        return int(config.wait_budget_s * 1e9)

    def barrier(self):
        if self.world > 1:
            if self.on_gpu:
                torch.cuda.synchronize()
            dist.barrier(group=self.host_group)

    def all_gather_object(self, obj):
        if self.world == 1:
            return [obj]
        out = [None] * self.world
        dist.all_gather_object(out, obj, group=self.host_group)
        return out

    def exchange_counts(self, counts) -> "torch.Tensor":
        """``out[src][dst]`` = what rank ``src`` passed as ``counts[dst]`` (one small tensor all-gather on the host group)."""
        mine = torch.as_tensor(counts, dtype=torch.int64).reshape(-1)
        if self.world == 1:
            return mine.reshape(1, -1)
        out = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(out, mine, group=self.host_group)
        return torch.stack(out)

    def exchange_bytes(self, send, recv_sizes):
        """All-to-all of raw host buffers on the host group: ``send[d]`` (uint8 tensor) goes to rank ``d`` and the
        result's entry ``s`` (``recv_sizes[s]`` bytes) came from rank ``s``.  Point-to-point messages, no pickling:
        this is the CPU path's stand-in for the reference's raw-attachment RPCs (core/ps_interface/ps_raw_interface.h)."""
        recv = [torch.empty(int(n), dtype=torch.uint8) for n in recv_sizes]
        recv[self.rank] = send[self.rank]
        if self.world > 1:
            ops = []
            for k in range(1, self.world):
                dst, src = (self.rank + k) % self.world, (self.rank - k) % self.world
                if send[dst].numel():
                    ops.append(dist.P2POp(dist.isend, send[dst].contiguous(), dst, group=self.host_group))
                if recv[src].numel():
                    ops.append(dist.P2POp(dist.irecv, recv[src], src, group=self.host_group))
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
        return recv

    def exchange_bytes_many(self, exchanges):
        """Several :meth:`exchange_bytes` at once: ``exchanges`` is a list of ``(send, recv_sizes)``; all messages are
        posted together and waited for together, so N independent all-to-alls cost one round trip instead of N.
        Messages between one pair of ranks are matched in posting order, which is the same on every rank."""
        recvs = []
        for send, recv_sizes in exchanges:
            recv = [torch.empty(int(n), dtype=torch.uint8) for n in recv_sizes]
            recv[self.rank] = send[self.rank]
            recvs.append(recv)
        if self.world > 1:
            ops = []
            for (send, _), recv in zip(exchanges, recvs):
                for k in range(1, self.world):
                    dst, src = (self.rank + k) % self.world, (self.rank - k) % self.world
                    if send[dst].numel():
                        ops.append(dist.P2POp(dist.isend, send[dst].contiguous(), dst, group=self.host_group))
                    if recv[src].numel():
                        ops.append(dist.P2POp(dist.irecv, recv[src], src, group=self.host_group))
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()
        return recvs

    def broadcast_object(self, obj, src: int = 0):
        if self.world == 1:
            return obj
        lst = [obj]
        dist.broadcast_object_list(lst, src=src, group=self.host_group)
        return lst[0]


_RT = Runtime()


def runtime() -> Runtime:
    if not _RT.initialized:
        _RT.init()
    return _RT
