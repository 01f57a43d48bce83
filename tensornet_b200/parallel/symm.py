"""Symmetric device memory: the same buffer on every GPU of the job, each mapped into every
peer's address space so kernels can issue plain loads/stores (or NVSwitch ``multimem``
operations) on it.

Allocation and handle exchange ride on ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations exchanged over the process group).  Only the plumbing is borrowed: every byte
that crosses NVLink is moved by this library's own kernels.  With one GPU the "symmetric"
buffer is an ordinary tensor and the peer table has a single entry.
"""
from __future__ import annotations

import os
import weakref
from typing import List

import torch

from ..core.runtime import runtime


class SymmBuffer:
    """A byte buffer present on every rank.  ``ptrs[p]`` is rank p's copy as seen from here."""

    def __init__(self, nbytes: int, zero: bool = True):
        rt = runtime()
        nbytes = (int(nbytes) + 255) // 256 * 256
        self.nbytes = nbytes
        self.mc_ptr = 0
        self._hdl = None
        if rt.world == 1 or not rt.on_gpu:
            self.local = torch.empty(nbytes, dtype=torch.uint8, device=rt.device)
            if zero:
                self.local.zero_()
            self.ptrs: List[int] = [self.local.data_ptr()]
        elif os.environ.get("TN_SYMM_BACKEND", "torch") == "ipc":
            # CUDA IPC: every rank cudaMallocs its copy, the handles travel over the host group and
            # each peer maps them.  No NVSwitch multicast mapping in this mode.
            from .. import _build

            ext = _build.cuda_ext()
            ptr, handle = ext.ipc_alloc(nbytes)
            self._ipc_own = ptr
            handles = rt.all_gather_object(handle)
            self.ptrs = [ptr if r == rt.rank else int(ext.ipc_open(h)) for r, h in enumerate(handles)]
            self.local = ext.tensor_from_ptr(ptr, nbytes, rt.device.index)
            torch.cuda.synchronize()
            rt.barrier()
        else:
            import torch.distributed._symmetric_memory as symm_mem

            self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=rt.device)
            if zero:
                self.local.zero_()
            torch.cuda.synchronize()
            self._hdl = symm_mem.rendezvous(self.local, rt.device_group.group_name)
            self.ptrs = [int(p) for p in self._hdl.buffer_ptrs]
            try:
                self.mc_ptr = int(self._hdl.multicast_ptr or 0)
            except Exception:  # pragma: no cover - depends on driver support
                self.mc_ptr = 0
            rt.barrier()

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nb = n * torch.empty((), dtype=dtype).element_size()
        return self.local[offset:offset + nb].view(dtype).view(*shape)

    def peer_ptrs(self, offset: int) -> List[int]:
        return [p + offset for p in self.ptrs]

    def mc(self, offset: int) -> int:
        return self.mc_ptr + offset if self.mc_ptr else 0


_GUARD_BYTES = 256
_GUARD_PATTERN = 0xA5
_arenas = weakref.WeakSet()


class SymmArena:
    """Carves named, 256-byte aligned regions out of one SymmBuffer.

    Every region is followed by a 256-byte guard filled with a fixed pattern.  Peers write into these regions at
    offsets their kernels compute, so an offset bug on any GPU shows up as a damaged guard on the GPU that owns
    the memory; ``verify`` (and ``verify_all_arenas``, called before a checkpoint is written, when a step-log window
    closes and, with ``config.verify_guards_each_pass``, after every training pass) reads the guards back and
    names the region in front of the damaged one."""

    def __init__(self, layout):
        # layout: list of (name, shape, dtype)
        self.offsets = {}
        self.meta = {}
        self.guards = {}
        off = 0
        for name, shape, dtype in layout:
            n = 1
            for s in shape:
                n *= int(s)
            nb = n * torch.empty((), dtype=dtype).element_size()
            self.offsets[name] = off
            self.meta[name] = (tuple(int(s) for s in shape), dtype)
            off += (nb + 255) // 256 * 256
            self.guards[name] = off
            off += _GUARD_BYTES
        self.buf = SymmBuffer(max(off, 256))
        if self.guards:
            g = self.buf.local[: off].view(-1, _GUARD_BYTES)
            idx = torch.tensor([o // _GUARD_BYTES for o in self.guards.values()], device=g.device)
            g[idx] = _GUARD_PATTERN
            self._guard_idx = idx
            self._guard_rows = g
            if runtime().on_gpu:
                torch.cuda.synchronize()
            if runtime().world > 1:
                runtime().barrier()       # no peer may start writing before every guard is in place
        _arenas.add(self)

    def tensor(self, name: str) -> torch.Tensor:
        shape, dtype = self.meta[name]
        return self.buf.view(self.offsets[name], shape, dtype)

    def ptrs(self, name: str) -> List[int]:
        return self.buf.peer_ptrs(self.offsets[name])

    def mc(self, name: str) -> int:
        return self.buf.mc(self.offsets[name])

    def damaged(self) -> List[str]:
        """Names of the regions whose trailing guard no longer holds the pattern (one small device read)."""
        if not self.guards:
            return []
        g = self._guard_rows[self._guard_idx]
        if bool((g == _GUARD_PATTERN).all()):          # the common case: one gather, one reduction, one read-back
            return []
        bad = (g != _GUARD_PATTERN).any(dim=1).cpu().tolist()
        return [name for name, b in zip(self.guards, bad) if b]

    def verify(self):
        bad = self.damaged()
        if bad:
            raise RuntimeError("symmetric memory was written out of bounds: the guard behind region(s) "
                               + ", ".join(repr(b) for b in bad) + f" on rank {runtime().rank} is damaged")


def verify_all_arenas():
    """Check the guards of every live arena of this process."""
    for a in list(_arenas):
        a.verify()
