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
from typing import List, Optional

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


class SymmArena:
    """Carves named, 256-byte aligned regions out of one SymmBuffer."""

    def __init__(self, layout):
        # layout: list of (name, shape, dtype)
        self.offsets = {}
        self.meta = {}
        off = 0
        for name, shape, dtype in layout:
            n = 1
            for s in shape:
                n *= int(s)
            nb = n * torch.empty((), dtype=dtype).element_size()
            self.offsets[name] = off
            self.meta[name] = (tuple(int(s) for s in shape), dtype)
            off += (nb + 255) // 256 * 256
        self.buf = SymmBuffer(max(off, 256))

    def tensor(self, name: str) -> torch.Tensor:
        shape, dtype = self.meta[name]
        return self.buf.view(self.offsets[name], shape, dtype)

    def ptrs(self, name: str) -> List[int]:
        return self.buf.peer_ptrs(self.offsets[name])

    def mc(self, name: str) -> int:
        return self.buf.mc(self.offsets[name])
