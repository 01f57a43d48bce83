"""The allocation-free dedup entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory at call time (a serving process whose
memory is fully handed out at start-up, a thread running next to a CUDA-graph capture, a plug-in
inside a framework that owns the allocator).  For them ``tn_unique_assign_static`` keeps its
scratch in a fixed array inside the library.  This test loads the shared object with ctypes,
calls the symbol twice in a row on caller-owned buffers and checks the results against the
ordinary (allocating) ``unique_assign`` entry point.  Virtual indices depend on which thread wins
an insert race, so the two outputs are compared after ordering the distinct signs.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from tensornet_b200 import _build

    _build.cuda_ext()
    lib = ctypes.CDLL(_build._so_path("_tn_cuda"))
    lib.tn_unique_assign_static.restype = ctypes.c_int
    lib.tn_unique_assign_static.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.tn_unique_assign_static_error.restype = ctypes.c_char_p
    lib.tn_unique_assign_static_status.restype = ctypes.c_int
    lib.tn_unique_assign_static_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    return lib


def _canon(uniq, inverse, show, click, n):
    u = uniq[:n].cpu().numpy().view(np.uint64)
    order = np.argsort(u)
    rank = np.empty(n, dtype=np.int64)
    rank[order] = np.arange(n)
    return u[order], rank[inverse.cpu().numpy()], show[:n].cpu().numpy()[order], click[:n].cpu().numpy()[order]


def test_static_entry_point_matches_allocating_one(tn_gpu):
    from tensornet_b200.ops.unique import UniqueAssign

    lib = _lib()
    dev = tn_gpu.core.runtime().device
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ua = UniqueAssign(65536)
    g = torch.Generator().manual_seed(11)
    for call in range(2):                      # two calls in a row share the built-in scratch
        n = 50000 - 7000 * call
        ids = (torch.randint(0, 9000 + 500 * call, (n,), generator=g, dtype=torch.int64) * 2862933555777941757 + 3037000493).to(dev)
        labels = (torch.rand(n, generator=g) < 0.25).float().to(dev)
        cap = 65536
        uniq = torch.empty(cap, dtype=torch.int64, device=dev)
        inverse = torch.empty(n, dtype=torch.int32, device=dev)
        show = torch.full((cap,), 7.0, device=dev)     # dirty on purpose: the entry point must clear what it uses
        click = torch.full((cap,), 7.0, device=dev)
        count = torch.full((1,), 123, dtype=torch.int32, device=dev)
        rc = lib.tn_unique_assign_static(ids.data_ptr(), n, labels.data_ptr(), uniq.data_ptr(), cap, inverse.data_ptr(),
                                         show.data_ptr(), click.data_ptr(), count.data_ptr(), stream)
        assert rc == 0, lib.tn_unique_assign_static_error()
        st = (ctypes.c_int * 4)()
        assert lib.tn_unique_assign_static_status(st, stream) == 0 and st[0] == 0
        u2, inv2, show2, click2, count2 = ua(ids, labels)
        torch.cuda.synchronize()
        k = int(count.item())
        assert k == int(count2.item())
        a = _canon(uniq, inverse, show, click, k)
        b = _canon(u2, inv2, show2, click2, k)
        for x, y in zip(a, b):
            assert np.array_equal(x, y)
        assert np.array_equal(a[0][a[1]], ids.cpu().numpy().view(np.uint64))
    tn_gpu.core.runtime().check_status()


def test_static_entry_point_rejects_oversize(tn_gpu):
    lib = _lib()
    dev = tn_gpu.core.runtime().device
    count = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.tn_unique_assign_static(None, 65537, None, None, 0, None, None, None, count.data_ptr(), None)
    assert rc == 1
    assert b"exceed" in lib.tn_unique_assign_static_error()
