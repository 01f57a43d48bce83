"""SM-issued peer copy bandwidth: what plain loads / stores from inside a kernel reach between
this GPU and a peer over NVLink (and, for comparison, inside this GPU's own memory).

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/p2p_microbench.py

These figures are the link-side denominators of the fused sparse pull / push and dense-step
rooflines.  Rank 0 prints one JSON line per (direction, size, launch shape)."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensornet_b200 as tn  # noqa: E402
from tensornet_b200 import _build  # noqa: E402
from tensornet_b200.parallel.symm import SymmBuffer  # noqa: E402


def load_probe():
    """Compile (once, next to this file) and import the probe kernel."""
    from torch.utils import cpp_extension

    here = os.path.dirname(os.path.abspath(__file__))
    out = os.path.join(here, "_ext", "peer_probe")
    os.makedirs(out, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    return cpp_extension.load(name="tn_peer_probe", sources=[os.path.join(here, "peer_probe.cu")], build_directory=out,
                              extra_cuda_cflags=_build.NVCC_FLAGS, with_cuda=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", type=float, nargs="+", default=[0.5, 4, 32, 256])
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    tn.core.init()
    rt = tn.core.runtime()
    ext = load_probe()
    big = int(max(args.sizes_mb) * (1 << 20))
    buf = SymmBuffer(big)
    local = torch.ones(big, dtype=torch.uint8, device=rt.device)
    peer = (rt.rank + 1) % rt.world
    rows = []
    cases = [("store_to_peer", buf.ptrs[peer], local.data_ptr()), ("load_from_peer", local.data_ptr(), buf.ptrs[peer]),
             ("local", buf.ptrs[rt.rank], local.data_ptr())]
    shapes = [(148, 1024, 0), (148, 1024, 1), (296, 512, 1), (148, 256, 1), (32, 1024, 1), (148, 1024, 2), (148, 1024, 3)]
    for name, dst, src in cases:
        if rt.world == 1 and name != "local":
            continue
        for mb in args.sizes_mb:
            nbytes = int(mb * (1 << 20)) // 16 * 16
            for blocks, threads, mode in shapes:
                if mode >= 2 and name == "load_from_peer":
                    continue
                for _ in range(3):
                    ext.peer_copy(dst, src, nbytes, mode, blocks, threads, True)
                rt.barrier()
                torch.cuda.synchronize()
                evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.iters)]
                for e0, e1 in evs:
                    e0.record()
                    ext.peer_copy(dst, src, nbytes, mode, blocks, threads, True)
                    e1.record()
                torch.cuda.synchronize()
                us = sorted(e0.elapsed_time(e1) * 1e3 for e0, e1 in evs)[len(evs) // 2]
                t = torch.tensor([us], device=rt.device)
                if rt.world > 1:
                    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=rt.device_group)
                rows.append(dict(case=name, mb=mb, blocks=blocks, threads=threads, mode=mode, us=round(float(t), 2),
                                 gbs=round(nbytes / float(t) / 1e3, 1)))
    rt.barrier()
    if rt.rank == 0:
        for r in rows:
            print(json.dumps(r))
    tn.core.shutdown()


if __name__ == "__main__":
    main()
