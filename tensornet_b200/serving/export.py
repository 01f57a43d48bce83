"""Dense tower of a trained model as one flat file for serving programs that do not run Python.

The reference exports its dense sub-graph as a TensorFlow SavedModel and compiles it ahead of time for its C++ demo
(doc/tutorial/04-deploy-tf-graph-online.ipynb, examples/online_serving/main.cc).  Here a tower is a chain of dense
layers, so the file is just their matrices: ``TNTW0001`` | u32 layers | per layer: u32 out, u32 in, u32 relu,
float32 ``W[out][in]``, float32 ``b[out]``.  ``examples/native_serving/serve.cpp`` reads it.
"""
from __future__ import annotations

import struct

import numpy as np
import torch


@torch.no_grad()
def export_tower(mlp, head, path: str) -> int:
    """Write ``mlp`` (:class:`tensornet_b200.layers.MLP`) followed by ``head`` (:class:`DenseHead`) to ``path``;
    returns the number of layers written."""
    layers = []
    n = len(mlp.hidden_units)
    for i in range(n):
        relu = 1 if (i < n - 1 or mlp.relu_last) else 0
        layers.append((mlp.weight(i).detach().float().cpu().numpy(), mlp.bias(i).detach().float().cpu().numpy(), relu))
    hw = head.weight.detach().float().cpu().numpy()
    layers.append((hw[None, : head.in_dim], hw[head.in_dim:head.in_dim + 1], 0))
    with open(path, "wb") as f:
        f.write(b"TNTW0001" + struct.pack("<I", len(layers)))
        for w, b, relu in layers:
            f.write(struct.pack("<III", w.shape[0], w.shape[1], relu))
            f.write(np.ascontiguousarray(w, dtype=np.float32).tobytes())
            f.write(np.ascontiguousarray(b, dtype=np.float32).tobytes())
    return len(layers)
