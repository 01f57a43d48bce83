"""Builds and loads the native extensions in-tree.

Two shared objects are produced under ``tensornet_b200/_ext``:

* ``_tn_cuda`` - the sm_100a kernels (``csrc/*.cu``) plus their bindings.  Compiled with
  ``-gencode arch=compute_100a,code=sm_100a`` so the tcgen05 / TMA instructions are legal;
  nvcc cross-compiles on a machine without a GPU.
* ``_tn_cpu``  - the plain C++ restatement of the reference's parameter-server algorithms
  (CPU oracle and CPU execution path) and the checkpoint reader/writer.

At import time a previously built ``.so`` is loaded directly; building happens only through
:func:`build_all` (or lazily on first use when no built object exists).
"""
from __future__ import annotations

import importlib.util
import os
import sys
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, "csrc")
_EXT = os.path.join(_HERE, "_ext")
_LOCK = threading.Lock()
_LOADED: dict[str, object] = {}

CUDA_SOURCES = [
    "bindings.cpp",
    "sparse_fused.cu",
    "pooling.cu",
    "table_ops.cu",
    "gemm_tcgen05.cu",
    "dense_fused.cu",
    "elementwise.cu",
    "serving.cu",
    "peer_probe.cu",
    "bn.cu",
    "unique.cu",
    "deepfm_fused.cu",
    "no_alloc.cu",
]
CPU_SOURCES = ["cpu_ref.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "--expt-relaxed-constexpr", "-std=c++17",
]


def _existing(names):
    return [os.path.join(_CSRC, n) for n in names if os.path.exists(os.path.join(_CSRC, n))]


def _so_path(name: str) -> str:
    return os.path.join(_EXT, name, name + ".so")


def _import_so(name: str):
    import torch  # noqa: F401  (libtorch / libc10 must be loaded before the extension)

    path = _so_path(name)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules.setdefault(name, mod)
    return mod


def _build(name: str, sources, cuda: bool, verbose: bool = False):
    from torch.utils import cpp_extension

    os.makedirs(os.path.join(_EXT, name), exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    kwargs = dict(
        name=name,
        sources=sources,
        extra_cflags=["-O3", "-std=c++17"],
        extra_include_paths=[_CSRC],
        build_directory=os.path.join(_EXT, name),
        verbose=verbose,
    )
    if cuda:
        kwargs["extra_cuda_cflags"] = NVCC_FLAGS
        kwargs["with_cuda"] = True
        kwargs["extra_ldflags"] = ["-lcuda"] if _has_libcuda() else []
    else:
        kwargs["extra_ldflags"] = ["-lz"]
    return cpp_extension.load(**kwargs)


def _has_libcuda() -> bool:
    # The kernels reach the driver API only through cudaGetDriverEntryPoint, so libcuda is
    # not needed at link time.
    return False


def _stale(name: str, sources) -> bool:
    so = _so_path(name)
    if not os.path.exists(so):
        return True
    t = os.path.getmtime(so)
    deps = list(sources) + [os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if f.endswith((".h", ".cuh"))]
    return any(os.path.getmtime(d) > t for d in deps)


def load(name: str, *, rebuild: bool = False, verbose: bool = False):
    """Return the extension module ``name`` (``_tn_cuda`` or ``_tn_cpu``)."""
    with _LOCK:
        if name in _LOADED and not rebuild:
            return _LOADED[name]
        cuda = name == "_tn_cuda"
        sources = _existing(CUDA_SOURCES if cuda else CPU_SOURCES)
        if rebuild or not os.path.exists(_so_path(name)):
            mod = _build(name, sources, cuda, verbose)
        else:
            mod = _import_so(name)
        _LOADED[name] = mod
        return mod


def build_all(verbose: bool = False, force: bool = False):
    """Compile every extension (used by the repository's build entry point)."""
    out = {}
    for name, srcs, cuda in (("_tn_cpu", CPU_SOURCES, False), ("_tn_cuda", CUDA_SOURCES, True)):
        sources = _existing(srcs)
        if not sources:
            continue
        with _LOCK:
            if force or _stale(name, sources):
                _LOADED[name] = _build(name, sources, cuda, verbose)
            elif name not in _LOADED:
                _LOADED[name] = _import_so(name)
            out[name] = _LOADED[name]
    return out


def cuda_ext():
    return load("_tn_cuda")


def cpu_ext():
    return load("_tn_cpu")
