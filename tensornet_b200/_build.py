"""Builds and loads the native extensions in-tree.

Two shared objects are produced under ``tensornet_b200/_ext``:

* ``_tn_cuda`` - the sm_100a kernels (``csrc/*.cu``) plus their bindings.  Compiled with
  ``-gencode arch=compute_100a,code=sm_100a`` so the tcgen05 / TMA instructions are legal;
  nvcc cross-compiles on a machine without a GPU.
* ``_tn_cpu``  - the plain C++ restatement of the reference's parameter-server algorithms
  (CPU oracle and CPU execution path) and the checkpoint reader/writer.

With ``TN_CPU_SANITIZE=1`` the C++ runtime is built a second time as ``_tn_cpu_san`` with AddressSanitizer and
UndefinedBehaviorSanitizer and used in place of ``_tn_cpu`` (run Python with the ASan runtime preloaded:
``LD_PRELOAD=$(gcc -print-file-name=libasan.so) ASAN_OPTIONS=detect_leaks=0``); the CI job ``cpu-sanitizers`` runs the
table, checkpoint and streaming tests that way.  ``TN_CPU_SANITIZE=thread`` does the same with ThreadSanitizer
(``_tn_cpu_tsan``, ``LD_PRELOAD=$(gcc -print-file-name=libtsan.so)``) for the code that runs its own threads: the
TFRecord reader's workers, the lock-striped tables, the parallel block readers.

A built ``.so`` is loaded directly when the digest of the sources it was built from (kept next
to it) still matches ``csrc``; otherwise it is rebuilt first, so an edited kernel can never run
as its previous build.
"""
from __future__ import annotations

import hashlib
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
    "mlp_fused.cu", "gemm_2sm.cu",
    "dense_fused.cu",
    "elementwise.cu",
    "serving.cu",
    "bn.cu",
    "unique.cu",
    "deepfm_fused.cu",
    "no_alloc.cu",
]
CPU_SOURCES = ["cpu_ref.cpp", "tfrecord.cpp"]

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
    sanitize = name.endswith("_san")
    tsan = name.endswith("_tsan")
    kwargs = dict(
        name=name,
        sources=sources,
        extra_cflags=(["-O1", "-g", "-std=c++17", "-fsanitize=address,undefined", "-fno-omit-frame-pointer"] if sanitize
                      else ["-O1", "-g", "-std=c++17", "-fsanitize=thread", "-fno-omit-frame-pointer"] if tsan
                      else ["-O3", "-std=c++17"]),
        extra_include_paths=[_CSRC],
        build_directory=os.path.join(_EXT, name),
        verbose=verbose,
    )
    if cuda:
        kwargs["extra_cuda_cflags"] = NVCC_FLAGS
        kwargs["with_cuda"] = True
        kwargs["extra_ldflags"] = ["-lcuda"] if _has_libcuda() else []
    else:
        kwargs["extra_ldflags"] = ["-lz"] + (["-fsanitize=address,undefined"] if sanitize else ["-fsanitize=thread"] if tsan else [])
    # The compiler and ninja must not inherit a preloaded sanitizer runtime (this process keeps its own copy).
    preload = os.environ.pop("LD_PRELOAD", None) if (sanitize or tsan) else None
    try:
        mod = cpp_extension.load(**kwargs)
    finally:
        if preload is not None:
            os.environ["LD_PRELOAD"] = preload
    with open(_digest_path(name), "w") as f:
        f.write(_digest(sources))
    return mod


def _has_libcuda() -> bool:
    # The kernels reach the driver API only through cudaGetDriverEntryPoint, so libcuda is
    # not needed at link time.
    return False


def _digest(sources) -> str:
    """SHA-256 over the sources and every header of ``csrc`` (content, not time stamps: a checkout or a copy of
    the tree changes the latter)."""
    h = hashlib.sha256()
    deps = sorted(set(sources) | {os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if f.endswith((".h", ".cuh"))})
    for d in deps:
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _digest_path(name: str) -> str:
    return os.path.join(_EXT, name, "sources.sha256")


def _stale(name: str, sources) -> bool:
    if not os.path.exists(_so_path(name)):
        return True
    try:
        with open(_digest_path(name)) as f:
            return f.read().strip() != _digest(sources)
    except OSError:
        return True


def load(name: str, *, rebuild: bool = False, verbose: bool = False):
    """Return the extension module ``name`` (``_tn_cuda`` or ``_tn_cpu``)."""
    with _LOCK:
        if name in _LOADED and not rebuild:
            return _LOADED[name]
        cuda = name == "_tn_cuda"
        sources = _existing(CUDA_SOURCES if cuda else CPU_SOURCES)
        if rebuild or _stale(name, sources):
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
    mode = os.environ.get("TN_CPU_SANITIZE", "")
    if mode == "thread":
        return load("_tn_cpu_tsan")
    if mode not in ("", "0"):
        return load("_tn_cpu_san")
    return load("_tn_cpu")
