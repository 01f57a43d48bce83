"""Batches stored the way the device takes them.

Parsing records costs the host about a microsecond per example (``benchmarks/input_bench.py``), thirty
times what a B200 needs to train on it; the reference has the same imbalance between its TensorFlow input
pipeline and its parameter servers and hides it behind ``prefetch``.  A batch cache removes the parsing from the
training run: a pass over the input (``TFRecordDataset`` or any iterable of ``(features, labels)``) is written once as
whole batches, each one blob holding exactly the arrays a step copies to the GPU (ids of all slots slot-major, bag
offsets when slots are ragged, dense features, labels).  Reading a batch is one read of one contiguous byte range
into page-locked memory; the tensors of the batch are views of that buffer.

File layout: ``TNBC0001`` | u64 length of the header | header (JSON: slot names, dense width, label flag, batch
size) | blobs, each 64-byte aligned | index (per batch: offset, bytes, examples, ids, ragged flag) | u64 offset of
the index | u64 number of batches | ``TNBC0001``.  The index comes last so that a writer streams.
"""
from __future__ import annotations

import collections
import json
import os
import struct
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch

from .features import PACKED_KEY, PackedFeatures, gather_columns

_MAGIC = b"TNBC0001"
_ALIGN = 64
_ENTRY = struct.Struct("<QQIQI")          # offset, bytes, examples, ids, flags (1 = ragged)


def _pad(n: int) -> int:
    return (-n) % _ALIGN


class BatchCacheWriter:
    """Appends batches to a cache file.  ``sparse_keys``: the slots, in the order the model's embedding layers take
    them.  ``dense_name`` / ``label``: what else a batch carries (looked up in ``features`` / given as ``labels``)."""

    def __init__(self, path: str, sparse_keys: Sequence[str], dense_name: Optional[str] = None, label: bool = True):
        self.path, self.keys, self.dense_name, self.label = str(path), [str(k) for k in sparse_keys], dense_name, bool(label)
        self._f = open(self.path, "wb")
        self._index: List[bytes] = []
        self._dense_width: Optional[int] = None
        self._header_written = False
        self.examples = 0

    def _header(self, dense_width: int):
        head = json.dumps({"version": 1, "sparse_keys": self.keys, "dense_name": self.dense_name, "dense_width": dense_width,
                           "label": self.label}).encode()
        self._f.write(_MAGIC + struct.pack("<Q", len(head)) + head)
        self._f.write(b"\0" * _pad(self._f.tell()))
        self._dense_width, self._header_written = dense_width, True

    def append(self, features: Dict, labels: Optional[torch.Tensor] = None) -> None:
        ids, offsets, B = gather_columns(features, self.keys, torch.device("cpu"))
        dense = features[self.dense_name].reshape(B, -1).float().contiguous() if self.dense_name else None
        if not self._header_written:
            self._header(0 if dense is None else int(dense.shape[1]))
        if (0 if dense is None else int(dense.shape[1])) != self._dense_width:
            raise ValueError("the dense width changed between batches")
        parts = [ids.long().contiguous().numpy()]
        if offsets is not None:
            parts.append(offsets.int().contiguous().numpy())
        if dense is not None:
            parts.append(dense.numpy())
        if self.label:
            if labels is None:
                raise ValueError("this cache stores labels; pass them")
            parts.append(labels.reshape(-1).float().contiguous().numpy())
            if parts[-1].shape[0] != B:
                raise ValueError("one label per example")
        start = self._f.tell()
        for a in parts:
            self._f.write(a.tobytes())
            self._f.write(b"\0" * _pad(self._f.tell()))
        self._index.append(_ENTRY.pack(start, self._f.tell() - start, B, int(ids.numel()), 0 if offsets is None else 1))
        self.examples += B

    def close(self) -> None:
        if self._f is None:
            return
        if not self._header_written:
            self._header(0)
        at = self._f.tell()
        self._f.write(b"".join(self._index))
        self._f.write(struct.pack("<QQ", at, len(self._index)) + _MAGIC)
        self._f.close()
        self._f = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def write_batch_cache(path: str, dataset: Iterable, sparse_keys: Sequence[str], dense_name: Optional[str] = None,
                      label: bool = True) -> int:
    """One pass over ``dataset`` (an iterable of ``(features, labels)``) into a cache file; returns the number of
    examples written."""
    with BatchCacheWriter(path, sparse_keys, dense_name, label) as w:
        for features, labels in dataset:
            w.append(features, labels)
        return w.examples


class _CacheFile:
    def __init__(self, path: str):
        self.path = path
        self.fd = os.open(path, os.O_RDONLY)
        size = os.fstat(self.fd).st_size
        tail = os.pread(self.fd, 24, size - 24) if size >= 40 else b""
        head = os.pread(self.fd, 16, 0)
        if len(tail) != 24 or tail[16:] != _MAGIC or head[:8] != _MAGIC:
            os.close(self.fd)
            raise ValueError(f"{path} is not a batch cache (or was not closed by its writer)")
        at, n = struct.unpack("<QQ", tail[:16])
        self.meta = json.loads(os.pread(self.fd, struct.unpack("<Q", head[8:])[0], 16))
        raw = os.pread(self.fd, n * _ENTRY.size, at)
        self.entries = [_ENTRY.unpack_from(raw, i * _ENTRY.size) for i in range(n)]

    def close(self):
        if self.fd >= 0:
            os.close(self.fd)
            self.fd = -1


class BatchCacheDataset:
    """Iterable of ``(features, labels)`` read back from cache files, in the order they were written.

    ``features`` holds one :class:`PackedFeatures` under ``PACKED_KEY`` (plus the dense tensor and, under
    ``label_name``, the labels).  ``shard=(index, count)`` keeps every ``count``-th batch starting at ``index`` (ranks
    of one job reading one cache).  ``threads`` background threads keep ``prefetch`` batches in flight, each read into
    its own page-locked buffer when a GPU is present, so a step's input is ready before the step is issued."""

    def __init__(self, paths, shard: Tuple[int, int] = (0, 1), prefetch: int = 4, pin_memory: Optional[bool] = None,
                 label_name: str = "label", threads: int = 2):
        self.paths = [str(paths)] if isinstance(paths, (str, os.PathLike)) else [str(p) for p in paths]
        self.shard, self.prefetch, self.label_name = (int(shard[0]), int(shard[1])), max(1, int(prefetch)), label_name
        self.pin_memory = torch.cuda.is_available() if pin_memory is None else bool(pin_memory)
        self.threads = max(1, min(int(threads), self.prefetch))

    def __len__(self) -> int:
        n = 0
        for p in self.paths:
            f = _CacheFile(p)
            n += len(f.entries)
            f.close()
        i, c = self.shard
        return (n - i + c - 1) // c if n > i else 0

    def _load(self, f: _CacheFile, entry) -> Tuple[Dict, Optional[torch.Tensor]]:
        off, nbytes, B, nids, flags = entry
        buf = torch.empty(nbytes, dtype=torch.uint8, pin_memory=self.pin_memory)
        view = memoryview(buf.numpy())
        got = 0
        while got < nbytes:
            r = os.preadv(f.fd, [view[got:]], off + got)
            if r <= 0:
                raise IOError(f"{f.path} ends inside a batch")
            got += r
        meta, at = f.meta, 0

        def take(count: int, dtype: torch.dtype, width: int) -> torch.Tensor:
            nonlocal at
            t = buf[at:at + count * width].view(dtype)
            at += count * width
            at += _pad(at)
            return t

        keys = meta["sparse_keys"]
        ids = take(nids, torch.int64, 8)
        if flags & 1:
            packed = PackedFeatures(keys, values=ids, offsets=take(len(keys) * B + 1, torch.int32, 4), batch_size=B)
        else:
            packed = PackedFeatures(keys, ids=ids.view(len(keys), B))
        feats: Dict = {PACKED_KEY: packed}
        if meta["dense_width"]:
            feats[meta["dense_name"]] = take(B * meta["dense_width"], torch.float32, 4).view(B, meta["dense_width"])
        labels = None
        if meta["label"]:
            labels = take(B, torch.float32, 4)
            feats[self.label_name] = labels
        return feats, labels

    def __iter__(self) -> Iterator[Tuple[Dict, Optional[torch.Tensor]]]:
        files = [_CacheFile(p) for p in self.paths]
        todo, k = [], 0
        for f in files:
            for entry in f.entries:
                if k % self.shard[1] == self.shard[0]:
                    todo.append((f, entry))
                k += 1
        pool = ThreadPoolExecutor(max_workers=self.threads, thread_name_prefix="tn-batch-cache")
        pending: "collections.deque" = collections.deque()
        try:
            nxt = 0
            while nxt < len(todo) or pending:
                while nxt < len(todo) and len(pending) < self.prefetch:     # reads run side by side, batches leave in order
                    pending.append(pool.submit(self._load, *todo[nxt]))
                    nxt += 1
                yield pending.popleft().result()
        finally:
            for fut in pending:
                fut.cancel()
            pool.shutdown(wait=True)
            for f in files:
                f.close()
