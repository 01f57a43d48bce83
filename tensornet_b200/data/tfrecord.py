"""TFRecord files of ``tf.train.Example`` records as training input, without TensorFlow.

The reference reads its input through ``tf.data``: files sharded by rank, an interleave of ``TFRecordDataset``
readers, ``batch`` and a parallel ``parse_example`` with one ``VarLenFeature(int64)`` per slot
(examples/common/util.py:23-39, examples/models/wide_deep.py parse function); its example data holds an int64
``label``, a bytes ``uniq_id`` and one int64 list per slot, where a slot may be missing from a record
(examples/gen_example_data.py:20-60).  :class:`TFRecordDataset` reads the same files through the native reader of
``csrc/tfrecord.cpp`` (worker threads, plain or gzip files, checksums verified) and yields ``(features, labels)``
batches in the containers the embedding layers take:

* default: ``{slot: Ragged(values, offsets)}``, any number of ids per example, none when the record lacks the slot;
* ``packed=True``: instead one :class:`PackedFeatures` under ``PACKED_KEY`` holding all slots in one buffer (one
  host-to-device copy per batch); for models whose embedding layers all take exactly ``sparse_keys``, in that
  order (with ``single_hot=True`` a layer may also take a subset);
* ``single_hot=True``: every slot has one id per example (``default_id`` when missing, the first of several), so
  batches have fixed shapes and replay from CUDA graphs: ``{slot: int64 [B]}`` or packed ``ids [S, B]``.

``TFRecordWriter`` and ``encode_example`` write such files (the example data generator and the tests use them).
"""
from __future__ import annotations

import os
import shutil
import tempfile
import threading
from typing import Dict, Iterator, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .. import _build
from ..utils.checkpoint import _fs_for, is_remote
from .features import PACKED_KEY, PackedFeatures, Ragged


def encode_example(ints: Optional[Mapping[str, Sequence[int]]] = None, floats: Optional[Mapping[str, Sequence[float]]] = None,
                   raw: Optional[Mapping[str, bytes]] = None) -> bytes:
    """Serialized ``tf.train.Example`` with int64-list, float-list and (single-value) bytes-list features."""
    ext = _build.cpu_ext()
    return ext.tf_example_encode({k: np.asarray(v, dtype=np.int64).reshape(-1) for k, v in (ints or {}).items()},
                                 {k: np.asarray(v, dtype=np.float32).reshape(-1) for k, v in (floats or {}).items()},
                                 dict(raw or {}))


class TFRecordWriter:
    """Writes records in TensorFlow's record framing (length, masked crc32c, data, masked crc32c); ``gzip=True``
    compresses the whole file the way ``TFRecordOptions(compression_type="GZIP")`` does."""

    def __init__(self, path: str, gzip: bool = False):
        self._w = _build.cpu_ext().TFRecordWriter(str(path), bool(gzip))

    def write(self, record: bytes) -> None:
        self._w.write(record)

    def close(self) -> None:
        self._w.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


class TFRecordDataset:
    """Iterable of ``(features, labels)`` batches read from TFRecord files.

    ``files``: the files THIS rank reads (``tn.data.list_files(...)[rank::world]``); names with a URL scheme
    (``hdfs://...``) are fetched to a scratch directory one by one as the readers get to them.  ``sparse_keys``: int64 features
    (slots).  ``dense_keys``: ``{name: width}`` of float features (shorter lists are zero-filled, int64 lists are
    converted) returned as one ``float32 [B, sum(widths)]`` tensor under ``dense_name``.  ``label_key``: int64 or
    float feature whose first value is the label (also copied into ``features[label_key]``).  ``bytes_keys``: bytes
    features returned as Python lists (for prediction dumps).

    ``num_workers`` threads each own every ``num_workers``-th file, keep ``cycle_length`` of them open and take
    ``block_length`` records from each in turn; batches are handed out worker after worker, so their order depends
    only on these arguments.  Every iteration starts from the first file again; ``shuffle_files=True`` reads the files in
    another order in every pass (determined by ``seed`` and the number of the pass).  Batches never mix records
    of two workers, so a pass ends with at most one short batch per worker (none with ``drop_remainder=True``).
    """

    def __init__(self, files: Sequence[str], batch_size: int, sparse_keys: Sequence[str],
                 dense_keys: Optional[Union[Mapping[str, int], Sequence[Tuple[str, int]]]] = None, label_key: Optional[str] = "label",
                 bytes_keys: Sequence[str] = (), *, dense_name: str = "dense", packed: bool = False, single_hot: bool = False,
                 default_id: int = 0, drop_remainder: bool = False, verify_checksums: bool = True, num_workers: int = 4,
                 cycle_length: int = 4, block_length: int = 8, queue_depth: int = 4, pin_memory: Optional[bool] = None,
                 shuffle_files: bool = False, seed: int = 0):
        self.files = [str(files)] if isinstance(files, (str, os.PathLike)) else [str(f) for f in files]
        self.batch_size = int(batch_size)
        self.sparse_keys = [str(k) for k in sparse_keys]
        items = list(dense_keys.items()) if isinstance(dense_keys, Mapping) else list(dense_keys or [])
        self.dense_keys = [(str(k), int(w)) for k, w in items]
        self.label_key = label_key or ""
        self.bytes_keys = [str(k) for k in bytes_keys]
        self.dense_name, self.packed, self.single_hot, self.default_id = dense_name, bool(packed), bool(single_hot), int(default_id)
        self.drop_remainder, self.verify = bool(drop_remainder), bool(verify_checksums)
        self.num_workers, self.cycle_length, self.block_length, self.queue_depth = int(num_workers), int(cycle_length), int(block_length), int(queue_depth)
        self.pin_memory = torch.cuda.is_available() if pin_memory is None else bool(pin_memory)
        self.shuffle_files, self.seed, self._passes = bool(shuffle_files), int(seed), 0

    @classmethod
    def from_columns(cls, files: Sequence[str], batch_size: int, feature_columns: Sequence, **kwargs) -> "TFRecordDataset":
        """The dataset that reads what ``feature_columns`` (category, sequence or embedding columns, e.g. the list an
        ``EmbeddingFeatures`` layer was built from) declare in their ``parse_example_spec``: one int64 list per
        column key, in the columns' order.  Other arguments as for the constructor."""
        keys = []
        for c in feature_columns:
            for k in c.parse_example_spec:
                if k not in keys:
                    keys.append(k)
        return cls(files, batch_size, keys, **kwargs)

    def _tensor(self, a: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(a)
        return t.pin_memory() if self.pin_memory and t.numel() else t

    def _convert(self, raw: Dict) -> Tuple[Dict, Optional[torch.Tensor]]:
        n, keys = int(raw["n"]), self.sparse_keys
        feats: Dict = {}
        if self.single_hot:
            ids = self._tensor(raw["ids"])
            if self.packed:
                feats[PACKED_KEY] = PackedFeatures(keys, ids=ids)
            else:
                for s, k in enumerate(keys):
                    feats[k] = ids[s]
        else:
            values = self._tensor(raw["values"])
            if self.packed:
                feats[PACKED_KEY] = PackedFeatures(keys, values=values, offsets=self._tensor(raw["offsets"]), batch_size=n)
            else:
                base, local = raw["slot_base"], self._tensor(raw["local_offsets"])
                for s, k in enumerate(keys):
                    feats[k] = Ragged(values[int(base[s]):int(base[s + 1])], local[s])
        if self.dense_keys:
            feats[self.dense_name] = self._tensor(raw["dense"])
        labels = None
        if self.label_key:
            labels = self._tensor(raw["label"])
            feats[self.label_key] = labels
        for k in self.bytes_keys:
            feats[k] = raw[k]
        return feats, labels

    def __iter__(self) -> Iterator[Tuple[Dict, Optional[torch.Tensor]]]:
        ext = _build.cpu_ext()
        scratch = _Scratch() if any(is_remote(f) for f in self.files) else None
        files = self.files
        if self.shuffle_files:                 # another order in every pass, the same on every run with this seed
            order = np.random.default_rng([self.seed, self._passes]).permutation(len(files))
            files = [files[i] for i in order]
        self._passes += 1
        b = ext.TFRecordBatcher(files, self.batch_size, self.sparse_keys, [k for k, _ in self.dense_keys],
                                [w for _, w in self.dense_keys], self.label_key, self.bytes_keys, self.single_hot,
                                self.default_id, self.drop_remainder, self.verify, self.num_workers, self.cycle_length,
                                self.block_length, self.queue_depth, scratch.localize if scratch else None,
                                scratch.release if scratch else None)
        try:
            while True:
                raw = b.next()
                if raw is None:
                    return
                yield self._convert(raw)
        finally:
            b.close()
            if scratch:
                scratch.close()


class _Scratch:
    """Local copies of remote input files (``hdfs://...``, any scheme the installed file-system layer knows): a reader
    thread asks for a file when its turn comes and gives it back when it has read it, so at most
    ``num_workers x cycle_length`` copies exist at a time.  The reference reaches such files through TensorFlow's
    file-system layer (core/utility/file_io.cc:47-50); here they come through fsspec or an installed client
    (``tn.utils.checkpoint.set_remote_fs``)."""

    def __init__(self):
        self.dir = tempfile.mkdtemp(prefix="tn_input_")
        self._lock = threading.Lock()
        self._local: Dict[str, str] = {}
        self._count = 0

    def localize(self, name: str) -> str:
        if not is_remote(name):
            return name[7:] if name.startswith("file://") else name
        fs, rpath = _fs_for(name)
        with self._lock:
            dst = os.path.join(self.dir, "%06d_%s" % (self._count, os.path.basename(rpath.rstrip("/"))))
            self._count += 1
            self._local[name] = dst
        fs.get(rpath, dst)
        return dst

    def release(self, name: str) -> None:
        with self._lock:
            dst = self._local.pop(name, None)
        if dst and os.path.exists(dst):
            os.remove(dst)

    def close(self) -> None:
        shutil.rmtree(self.dir, ignore_errors=True)
