from __future__ import annotations

import os
from typing import Optional

import numpy as np
import torch

from .. import _build
from ..core.runtime import runtime
from ..ops import functional as F
from ..tools import merge_sparse


def export_sparse_dictionary(checkpoint_dir: str, table_name: str, out_file: str, **kw) -> int:
    """Merge ``<checkpoint_dir>/sparse_table/<table_name>/rank_*/block_*`` into one text dictionary."""
    return merge_sparse(os.path.join(checkpoint_dir, "sparse_table", table_name), out_file, **kw)


class EmbeddingDictionary:
    """Read-only ``sign -> embedding`` table.  On a GPU it is an open-addressing hash table probed by the
    lookup kernel; on the CPU a sorted array searched with numpy."""

    def __init__(self, signs: np.ndarray, weights: np.ndarray):
        rt = runtime()
        self.dim = int(weights.shape[1])
        self.n = int(len(signs))
        self.on_gpu = rt.on_gpu
        if self.on_gpu:
            ext = _build.cuda_ext()
            dev = rt.device
            cap = 1 << max(4, int(np.ceil(np.log2(max(self.n, 1) * 2 + 1))))
            self.stride = (self.dim + 3) // 4 * 4
            self.keys = torch.full((cap,), -1, dtype=torch.int64, device=dev)
            self.slots = torch.full((cap,), -1, dtype=torch.int32, device=dev)
            self.rows = torch.zeros((max(self.n, 1), self.stride), dtype=torch.float32, device=dev)
            self.row_keys = torch.zeros(max(self.n, 1), dtype=torch.int64, device=dev)
            self.row_tag = torch.zeros(max(self.n, 1), dtype=torch.int64, device=dev)
            self.n_rows = torch.zeros(1, dtype=torch.int32, device=dev)
            k = torch.from_numpy(np.ascontiguousarray(signs, dtype=np.uint64).view(np.int64)).to(dev)
            idx = torch.empty(self.n, dtype=torch.int32, device=dev)
            if self.n:
                ext.table_insert_keys(self.table_dict(), k, idx, rt.status)
                w = torch.zeros((self.n, self.stride), dtype=torch.float32, device=dev)
                w[:, : self.dim] = torch.from_numpy(np.ascontiguousarray(weights, dtype=np.float32)).to(dev)
                self.rows.index_copy_(0, idx.long(), w)
            rt.check_status()
        else:
            order = np.argsort(signs)
            self.signs = np.ascontiguousarray(signs[order], dtype=np.uint64)
            self.weights = np.ascontiguousarray(weights[order], dtype=np.float32)

    def table_dict(self):
        return dict(keys=self.keys, slots=self.slots, rows=self.rows, row_keys=self.row_keys, row_tag=self.row_tag,
                    n_rows=self.n_rows, dim=self.dim, stride=self.stride, use_cvm=0)

    @classmethod
    def from_file(cls, path: str, dim: Optional[int] = None, chunk_rows: int = 1 << 18) -> "EmbeddingDictionary":
        """Load ``sign \\t [ \\t w... \\t ]`` lines (brackets optional), plain or gzip.  The file is read and parsed in
        native code, ``chunk_rows`` lines at a time; ``dim`` keeps only the first ``dim`` weights of a row."""
        reader = _build.cpu_ext().DictionaryReader(path)
        signs, rows = [], []
        while True:
            s, r = reader.next(int(chunk_rows))
            if not len(s):
                break
            signs.append(s)
            rows.append(np.ascontiguousarray(r[:, :dim]) if dim else r)
        if not signs:
            return cls(np.zeros(0, np.uint64), np.zeros((0, dim or 1), np.float32))
        return cls(np.concatenate(signs), np.concatenate(rows))

    @classmethod
    def from_table(cls, table) -> "EmbeddingDictionary":
        signs, rows = table.dump()
        return cls(signs, rows[:, : table.dim])

    def lookup_cpu(self, ids: np.ndarray) -> np.ndarray:
        pos = np.searchsorted(self.signs, ids)
        pos = np.clip(pos, 0, max(self.n - 1, 0))
        hit = self.signs[pos] == ids if self.n else np.zeros(len(ids), bool)
        out = np.zeros((len(ids), self.dim), np.float32)
        out[hit] = self.weights[pos[hit]]
        return out


class InferenceEngine:
    """``ids [S, B]`` (or ragged) -> click probabilities, for a dense tower ``MLP`` + ``DenseHead``.

    The first call for a batch shape captures lookup + towers + sigmoid in a CUDA graph; later calls copy
    the ids into the static buffer and replay it."""

    def __init__(self, dictionary: EmbeddingDictionary, mlp, head, n_slots: int, combiner: str = "mean"):
        self.dict, self.mlp, self.head, self.S = dictionary, mlp, head, n_slots
        self.combiner = {"sum": 0, "mean": 1, "sqrtn": 2}[combiner]
        self._graphs = {}
        assert mlp.in_dim == n_slots * dictionary.dim, "tower input width must equal slots * dim"

    def _forward_gpu(self, ids, offsets, B):
        ext = _build.cuda_ext()
        ld = F.pad8(self.mlp.in_dim + 1)
        x0 = torch.empty((B, ld), dtype=torch.bfloat16, device=ids.device)
        ext.dict_lookup_pool(self.dict.table_dict(), ids, offsets, B, self.S, self.combiner, x0, ld, self.mlp.in_dim)
        logit = self.head(self.mlp(x0)).view(-1)
        prob = torch.empty_like(logit)
        ext.sigmoid(logit, prob)
        return prob

    @torch.no_grad()
    def infer(self, ids: torch.Tensor, offsets: Optional[torch.Tensor] = None, use_graph: bool = True) -> torch.Tensor:
        rt = runtime()
        if not rt.on_gpu:
            B = ids.shape[1] if offsets is None else (offsets.numel() - 1) // self.S
            flat = ids.reshape(-1).cpu().numpy().astype(np.uint64)
            emb = torch.from_numpy(self.dict.lookup_cpu(flat))
            if offsets is None:
                pooled = emb.view(self.S, B, -1)
            else:
                lens = (offsets[1:] - offsets[:-1]).long()
                bag = torch.repeat_interleave(torch.arange(self.S * B), lens)
                pooled = torch.zeros(self.S * B, self.dict.dim).index_add_(0, bag, emb)
                if self.combiner == 1:
                    pooled = pooled / lens.clamp(min=1).unsqueeze(1)
                pooled = pooled.view(self.S, B, -1)
            x = pooled.permute(1, 0, 2).reshape(B, -1)
            return torch.sigmoid(self.head(self.mlp(F.concat_cast([x], ones=True)))).view(-1)
        dev = rt.device
        if offsets is not None or not use_graph:
            B = ids.shape[1] if offsets is None else (offsets.numel() - 1) // self.S
            return self._forward_gpu(ids.to(dev).reshape(-1), None if offsets is None else offsets.to(dev).int(), B)
        B = int(ids.shape[1])
        entry = self._graphs.get(B)
        if entry is None:
            static_ids = torch.empty((self.S * B,), dtype=torch.int64, device=dev)
            static_ids.copy_(ids.reshape(-1), non_blocking=True)
            for _ in range(2):
                self._forward_gpu(static_ids, None, B)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = self._forward_gpu(static_ids, None, B)
            entry = (g, static_ids, out)
            self._graphs[B] = entry
        g, static_ids, out = entry
        static_ids.copy_(ids.reshape(-1), non_blocking=True)
        g.replay()
        return out


class ShardedInferenceEngine:
    """Serving with the dictionary sharded over all GPUs of the job (``sign % world`` decides the owner), for
    dictionaries too large for one GPU's memory.  The reference's exported dictionary "may approach TB"
    (doc/tutorial/05-export-sparse-feature-embedding.ipynb:156) and its demo fakes the lookup
    (examples/online_serving/main.cc:76-81); here every rank takes its own request batches and the lookups cross
    NVLink inside the fused pull kernel running read-only (``lookup_only``: signs no shard holds pull zeros and
    nothing is inserted).  Lookup, pooling, towers and sigmoid are captured in one CUDA graph per batch shape.

    All ranks must call :meth:`infer` the same number of times with the same batch shape: the pull is collective.
    With one GPU it behaves like :class:`InferenceEngine` over a training-format table."""

    def __init__(self, table, mlp, head, n_slots: int, max_ids: int, combiner: str = "mean"):
        from ..ops.embedding import COMBINERS

        self.table, self.mlp, self.head, self.S = table, mlp, head, n_slots
        self.combiner = COMBINERS[combiner]
        self.link = table.link(max_ids)
        self._graphs = {}
        assert mlp.in_dim == n_slots * table.dim, "tower input width must equal slots * dim"

    @classmethod
    def from_dictionary(cls, signs: np.ndarray, weights: np.ndarray, mlp, head, n_slots: int, max_ids: int,
                        combiner: str = "mean", rows_per_gpu: Optional[int] = None):
        """Build the sharded table from a full ``sign -> embedding`` dictionary held on the host: every rank keeps
        the signs it owns."""
        from ..core.optimizers import Adam
        from ..ops.sparse_table_gpu import GpuSparseTable, row_floats

        rt = runtime()
        signs = np.ascontiguousarray(signs, dtype=np.uint64)
        mine = (signs % np.uint64(rt.world)) == np.uint64(rt.rank)
        opt = Adam(learning_rate=0.0)
        dim = int(weights.shape[1])
        table = GpuSparseTable(opt, dim, rows=rows_per_gpu or max(1024, int(mine.sum()) + 1024))
        rows = np.zeros((int(mine.sum()), row_floats(table.kind, dim)), dtype=np.float32)
        rows[:, :dim] = weights[mine]
        table.load_rows(signs[mine], rows)
        return cls(table, mlp, head, n_slots, max_ids, combiner)

    def _forward(self, ids, offsets, B):
        ext = _build.cuda_ext()
        lk = self.link
        inverse = lk.pull(ids, None, 0, training=False, lookup_only=True)
        pd = lk.pdim
        pooled = torch.empty((B, self.S * pd), dtype=torch.float32, device=ids.device)
        ext.pool_fwd(lk.U, lk.ustride, inverse, offsets, B, self.S, pd, self.combiner, pooled, self.S * pd)
        x0 = F.concat_cast([pooled], ones=True)
        logit = self.head(self.mlp(x0)).view(-1)
        prob = torch.empty_like(logit)
        ext.sigmoid(logit, prob)
        return prob

    @torch.no_grad()
    def infer(self, ids: torch.Tensor, offsets: Optional[torch.Tensor] = None, use_graph: bool = True) -> torch.Tensor:
        rt = runtime()
        assert rt.on_gpu, "sharded serving runs on GPUs"
        dev = rt.device
        if offsets is not None or not use_graph:
            B = ids.shape[1] if offsets is None else (offsets.numel() - 1) // self.S
            return self._forward(ids.to(dev).reshape(-1), None if offsets is None else offsets.to(dev).int(), B)
        B = int(ids.shape[1])
        entry = self._graphs.get(B)
        if entry is None:
            static_ids = torch.empty((self.S * B,), dtype=torch.int64, device=dev)
            static_ids.copy_(ids.reshape(-1), non_blocking=True)
            for _ in range(2):
                self._forward(static_ids, None, B)
            torch.cuda.synchronize()
            rt.check_status()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = self._forward(static_ids, None, B)
            entry = (g, static_ids, out)
            self._graphs[B] = entry
        g, static_ids, out = entry
        static_ids.copy_(ids.reshape(-1), non_blocking=True)
        g.replay()
        return out
