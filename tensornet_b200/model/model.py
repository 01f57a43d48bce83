"""``tn.model.Model``: training / inference driver around an ``nn.Module``.

Same life-cycle as the reference's Keras subclass (tensornet/model/Model.py:60-256): a custom
train step (forward, backward, ONE fused dense update, then ``backwards`` = sparse push on every
embedding layer), ``predict_step`` returning ``(y, y_pred)``, composite
``save_weights / load_weights / load_sparse_weights / show_decay`` over sparse tables, dense
table and batch-norm tables, and a ``_checkpoint`` done-file written last.

B200 specifics: after a few eager steps the whole step (pull kernel, towers, loss, dense
update, push kernel) is captured into CUDA graphs and replayed.  Two graphs with two sets of
static input buffers take turns, so the inputs of step k+1 are copied (straight from pinned host
memory, on a second stream) while the graph of step k still runs.  The loss kernels keep the
sums and prediction histograms that the compiled metrics need on the device; the host reads
them when a result is asked for, not every step.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence

import torch
from torch import nn

from .. import core, metric as _metric
from .._opentelemetry import phase, start_as_current_span
from ..data.features import PackedFeatures, Ragged
from ..ops import functional as F
from ..parallel.symm import verify_all_arenas


# ----------------------------------------------------------------------------------------------
# done-file helpers (tensornet/model/Model.py:27-58)
# ----------------------------------------------------------------------------------------------
def load_done_info(cp_dir: str):
    done_file = os.path.join(cp_dir, "_checkpoint")
    if not os.path.exists(done_file):
        return None
    with open(done_file) as f:
        return json.load(f)


def save_done_info(cp_dir: str, dt: str):
    os.makedirs(cp_dir, exist_ok=True)
    tmp = os.path.join(cp_dir, "_checkpoint.tmp")
    with open(tmp, "w") as f:
        json.dump({"dt": dt}, f)
    os.replace(tmp, os.path.join(cp_dir, "_checkpoint"))


def read_last_train_dt(filepath: str):
    info = load_done_info(filepath)
    return info.get("dt") if info else None


def match_dtype_and_rank(y_t, y_p, sw=None):
    """Bring labels (and sample weights) to the prediction's dtype and rank
    (tensornet/model/compile_utils.py)."""
    if y_t.dim() == 1 and y_p.dim() == 2:
        y_t = y_t.unsqueeze(-1)
    y_t = y_t.to(y_p.dtype)
    if sw is not None:
        if sw.dim() == 1 and y_p.dim() == 2:
            sw = sw.unsqueeze(-1)
        sw = sw.to(y_p.dtype)
    return y_t, y_p, sw


def apply_mask(y_p, sw, mask):
    """Fold a boolean mask into the sample weights (tensornet/model/compile_utils.py)."""
    if mask is None:
        return sw
    mask = mask.to(y_p.dtype)
    if sw is None:
        return mask
    return sw * mask


# ----------------------------------------------------------------------------------------------
def _flatten(obj, out: List[torch.Tensor]):
    """Structure-preserving flatten of (nested) batch containers into a list of tensors."""
    if torch.is_tensor(obj):
        out.append(obj)
        return ("t",)
    if isinstance(obj, PackedFeatures):
        spec = []
        for name in ("ids", "values", "offsets"):
            t = getattr(obj, name)
            spec.append(None if t is None else _flatten(t, out))
        return ("packed", tuple(obj.keys), obj.batch_size, tuple(spec))
    if isinstance(obj, Ragged):
        return ("ragged", (_flatten(obj.values, out), _flatten(obj.offsets, out)))
    if isinstance(obj, dict):
        return ("dict", tuple((k, _flatten(v, out)) for k, v in obj.items()))
    if isinstance(obj, (list, tuple)):
        return ("list", tuple(_flatten(v, out) for v in obj))
    return ("const", obj)


def _unflatten(spec, it):
    kind = spec[0]
    if kind == "t":
        return next(it)
    if kind == "packed":
        _, keys, bs, sub = spec
        vals = [None if s is None else _unflatten(s, it) for s in sub]
        return PackedFeatures(list(keys), vals[0], vals[1], vals[2], bs)
    if kind == "ragged":
        return Ragged(*[_unflatten(s, it) for s in spec[1]])
    if kind == "dict":
        return {k: _unflatten(s, it) for k, s in spec[1]}
    if kind == "list":
        return [_unflatten(s, it) for s in spec[1]]
    return spec[1]


def _is_static(spec) -> bool:
    """True when every tensor of the batch has a batch-independent shape (no ragged features)."""
    kind = spec[0]
    if kind == "ragged":
        return False
    if kind == "packed":
        return spec[3][0] is not None
    if kind == "dict":
        return all(_is_static(s) for _, s in spec[1])
    if kind == "list":
        return all(_is_static(s) for s in spec[1])
    return True


_LOSS_RING = 32     # pinned slots for per-step losses on their way to the host: how far the host may run ahead


def graph_decision(world: int, known: bool, static: bool, n_graphs: int, max_graphs: int, eager_steps: int,
                   warmup: int) -> str:
    """What ``train_step`` does with a batch: ``"eager"``, ``"capture"`` (then replay) or ``"replay"``.

    Capturing ends with a host barrier, so with several ranks every rank must capture at the same step or none
    may.  The rule that guarantees it without any exchange: the first capture happens at the same step count on
    every rank (right after the ``warmup`` eager steps, whatever shape each rank's batch has), and with several
    ranks no further shape is ever captured - a shorter last batch or a ragged batch runs eagerly, which issues the
    same kernels as a replay and needs no barrier.  One rank may capture up to ``max_graphs`` shapes."""
    if known:
        return "replay"
    if eager_steps < warmup:
        return "eager"
    if world > 1:
        return "capture" if (n_graphs == 0 and static) else "eager"
    if n_graphs >= max_graphs and not static:
        return "eager"
    return "capture"


def _with_next(it):
    """(item, following item or None) for every item of ``it``."""
    prev = _with_next        # sentinel
    for b in it:
        if prev is not _with_next:
            yield prev, b
        prev = b
    if prev is not _with_next:
        yield prev, None


class _GraphPair:
    """Two captures of the same step that take turns.  Each has its own static input buffers, so the inputs of the
    next step land (on the copy stream) while the previous replay still reads the other set."""

    def __init__(self):
        self.graphs: List[Any] = []
        self.leaves: List[List[torch.Tensor]] = []
        self.loss: List[torch.Tensor] = []
        self.done = [torch.cuda.Event(), torch.cuda.Event()]        # replay that last read set p has finished
        self.copied = [torch.cuda.Event(), torch.cuda.Event()]      # inputs of set p have landed
        self.done_recorded = [False, False]
        for e in self.copied:
            e.record()               # events get their CUDA handle at the first record
        self.turn = 0


_FRONT_IN_GRAPH = ("front pending in a replayed graph",)      # marks a link whose device state holds a run-ahead front


class _GraphRing:
    """Captured steps for callers that name the batch of the FOLLOWING step: three sets of static input buffers
    take turns.  The graph of set i runs the step on set i with the probe-only pull (the front for set i ran in
    the previous graph) and, on a second stream, the pull front for set i+1.  A fourth capture on set 0 does the
    whole pull itself; it starts the ring, and restarts it after anything else touched the tables."""

    SETS = 3

    def __init__(self):
        self.cold = None
        self.cold_loss = None
        self.warm: List[Any] = []
        self.leaves: List[List[torch.Tensor]] = []
        self.loss: List[torch.Tensor] = []
        self.done = [torch.cuda.Event() for _ in range(self.SETS)]       # the graph that ran set i as its step is over
        self.copied = [torch.cuda.Event() for _ in range(self.SETS)]     # inputs of set i have landed
        self.done_recorded = [False] * self.SETS
        for e in self.copied:
            e.record()
        self.sig: List[Any] = [None] * self.SETS                        # which batch (leaf addresses) set i holds
        self.turn = 0
        self.links: List[Any] = []


class _StatusPoll:
    """Looks at the device status words every few steps without stalling: an asynchronous copy into pinned memory
    now, read when the next poll comes round.  A device error therefore surfaces at most two polling periods
    after the step that hit it."""

    def __init__(self, rt, every: int, tables=()):
        self.rt, self.every = rt, max(1, int(every))
        self.tables = [t for t in tables if hasattr(t, "n_rows_dev")]      # GPU shards whose fill level is watched too
        self.host = torch.zeros(8 + len(self.tables), dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False
        self.count = 0

    def tick(self):
        self.count += 1
        if self.count % self.every:
            return
        if self.pending and self.event.query():
            self.pending = False
            code = int(self.host[0])
            if code != 0:
                self.rt.raise_status(code, int(self.host[1]), int(self.host[2]))
            if core.config.table_grow_at > 0:
                for i, t in enumerate(self.tables):       # a shard that is filling up gets a longer slab before it overflows
                    t.maybe_grow(int(self.host[8 + i]), core.config.table_grow_at)
        if not self.pending:
            self.host[:8].copy_(self.rt.status, non_blocking=True)
            for i, t in enumerate(self.tables):
                self.host[8 + i: 9 + i].copy_(t.n_rows_dev, non_blocking=True)
            self.event.record()
            self.pending = True


class Model(nn.Module):
    """Wrap a network that maps a feature dict to logits ``[B, 1]``.

    Either subclass and define ``forward`` or pass ``network=`` (any ``nn.Module``)."""

    def __init__(self, network: Optional[nn.Module] = None, name: str = "model"):
        super().__init__()
        self.network = network
        self.model_name = name
        self.optimizer = None
        self.loss_fn: Optional[Callable] = None
        self.metrics: List[Any] = []
        self.is_loaded_from_checkpoint = False
        self._sums: Optional[torch.Tensor] = None
        self._sums_seen = None       # host copy of ``_sums`` at the last hand-over to the metrics
        self._steps_seen = 0
        self._loss_steps = 0         # steps whose loss went into ``_sums``
        self._auc_bins = 0
        self._host_metrics: List[Any] = []    # metrics that need (labels, predictions) tensors every step
        self._graph = None
        self._graphs: Dict[Any, _GraphPair] = {}     # batch signature -> the two captures of the step
        self._rings: Dict[Any, _GraphRing] = {}      # same, for callers that name the following batch
        self._ring_refused = False
        self._flat_cache = None                      # (batch object, its flattened form) of the batch named as next
        self._fronts_now = ()                        # (layer, next ids) of the step being issued
        self._last_done = None                       # event behind the last replayed step (None after an eager one)
        self._max_graphs = 8
        self._graph_key = None
        self._static_leaves: List[torch.Tensor] = []
        self._static_loss = None
        self._eager_steps = 0
        self._use_graph = False
        self._status_poll: Optional[_StatusPoll] = None
        self.use_fused = True
        self.stop_training = False

    # ------------------------------------------------------------------ construction
    def forward(self, features):
        if self.network is None:
            raise NotImplementedError("subclass Model or pass network=")
        return self.network(features)

    def compile(self, optimizer=None, loss="binary_crossentropy", metrics: Optional[Sequence] = None,
                cuda_graph: Optional[bool] = None, graph_warmup: int = 3):
        """``metrics``: objects with ``update_state / result`` or names.  ``auc, ctr, pctr, copc, loss`` (the classes of
        ``tn.metric``) are fed from sums the loss kernel keeps on the device (no per-step cost).  The Keras names
        ``acc, mse, mae, mape`` and any other metric object get ``update_state(labels, predictions)`` after every
        step; such a model runs its steps without CUDA graphs."""
        rt = core.runtime()
        self.to(rt.device)
        self.optimizer = optimizer
        self.loss_fn = loss
        self.metrics = [_metric.get(m) for m in (metrics or [])]
        fed_by_kernel = not callable(loss)
        self._host_metrics = [m for m in self.metrics if not (fed_by_kernel and getattr(m, "device_backed", False))]
        bins = {m.n for m in self.metrics if isinstance(m, _metric.AUC) and m not in self._host_metrics}
        if len(bins) > 1:
            raise ValueError("all AUC metrics of one model must use the same number of thresholds")
        self._auc_bins = bins.pop() if bins else 0
        self._sums = torch.zeros(4 + 2 * self._auc_bins, dtype=torch.float32, device=rt.device)
        self._sums_seen = None
        self._steps_seen = self._loss_steps = 0
        self._unit_grad = torch.ones((), dtype=torch.float32, device=rt.device)
        # metrics that read every step's predictions on the host cannot run inside a captured step
        self._use_graph = rt.on_gpu and (core.config.cuda_graph if cuda_graph is None else cuda_graph) and not self._host_metrics
        self._graph_warmup = graph_warmup
        if rt.on_gpu:
            tables = {id(l.table): l.table for l in self.sparse_layers() if hasattr(l, "table")}
            self._status_poll = _StatusPoll(rt, core.config.status_poll_steps, tables.values())
            self._copy_stream = torch.cuda.Stream(device=rt.device)
        if optimizer is not None:
            optimizer.attach(self.named_parameters())
            # A model whose first reader of dense weights is an MLP tower names it in ``first_dense_tower``; on
            # several GPUs that tower's first GEMM then waits for the optimizer's weight all-gather and the dense
            # kernel ends without a barrier of its own.
            tower = getattr(self, "first_dense_tower", None)
            if tower is not None and rt.on_gpu and rt.world > 1 and core.config.gate_first_gemm:
                tower().weight_gate = optimizer.table.enable_gate()
            # Several GPUs: the dense step and the sparse push both wait on their peers, so they may only share the
            # GPU if each fits beside the other whatever order the hardware picks.  The push gives up some SMs and
            # the dense kernel takes no more CTAs than those SMs hold; then neither can keep the other from
            # becoming resident and the two run side by side on two streams.  Small arrays (<= 4 M elements) ride
            # on the push kernel instead unless asked otherwise; large ones (a DCN-v2 cross tower: 130 M) are
            # bound by NVLink, which a quarter of the SMs saturates.
            small = optimizer.table.n <= (4 << 20)
            mode = int(core.config.overlap_dense_push)
            self._overlap_dense = bool(rt.on_gpu and rt.world > 1 and self.sparse_layers() and
                                       (mode == 1 or (mode < 0 and not small)))
            if rt.on_gpu and rt.world > 1 and core.config.dense_small_grid > 0 and small:
                optimizer.table.limit_grid(core.config.dense_small_grid)
            if self._overlap_dense:
                dense_sms = 12 if small else int(core.config.overlap_dense_sms)
                optimizer.table.limit_grid_to_sms(dense_sms)
                for layer in self.sparse_layers():
                    for lk in getattr(layer, "links", None) or [layer.link]:
                        lk.push_cta_cap = torch.cuda.get_device_properties(rt.device).multi_processor_count - dense_sms
        return self

    def sparse_layers(self):
        return [m for m in self.modules() if hasattr(m, "backwards") and m is not self]

    # ------------------------------------------------------------------ steps
    def _loss(self, logits, labels):
        if callable(self.loss_fn):
            return self.loss_fn(logits, labels), torch.sigmoid(logits.detach())
        self._loss_steps += 1
        return F.bce_with_logits(logits, labels, self._sums)

    def backwards(self, grads_and_vars=None):
        layers = self.sparse_layers()
        rt = core.runtime()
        if not rt.on_gpu and rt.world > 1:
            # CPU ranks: the gradient records of all embedding layers travel in one round trip
            from ..ops.sparse_table_cpu import CpuSparseLink
            pend = [l for l in layers if getattr(l, "_pending_push", False) and isinstance(getattr(l, "link", None), CpuSparseLink)]
            # with a handful of ranks the dense gradient rides in the same round: everybody sends its gradient to
            # everybody and takes the mean itself (an all-gather; beyond four ranks the all-reduce is the cheaper form)
            dense = None
            if (pend and rt.world <= 4 and self.optimizer is not None and self.optimizer.table.initialized
                    and grads_and_vars is None and not getattr(self, "_dense_exchange_off", False)):
                dense = self.optimizer.table
            if len(pend) > 1 or dense is not None:
                CpuSparseLink.push_many([l.link for l in pend], dense)
                for l in pend:
                    l._pending_push = False
        for layer in layers:
            layer.backwards(grads_and_vars)

    def _cpu_pulls_together(self, features):
        """CPU ranks: run the pulls of all embedding layers of a step with shared round trips (ids of every layer in
        one exchange, rows in a second one) before the forward pass asks for them layer by layer."""
        rt = core.runtime()
        if rt.on_gpu or rt.world == 1 or not isinstance(features, dict):
            return
        from ..ops.sparse_table_cpu import CpuSparseLink
        calls = []
        for layer in self.sparse_layers():
            if hasattr(layer, "stash_pull_args") and isinstance(getattr(layer, "link", None), CpuSparseLink):
                layer.table.set_training(True)
                ids, _, _, labels, label_mod, count = layer.stash_pull_args(features, True)
                calls.append((layer.link, ids, labels, label_mod, count))
        if len(calls) > 1:
            CpuSparseLink.pull_many(calls)

    @staticmethod
    def _front_ahead_on() -> bool:
        rt = core.runtime()
        mode = int(core.config.pull_front_ahead)
        return bool(rt.on_gpu and (mode > 0 or (mode < 0 and rt.world == 1)))

    def _front_layers(self, next_features):
        """(layer, ids) for every sparse layer whose next pull can be started ahead for ``next_features``; empty
        unless ALL trainable sparse layers of the model qualify (a step either runs every front ahead or none)."""
        if next_features is None or not self._front_ahead_on():
            return []
        out = []
        for layer in self.sparse_layers():
            if not getattr(layer, "trainable", True):
                continue
            ids = layer.ids_pulled_for(next_features) if hasattr(layer, "ids_pulled_for") else None
            if ids is None:
                return []
            out.append((layer, ids))
        return out

    def _step_impl(self, features, labels, next_features=None):
        fronts = self._front_layers(next_features) if self.training else []
        for layer, ids in fronts:
            layer.link.next_ids = ids
        object.__setattr__(self, "_fronts_now", fronts)
        loss = self._step_body(features, labels)
        object.__setattr__(self, "_fronts_now", ())
        for layer, _ in fronts:
            lk = layer.link
            lk.next_ids = None
            if lk.front_in_flight:             # join the side stream: the step (and a captured graph) ends after the front
                from ..ops.sparse_table_gpu import front_stream
                torch.cuda.current_stream().wait_stream(front_stream(lk.dev))
                lk.front_in_flight = False
        return loss

    def _step_body(self, features, labels):
        loss = None
        fused = getattr(self, "fused_train_loss", None)
        if fused is not None and not callable(self.loss_fn) and self.use_fused and not self._host_metrics:
            loss = fused(features, labels, self._sums)      # model-specific fused kernels, when the batch qualifies
            if loss is not None:
                self._loss_steps += 1
        if loss is None:
            with phase("tn.forward"):
                if self.training:
                    self._cpu_pulls_together(features)
                logits = self(features)
                loss, pred = self._loss(logits, labels)
            for m in self._host_metrics:
                m.update_state(labels, pred)
        rt = core.runtime()
        for layer, _ in self._fronts_now:          # forward pass issued: the next batch's pull fronts start here
            layer.link.fork_front()
        with phase("tn.backward"):
            if rt.on_gpu and loss.dim() == 0 and loss.dtype == torch.float32:
                loss.backward(self._unit_grad)      # a resident 1.0: autograd would otherwise launch a fill kernel for it
            else:
                loss.backward()
        if rt.on_gpu and rt.world == 1 and self.optimizer is not None:
            # one GPU: the sparse push and the dense update touch disjoint state and neither waits on other
            # CTAs, so they run side by side
            main = torch.cuda.current_stream()
            side = F._side_stream(rt.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                self.backwards()
            self.optimizer.step()
            main.wait_stream(side)
        elif rt.on_gpu and self.optimizer is not None and getattr(self, "_overlap_dense", False):
            main = torch.cuda.current_stream()
            side = F._side_stream(rt.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                self.optimizer.step()
            self.backwards()
            main.wait_stream(side)
        else:
            # Several GPUs.  Small dense arrays ride on the last sparse push: a few CTAs of that kernel run the dense
            # step while the rest exchange gradient records, so the step waits for its peers once, not twice.
            rider = None
            if (rt.on_gpu and self.optimizer is not None and core.config.dense_rides_push and
                    self.optimizer.table.initialized and self.optimizer.table.n <= (4 << 20)):
                pending = [l for l in self.sparse_layers() if getattr(l, "_pending_push", False)]
                if pending:
                    rider = (getattr(pending[-1], "links", None) or [pending[-1].link])[-1]
                    self.optimizer.table.set_lr(self.optimizer._lr())
                    rider.dense_rider = self.optimizer.table
            # Otherwise push first.  A push kernel only completes after every peer has shipped its gradient records,
            # i.e. after every peer's backward pass, so the dense kernel behind it needs no opening barrier.
            before = rt.peer_synced_pushes
            self.backwards()
            if self.optimizer is not None:
                if rider is not None and rider.dense_rider is None:      # the push took it along
                    self.optimizer.iterations += 1
                    self.optimizer.table.step_count += 1
                else:
                    if rider is not None:
                        rider.dense_rider = None
                    self.optimizer.step(peers_past_backward=rt.peer_synced_pushes > before)
        return loss.detach()

    def _to_device(self, obj):
        dev = core.runtime().device
        leaves: List[torch.Tensor] = []
        spec = _flatten(obj, leaves)
        moved = [t.to(dev, non_blocking=True) for t in leaves]
        return _unflatten(spec, iter(moved)), spec, leaves

    def _eager_step(self, features, labels):
        self._last_done = None
        (f, y), _, _ = self._to_device((features, labels))
        return self._step_impl(f, y)

    def train_step(self, data, next_data=None):
        """One optimisation step on ``data = (features, labels)``; returns the loss (device tensor).

        ``next_data``: the batch that will be passed as ``data`` at the next call (same tensors, unchanged).  On the
        captured path its sparse ids are deduplicated and sent to their owners on a second stream while this step
        runs, so the next step's pull only probes and returns rows.  ``fit`` passes it by itself."""
        if next_data is not None and self._use_graph and self._front_ahead_on():
            loss = self._ring_step(data, next_data)
            if loss is not None:
                return loss
        features, labels = data
        if not self.training:
            self.train()
        if self._status_poll is not None:
            self._status_poll.tick()
        if not self._use_graph:
            return self._eager_step(features, labels)
        rt = core.runtime()
        leaves: List[torch.Tensor] = []
        spec = _flatten((features, labels), leaves)
        key = (spec, tuple((t.shape, t.dtype) for t in leaves))
        what = graph_decision(rt.world, key in self._graphs, _is_static(spec), len(self._graphs) + len(self._rings), self._max_graphs,
                              self._eager_steps, self._graph_warmup)
        if what == "eager":
            self._eager_steps += 1
            loss = self._eager_step(features, labels)
            if self._eager_steps <= self._graph_warmup:
                rt.check_status()      # surface device-side errors before the step is frozen into a graph
            return loss
        if what == "capture":
            if _is_static(spec):
                self._capture(spec, leaves, key)
            else:
                try:
                    self._capture(spec, leaves, key)
                except Exception:           # an op of the ragged path that cannot be captured: stay eager for good
                    torch.cuda.synchronize()
                    self._max_graphs = 0
                    self._graphs.clear()
                    return self._eager_step(features, labels)
        gp = self._graphs[key]
        p = gp.turn
        gp.turn ^= 1
        main = torch.cuda.current_stream()
        if any(t.is_cuda for t in leaves):
            # inputs produced on the device come with the stream order of whatever produced them
            torch._foreach_copy_(gp.leaves[p], [t if t.is_cuda else t.to(rt.device, non_blocking=True) for t in leaves])
        elif core.config.native_step_path and all(t.is_contiguous() for t in leaves):
            # one native call: copy stream waits for the replay that last read this input set, the leaves go host ->
            # device, their arrival is recorded and the compute stream waits for it
            self._ext.stage_inputs(gp.leaves[p], leaves, self._copy_stream.cuda_stream, main.cuda_stream,
                                   gp.done[p].cuda_event if gp.done_recorded[p] else 0, gp.copied[p].cuda_event, 0)
        else:
            copy = self._copy_stream
            copy.wait_event(gp.done[p])          # the replay that last read this input set is over
            with torch.cuda.stream(copy):
                for dst, src in zip(gp.leaves[p], leaves):
                    dst.copy_(src, non_blocking=True)
                gp.copied[p].record(copy)
            main.wait_event(gp.copied[p])
        if self.optimizer is not None:
            self.optimizer.table.set_lr(self.optimizer._lr())
        gp.graphs[p].replay()
        gp.done[p].record(main)
        gp.done_recorded[p] = True
        self._last_done = gp.done[p]
        if self.optimizer is not None:
            self.optimizer.iterations += 1
            self.optimizer.table.step_count += 1
        self._loss_steps += self._graph_loss_steps
        self._graph, self._graph_key, self._static_leaves, self._static_loss = gp.graphs[p], key, gp.leaves[p], gp.loss[p]
        return gp.loss[p]

    # ---- captured steps with the next batch's pull front run ahead -------------------------------------------
    @staticmethod
    def _sig(leaves):
        return tuple((t.data_ptr(), tuple(t.shape)) for t in leaves)

    def _stage(self, ring, i, leaves, sig, main):
        """Inputs ``leaves`` into static set i of the ring (host leaves: native staged copy on the copy stream; device
        leaves: one foreach copy in stream order)."""
        if any(t.is_cuda for t in leaves):
            dev = core.runtime().device
            torch._foreach_copy_(ring.leaves[i], [t if t.is_cuda else t.to(dev, non_blocking=True) for t in leaves])
        else:
            srcs = [t if t.is_contiguous() else t.contiguous() for t in leaves]
            self._ext.stage_inputs(ring.leaves[i], srcs, self._copy_stream.cuda_stream, main.cuda_stream,
                                   ring.done[i].cuda_event if ring.done_recorded[i] else 0, ring.copied[i].cuda_event,
                                   0)
        ring.sig[i] = sig

    def _flat(self, batch):
        """(spec, leaves, shapes, addresses) of a batch; the batch named as ``next_data`` at the previous call is
        looked up instead of being walked again."""
        c = self._flat_cache
        if c is not None and c[0] is batch:
            return c[1]
        leaves: List[torch.Tensor] = []
        spec = _flatten(batch, leaves)
        return spec, leaves, tuple((t.shape, t.dtype) for t in leaves), self._sig(leaves)

    def _ring_step(self, data, next_data):
        """The step through the three-set ring, or None when this batch does not take that path."""
        setattr_ = object.__setattr__          # plain attributes: nn.Module's bookkeeping costs microseconds per write
        spec, leaves, shapes, sig = self._flat(data)
        if not _is_static(spec):
            return None
        nflat = self._flat(next_data)
        nspec, nleaves, nshapes, nsig = nflat
        if nspec != spec or nshapes != shapes:
            return None          # the following batch has another shape (a shorter last batch): no run-ahead for it
        setattr_(self, "_flat_cache", (next_data, nflat))
        key = (spec, shapes)
        ring = self._rings.get(key)
        if ring is None:
            if self._rings or self._ring_refused or self._eager_steps < self._graph_warmup or key in self._graphs:
                return None      # one ring per model, captured right after the warm-up steps on every rank alike
            if not self.training:
                self.train()
            ring = self._capture_ring(spec, leaves, nleaves, key)
            if ring is None:
                self._ring_refused = True
                return None
        if not self.training:
            self.train()
        if self._status_poll is not None:
            self._status_poll.tick()
        main = torch.cuda.current_stream()
        cur = ring.turn
        warm = ring.sig[cur] == sig and all(lk._front is _FRONT_IN_GRAPH for lk in ring.links)
        if not warm:
            # (re)start: whatever front is pending belongs to another batch
            for lk in ring.links:
                if lk._front is not None:
                    lk.discard_front()
            cur = ring.turn = 0
            self._stage(ring, 0, leaves, sig, main)
        nxt = (cur + 1) % ring.SETS
        self._stage(ring, nxt, nleaves, nsig, main)
        opt = self.optimizer
        if opt is not None:
            opt.table.set_lr(opt._lr())
        graph = ring.warm[cur] if warm else ring.cold
        graph.replay()
        ring.done[cur].record(main)
        ring.done_recorded[cur] = True
        for lk in ring.links:
            lk._front = _FRONT_IN_GRAPH
        ring.turn = nxt
        if opt is not None:
            opt.iterations += 1
            opt.table.step_count += 1
        loss = ring.loss[cur] if warm else ring.cold_loss
        setattr_(self, "_loss_steps", self._loss_steps + self._graph_loss_steps)
        setattr_(self, "_graph", graph)
        setattr_(self, "_graph_key", key)
        setattr_(self, "_static_leaves", ring.leaves[cur])
        setattr_(self, "_static_loss", loss)
        setattr_(self, "_last_done", ring.done[cur])
        return loss

    def _capture_ring(self, spec, leaves, nleaves, key):
        """Capture the cold graph (set 0, whole pull) and the three warm graphs; None when the model's sparse layers
        cannot start their pulls ahead for this kind of batch."""
        rt = core.runtime()
        dev = rt.device
        from .. import _build
        ext = self._ext = _build.cuda_ext()
        ring = _GraphRing()
        for i in range(ring.SETS):
            src = nleaves if i == 1 else leaves
            st = [torch.empty(t.shape, dtype=t.dtype, device=dev) for t in src]
            for d, h in zip(st, src):
                d.copy_(h, non_blocking=True)
            ring.leaves.append(st)
        feats = [_unflatten(spec, iter(st)) for st in ring.leaves]
        fronts = self._front_layers(feats[1][0])
        if not fronts:
            return None
        ring.links = [layer.link for layer, _ in fronts]
        for lk in ring.links:
            if lk._front is not None:
                lk.discard_front()
        hits0 = {id(lk): lk.front_hits for lk in ring.links}
        iters = self.optimizer.iterations if self.optimizer is not None else 0
        steps0 = self.optimizer.table.step_count if self.optimizer is not None else 0
        loss_steps0 = self._loss_steps
        pool = None
        order = [(0, True), (1, False), (2, False), (0, False)]          # (set, cold): every warm capture follows the
        ring.warm = [None] * ring.SETS                                    # capture that ran the front for its set
        ring.loss = [None] * ring.SETS
        for i, cold in order:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            c0 = ext.launch_count()
            f, y = feats[i]
            with torch.cuda.graph(g, pool=pool):
                static_loss = self._step_impl(f, y, next_features=feats[(i + 1) % ring.SETS][0])
            if pool is None:
                self._launches_per_step = ext.launch_count() - c0
                self._graph_loss_steps = self._loss_steps - loss_steps0
                pool = g.pool()
            if cold:
                ring.cold, ring.cold_loss = g, static_loss
            else:
                ring.warm[i], ring.loss[i] = g, static_loss
        if self.optimizer is not None:      # capture only records work, it does not run a step
            self.optimizer.iterations = iters
            self.optimizer.table.step_count = steps0
        self._loss_steps = loss_steps0
        for lk in ring.links:
            lk._front = None                # nothing ran: no front is pending on the device
        if any(lk.front_hits - hits0[id(lk)] < ring.SETS for lk in ring.links):
            # a layer whose front ran but whose pull never came in the step (an embedding the forward pass does not
            # use): its fronts would pile up unconsumed; such a model keeps the one-kernel pull
            rt.barrier()
            return None
        self._rings[key] = ring
        rt.barrier()                        # captures take a different time on every rank; line the ranks up again
        return ring

    def _capture(self, spec, leaves, key):
        """Capture the step twice (two sets of static inputs that take turns) into one memory pool."""
        dev = core.runtime().device
        gp = _GraphPair()
        from .. import _build
        ext = self._ext = _build.cuda_ext()
        for layer in self.sparse_layers():      # a pull front that ran ahead for another batch must not leak into the capture
            lk = getattr(layer, "link", None)
            if lk is not None and getattr(lk, "_front", None) is not None:
                lk.discard_front()
        iters = self.optimizer.iterations if self.optimizer is not None else 0
        steps0 = self.optimizer.table.step_count if self.optimizer is not None else 0
        loss_steps0 = self._loss_steps
        pool = None
        for p in range(2):
            static_leaves = [torch.empty(t.shape, dtype=t.dtype, device=dev) for t in leaves]
            for dst, src in zip(static_leaves, leaves):
                dst.copy_(src, non_blocking=True)
            f, y = _unflatten(spec, iter(static_leaves))
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            c0 = ext.launch_count()
            with torch.cuda.graph(g, pool=pool):
                static_loss = self._step_impl(f, y)
            if p == 0:
                self._launches_per_step = ext.launch_count() - c0
                self._graph_loss_steps = self._loss_steps - loss_steps0
                pool = g.pool()
            gp.graphs.append(g)
            gp.leaves.append(static_leaves)
            gp.loss.append(static_loss)
        if self.optimizer is not None:      # capture only records work, it does not run a step
            self.optimizer.iterations = iters
            self.optimizer.table.step_count = steps0
        self._loss_steps = loss_steps0
        if len(self._graphs) >= self._max_graphs:          # static shapes beyond the cap replace the oldest capture
            self._graphs.pop(next(iter(self._graphs)))
        self._graphs[key] = gp
        # Capture takes a different time on every rank; the first replay's kernels wait for their peers on the
        # device with a finite budget, so line the ranks up on the host first.
        core.runtime().barrier()

    def train_on_batch(self, x, y=None, return_dict: bool = False, next_batch=None):
        """One training step.  ``next_batch = (x, y)`` of the following call, when known, lets the captured step start
        that batch's sparse pull ahead (see :meth:`train_step`)."""
        with start_as_current_span("train_on_batch"):
            loss = self.train_step((x, y), next_batch)
        return {"loss": loss} if return_dict else loss

    def test_step(self, data):
        """Forward pass and loss on one batch without touching any parameter; the loss kernel adds the batch to the
        metric sums.  Returns ``(loss, predictions)`` (tensornet/model/Model.py:117-124 is the predict twin)."""
        features, labels = data
        self.eval()
        with torch.no_grad():
            (f, y), _, _ = self._to_device((features, labels))
            logits = self(f)
            loss, pred = self._loss(logits, y)
            for m in self._host_metrics:
                m.update_state(y, pred)
        return loss, pred

    def predict_step(self, data):
        """Returns ``(y, y_pred)`` like the reference (tensornet/model/Model.py:117-124)."""
        features, labels = data if isinstance(data, (tuple, list)) and len(data) == 2 else (data, None)
        self.eval()
        with torch.no_grad():
            (f, y), _, _ = self._to_device((features, labels))
            pred = torch.sigmoid(self(f))
        return y, pred

    def predict_on_batch(self, x):
        with start_as_current_span("predict_on_batch"):
            return self.predict_step((x, None))[1]

    def predict(self, dataset: Iterable, steps: Optional[int] = None, callbacks: Sequence = (), verbose: int = 0):
        """``(labels, predictions)`` over ``dataset``.  ``callbacks`` get ``on_predict_begin`` (where
        ``PsWeightCheckpoint`` loads the checkpoint and re-arms the balanced dataset) and ``on_predict_end``
        (tensornet/model/Model.py:79-81, tensornet/callbacks/callbacks.py:78-84).  ``verbose``: rank 0 prints the
        number of batches scored when the pass ends (the reference's example passes ``verbose=1``)."""
        with start_as_current_span("predict"):
            for cb in callbacks:
                cb.set_model(self)
                cb.on_predict_begin()
            ys, ps = [], []
            for i, batch in enumerate(dataset):
                if steps is not None and i >= steps:
                    break
                y, p = self.predict_step(batch)
                ps.append(p.cpu())
                if y is not None:
                    ys.append(y.cpu())
            core.runtime().check_status()
            for cb in callbacks:
                cb.on_predict_end()
            if verbose and core.runtime().rank == 0:
                print(f"predict: {len(ps)} batches", flush=True)
            return (torch.cat(ys) if ys else None), (torch.cat(ps) if ps else None)

    def evaluate(self, dataset: Iterable, steps: Optional[int] = None, callbacks: Sequence = (), return_dict: bool = True,
                 verbose: int = 0):
        """Loss and every compiled metric over ``dataset`` with the parameters left untouched (rows of unseen signs
        are created as zeros, as in the reference's inference mode).  ``callbacks`` get ``on_test_begin`` /
        ``on_test_end`` (tensornet/callbacks/callbacks.py:86-91).  Metric state is reset first, as Keras does."""
        with start_as_current_span("evaluate"):
            for cb in callbacks:
                cb.set_model(self)
                cb.on_test_begin()
            self.reset_metrics()
            total, n = 0.0, 0
            losses = []
            for i, batch in enumerate(dataset):
                if steps is not None and i >= steps:
                    break
                loss, _ = self.test_step(batch)
                losses.append(loss.detach())
                n += 1
            if losses:
                total = float(torch.stack([l.float().reshape(()) for l in losses]).sum())
            core.runtime().check_status()
            out = {"loss": total / n if n else float("nan")}
            out.update(self.metric_results())
            for cb in callbacks:
                cb.on_test_end(out)
            if verbose and core.runtime().rank == 0:
                print("evaluate: " + " ".join(f"{k} {v:.5f}" for k, v in out.items()), flush=True)
            return out if return_dict else [out["loss"]] + [out[m.name] for m in self.metrics]

    def _prefetched(self, dataset: Iterable):
        """Yield the batches of ``dataset`` already on the device: batch k+1 is copied host -> device on a second
        stream while step k runs (pinned host tensors make the copy asynchronous)."""
        rt = core.runtime()
        if not rt.on_gpu:
            yield from dataset
            return
        main = torch.cuda.current_stream()
        copy = self._copy_stream = getattr(self, "_copy_stream", None) or torch.cuda.Stream(device=rt.device)

        def stage(batch):
            leaves: List[torch.Tensor] = []
            spec = _flatten(batch, leaves)
            with torch.cuda.stream(copy):
                moved = [t.to(rt.device, non_blocking=True) for t in leaves]
                ev = torch.cuda.Event()
                ev.record(copy)
            for t in moved:
                t.record_stream(main)
            return _unflatten(spec, iter(moved)), ev

        it = iter(dataset)
        try:
            nxt = stage(next(it))
        except StopIteration:
            return
        while nxt is not None:
            cur, ev = nxt
            try:
                nxt = stage(next(it))
            except StopIteration:
                nxt = None
            main.wait_event(ev)
            yield cur

    def _batch_source(self, dataset: Iterable, prefetch: bool):
        """Batches for ``fit``.  Static batches on the graph path go to ``train_step`` as they are (it copies them into
        the idle input set itself, overlapped with the running step); everything else is staged one batch ahead."""
        if not (prefetch and core.runtime().on_gpu):
            return dataset
        if not self._use_graph:
            return self._prefetched(dataset)
        it = iter(dataset)
        try:
            first = next(it)
        except StopIteration:
            return iter(())
        import itertools
        rest = itertools.chain([first], it)
        return rest if _is_static(_flatten(first, [])) else self._prefetched(rest)

    def fit(self, dataset: Iterable, epochs: int = 1, steps_per_epoch: Optional[int] = None, callbacks: Sequence = (),
            verbose: int = 0, log_every: int = 100, prefetch: bool = True, record_step_loss: bool = False):
        """Iterate ``dataset`` (yielding ``(features, labels)``) for ``epochs`` passes.

        ``prefetch``: copy the next batch to the device on a second stream while the current step runs.
        ``record_step_loss``: read every step's loss back to the host (``history["step_loss"]``); the 4-byte copy
        of step k is issued right behind the step into a ring of pinned slots and collected when it has arrived, so
        the host may run a few steps ahead of the device and a late rank's hiccup does not stall the others.
        The history carries the loss of the last step of every pass and, per compiled metric, its value at the
        end of every pass (metric state is reset when a pass begins, as Keras does)."""
        with start_as_current_span("fit"):
            history: Dict[str, list] = {"loss": []}
            for m in self.metrics:
                history[m.name] = []
            if record_step_loss:
                history["step_loss"] = []
            rt = core.runtime()
            gpu = rt.on_gpu
            pinned = None
            if gpu and record_step_loss:
                if getattr(self, "_pinned_loss", None) is None:      # page-locked allocation is slow: once per model
                    self._pinned_loss = torch.zeros(_LOSS_RING, dtype=torch.float32).pin_memory()
                    self._loss_events = [torch.cuda.Event() for _ in range(_LOSS_RING)]
                    for e in self._loss_events:
                        e.record()           # events get their CUDA handle at the first record
                    from .. import _build
                    self._ext = _build.cuda_ext()
                    self._read_stream = torch.cuda.Stream(device=rt.device)
                pinned = self._pinned_loss
                events = self._loss_events
            for cb in callbacks:
                cb.set_model(self)
                cb.on_train_begin()
            batch_cbs = [cb for cb in callbacks if hasattr(cb, "on_train_batch_end")]
            for epoch in range(epochs):
                for cb in callbacks:
                    cb.on_epoch_begin(epoch)
                if self.metrics:
                    self.reset_metrics()
                last = None
                issued = collected = 0       # losses copied to / read from the pinned ring (the host runs up to _LOSS_RING - 1 steps ahead)
                ahead = gpu and self._use_graph and self._front_ahead_on()
                source = self._batch_source(dataset, prefetch)
                if steps_per_epoch is not None:
                    import itertools
                    source = itertools.islice(source, int(steps_per_epoch))      # the look-ahead stays inside the pass
                for i, (batch, nxt) in enumerate(_with_next(source)):
                    # the last batch of a pass names itself as its successor: the step stays on the same captured path
                    last = self.train_step(batch, (nxt if nxt is not None else batch) if ahead else None)
                    if record_step_loss:
                        if pinned is None:
                            history["step_loss"].append(float(last))
                        else:
                            slot = issued % _LOSS_RING
                            if core.config.native_step_path and last.dtype == torch.float32 and last.numel() == 1:
                                if self._last_done is not None:
                                    # behind the step's end event on a stream of its own: the compute stream
                                    # carries nothing between two replayed steps
                                    self._ext.read_scalar_async(pinned, slot, last, self._read_stream.cuda_stream,
                                                                events[slot].cuda_event, self._last_done.cuda_event)
                                else:
                                    self._ext.read_scalar_async(pinned, slot, last, torch.cuda.current_stream().cuda_stream,
                                                                events[slot].cuda_event, 0)
                            else:
                                pinned[slot: slot + 1].copy_(last.detach().reshape(1), non_blocking=True)
                                events[slot].record()
                            issued += 1
                            # read back what has arrived; wait only when the ring is about to wrap
                            while collected < issued and (issued - collected >= _LOSS_RING or events[collected % _LOSS_RING].query()):
                                events[collected % _LOSS_RING].synchronize()
                                history["step_loss"].append(float(pinned[collected % _LOSS_RING]))
                                collected += 1
                    for cb in batch_cbs:
                        cb.on_train_batch_end(i, {"batch": int(batch[1].shape[0]) if torch.is_tensor(batch[1]) else 0})
                    if verbose and (i + 1) % log_every == 0:
                        print(f"epoch {epoch} step {i + 1} loss {float(last):.5f}", flush=True)
                    if self.stop_training:
                        break
                while pinned is not None and collected < issued:
                    events[collected % _LOSS_RING].synchronize()
                    history["step_loss"].append(float(pinned[collected % _LOSS_RING]))
                    collected += 1
                core.runtime().check_status()
                if core.config.verify_guards_each_pass:
                    verify_all_arenas()
                history["loss"].append(float(last) if last is not None else float("nan"))
                logs = {"loss": history["loss"][-1]}
                if self.metrics:
                    logs.update(self.metric_results())
                    for m in self.metrics:
                        history[m.name].append(logs[m.name])
                for cb in callbacks:
                    cb.on_epoch_end(epoch, logs)
            for cb in callbacks:
                cb.on_train_end()
            return history

    # ------------------------------------------------------------------ metrics
    def _read_sums(self):
        """Host copy of the device accumulators: (four sums as float64, histogram counts as int64 or None)."""
        if self._sums is None:
            return torch.zeros(4, dtype=torch.float64), None
        host = self._sums.detach().cpu()
        hist = host[4:].view(torch.int32).to(torch.int64) & 0xFFFFFFFF if self._auc_bins else None
        return host[:4].double(), hist

    def _feed_metrics(self):
        """Hand the compiled metrics what the loss kernels accumulated since the last hand-over (one small read)."""
        fed = [m for m in self.metrics if m not in self._host_metrics]
        if not fed or self._sums is None:
            return
        sums, hist = self._read_sums()
        if self._sums_seen is None:
            prev_s, prev_h = torch.zeros(4, dtype=torch.float64), (torch.zeros_like(hist) if hist is not None else None)
        else:
            prev_s, prev_h = self._sums_seen
        d = sums - prev_s
        pos = neg = None
        if hist is not None:
            dh = (hist - prev_h) & 0xFFFFFFFF            # 32-bit counters wrap; differences stay exact
            pos, neg = dh[: self._auc_bins].double(), dh[self._auc_bins:].double()
        stats = _metric.BatchStats(float(d[0]), float(d[1]), float(d[2]), float(d[3]), self._loss_steps - self._steps_seen, pos, neg)
        self._sums_seen = (sums, hist)
        self._steps_seen = self._loss_steps
        if stats.count > 0:
            for m in fed:
                m.feed(stats)

    def metric_results(self) -> Dict[str, float]:
        """Current value of every compiled metric, by name."""
        self._feed_metrics()
        return {m.name: float(m.result()) for m in self.metrics}

    def metric_sums(self) -> Dict[str, float]:
        """Running loss / CTR / PCTR / COPC since the last reset."""
        s = self._sums[:4].tolist() if self._sums is not None else [0, 0, 0, 0]
        n = max(s[3], 1.0)
        return {"loss_sum": s[0], "ctr": s[1] / n, "pctr": s[2] / n, "copc": s[1] / max(s[2], 1e-12), "count": s[3]}

    def reset_metrics(self):
        if self._sums is not None:
            self._sums.zero_()
        self._sums_seen = None
        self._steps_seen = self._loss_steps
        for m in self.metrics:
            m.reset_state()

    # ------------------------------------------------------------------ checkpoints
    def _tn_children(self):
        from ..layers.embedding_features import EmbeddingFeatures

        seen_tables = set()
        for m in self.modules():
            if m is self:
                continue
            if isinstance(m, EmbeddingFeatures) or hasattr(m, "save_sparse_table"):
                h = getattr(m, "sparse_table_handle", None)
                if h in seen_tables:      # shared tables are written once
                    continue
                seen_tables.add(h)
                yield "sparse", m
            elif hasattr(m, "save_bn_table"):
                yield "bn", m

    def save(self, filepath: str) -> str:
        """Export the dense part for serving: ``<filepath>/sub_model.pt`` holds the ``state_dict`` of ``self.sub_model``
        (of the whole module when there is no such attribute).  The role of ``sub_model.save(...)`` in the reference's
        driver (examples/main.py:100-104), which writes a TensorFlow SavedModel; the sparse part is exported separately
        (``tn.serving.export_sparse_dictionary``).  Rank 0 writes; every rank returns the file's path."""
        rt = core.runtime()
        path = os.path.join(filepath, "sub_model.pt")
        if rt.rank == 0:
            os.makedirs(filepath, exist_ok=True)
            module = getattr(self, "sub_model", None) or self
            torch.save({k: v.detach().cpu() for k, v in module.state_dict().items()}, path)
        core.barrier()
        return path

    def save_weights(self, filepath: str, dt: str = "", mode: str = "txt", **kwargs):
        """<filepath>/<dt>/{sparse_table,dense_table,bn_table,torch_checkpoint.pt}; ``_checkpoint`` last."""
        rt = core.runtime()
        rt.check_status()         # nor one from a step that a device-side error cut short
        verify_all_arenas()       # never write a checkpoint from memory a stray peer store has damaged
        cp_dir = os.path.join(filepath, dt) if dt else filepath
        if rt.rank == 0:
            os.makedirs(cp_dir, exist_ok=True)
        core.barrier()
        for kind, m in self._tn_children():
            if kind == "sparse":
                m.save_sparse_table(cp_dir, mode)
            elif rt.rank == 0:
                m.save_bn_table(cp_dir)
        if self.optimizer is not None and self.optimizer.table.initialized:
            self.optimizer.save_dense_table(cp_dir)
        core.barrier()
        if rt.rank == 0:
            torch.save({k: v.detach().cpu() for k, v in self.state_dict().items()}, os.path.join(cp_dir, "torch_checkpoint.pt"))
            save_done_info(filepath, dt)
        core.barrier()

    def _resolve_cp_dir(self, filepath: str, include_dt: bool):
        if include_dt:
            return filepath if os.path.isdir(filepath) else None
        info = load_done_info(filepath)
        if not info:
            return None
        return os.path.join(filepath, info["dt"]) if info.get("dt") else filepath

    def load_weights(self, filepath: str, include_dt: bool = False, mode: str = "txt", **kwargs):
        cp_dir = self._resolve_cp_dir(filepath, include_dt)
        if cp_dir is None:
            return False      # nothing trained yet: silent no-op like the reference (Model.py:179-181)
        if not self.is_loaded_from_checkpoint:
            self._load_tn(cp_dir, mode, dense=True)
            self.is_loaded_from_checkpoint = True
        return True

    def load_sparse_weights(self, filepath: str, include_dt: bool = False, mode: str = "txt", **kwargs):
        cp_dir = self._resolve_cp_dir(filepath, include_dt)
        if cp_dir is None:
            return False
        self._load_tn(cp_dir, mode, dense=False)
        return True

    def _load_tn(self, cp_dir: str, mode: str, dense: bool):
        for kind, m in self._tn_children():
            if kind == "sparse":
                m.load_sparse_table(cp_dir, mode)
            else:
                m.load_bn_table(cp_dir)
        if dense and self.optimizer is not None:
            if not self.optimizer.table.initialized:
                self.optimizer.attach(self.named_parameters())
            self.optimizer.load_dense_table(cp_dir)
        # the dense table file is text with 6 significant digits (as in the reference); the exact
        # fp32 weights and buffers come from the framework checkpoint written next to it
        pt = os.path.join(cp_dir, "torch_checkpoint.pt")
        if os.path.exists(pt):
            sd = torch.load(pt, map_location="cpu")
            with torch.no_grad():
                own = self.state_dict()
                for k, v in sd.items():
                    if k in own and own[k].shape == v.shape:
                        own[k].copy_(v)
            if self.optimizer is not None and self.optimizer.table.initialized:
                self.optimizer.table.refresh_shadow()
        core.barrier()

    def show_decay(self, delta_days: int = 0):
        for kind, m in self._tn_children():
            if kind == "sparse":
                m.show_decay(delta_days)

    def evict_sparse_rows(self) -> int:
        """Drop from the live tables the rows that the optimizer's save-time rule would not write to a checkpoint
        (the reference applies that rule only while saving, core/ps/optimizer/optimizer_kernel.h:331-334; a long job
        on fixed HBM wants the memory back as well).  Call between steps; returns the number of rows dropped here."""
        n = 0
        for kind, m in self._tn_children():
            if kind == "sparse" and hasattr(m.table, "evict"):
                n += m.table.evict()
        return n


class PCGradModel(Model):
    """Multi-task variant: ``forward`` returns one logit column per task; every task loss is
    back-propagated separately and the dense gradients are combined by PCGrad
    (tensornet/model/Model.py:259-293, tensornet/model/compile_utils.py:55-126)."""

    _dense_exchange_off = True      # the projected gradient is written after the sparse pushes: it travels by itself

    def _front_layers(self, next_features):
        return []          # this step runs several backward passes per pull; it does not start pulls ahead

    def _step_impl(self, features, labels, next_features=None):
        from ..optimizer import PCGrad

        logits = self(features)
        n_task = logits.shape[1]
        labels = labels.reshape(logits.shape[0], -1).float()
        losses = [torch.nn.functional.binary_cross_entropy_with_logits(logits[:, k], labels[:, min(k, labels.shape[1] - 1)])
                  for k in range(n_task)]
        if isinstance(self.optimizer, PCGrad):
            self.optimizer.step_multi(losses)
        else:
            torch.stack(losses).sum().backward()
            self.optimizer.step()
        self.backwards()
        return torch.stack(losses).sum().detach()
