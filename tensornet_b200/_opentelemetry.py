"""Optional OpenTelemetry tracing (tensornet/_opentelemetry.py:31-59).

When ``OTEL_EXPORTER_OTLP_TRACES_ENDPOINT`` or ``OTEL_EXPORTER_OTLP_ENDPOINT`` is set and the
OpenTelemetry SDK is importable, spans named after the wrapped call (``fit``, ``predict``,
``train_on_batch``, ``predict_on_batch``) are exported with service name ``tensornet`` and a
``tensornet.version`` resource attribute; a parent trace context is taken from upper-cased
environment variables (``TRACEPARENT`` ...).  Otherwise the context manager does nothing.
On a GPU every span also opens an NVTX range so the phases show up in CUDA timelines.
"""
from __future__ import annotations

import contextlib
import os

_tracer = None
_enabled = False


def _setup():
    global _tracer, _enabled
    if _tracer is not None or _enabled:
        return
    if not (os.environ.get("OTEL_EXPORTER_OTLP_TRACES_ENDPOINT") or os.environ.get("OTEL_EXPORTER_OTLP_ENDPOINT")):
        return
    try:
        from opentelemetry import trace
        from opentelemetry.exporter.otlp.proto.grpc.trace_exporter import OTLPSpanExporter
        from opentelemetry.sdk.resources import Resource
        from opentelemetry.sdk.trace import TracerProvider
        from opentelemetry.sdk.trace.export import BatchSpanProcessor

        from .version import VERSION

        provider = TracerProvider(resource=Resource.create({"service.name": "tensornet", "tensornet.version": VERSION}))
        provider.add_span_processor(BatchSpanProcessor(OTLPSpanExporter()))
        trace.set_tracer_provider(provider)
        _tracer = trace.get_tracer("tensornet")
        _enabled = True
    except Exception:
        _enabled = False


def _parent_context():
    try:
        from opentelemetry.propagate import extract

        carrier = {k.lower(): v for k, v in os.environ.items() if k in ("TRACEPARENT", "TRACESTATE", "BAGGAGE")}
        return extract(carrier)
    except Exception:
        return None


@contextlib.contextmanager
def start_as_current_span(name: str):
    _setup()
    nvtx = None
    try:
        import torch

        if torch.cuda.is_available():
            nvtx = torch.cuda.nvtx
            nvtx.range_push(name)
    except Exception:
        nvtx = None
    try:
        if _enabled and _tracer is not None:
            with _tracer.start_as_current_span(name, context=_parent_context()) as span:
                yield span
        else:
            yield None
    finally:
        if nvtx is not None:
            nvtx.range_pop()


class _NoRange:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_RANGE = _NoRange()


class _NvtxRange:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        import torch

        torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        import torch

        torch.cuda.nvtx.range_pop()
        return False


def phase(name: str):
    """NVTX range around one phase of a training step (sparse pull, forward, backward, sparse push, dense step) when
    ``TN_NVTX_PHASES=1``; a no-op object otherwise, so the hot loop pays one attribute test.  The ranges show in a
    timeline of the eager steps (the first steps of a run, ``cuda_graph=False``, or ``ProfileBatches``); a replayed
    CUDA graph is one launch and has no host-side phases."""
    from .core import config

    if not config.nvtx_phases:
        return _NO_RANGE
    import torch

    return _NvtxRange(name) if torch.cuda.is_available() else _NO_RANGE
