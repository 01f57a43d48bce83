"""The optional OpenTelemetry shim (tensornet/_opentelemetry.py:31-59): silent without an endpoint, and with one it
configures the SDK once (service name, version attribute), names spans after the wrapped call and hands the parent
context from TRACEPARENT to the tracer.  A stand-in SDK is injected; nothing is exported anywhere."""
import contextlib
import sys
import types

import pytest

import tensornet_b200._opentelemetry as otel


class _FakeSdk:
    def __init__(self):
        self.spans, self.resources, self.extracted = [], [], []
        sdk = self

        class Tracer:
            @contextlib.contextmanager
            def start_as_current_span(self, name, context=None):
                sdk.spans.append((name, context))
                yield name

        class Provider:
            def __init__(self, resource=None):
                sdk.resources.append(resource)

            def add_span_processor(self, p):
                pass

        def mod(name, **attrs):
            m = types.ModuleType(name)
            m.__dict__.update(attrs)
            return m

        self.modules = {
            "opentelemetry": mod("opentelemetry"),
            "opentelemetry.trace": mod("opentelemetry.trace", set_tracer_provider=lambda p: None, get_tracer=lambda n: Tracer()),
            "opentelemetry.exporter": mod("opentelemetry.exporter"),
            "opentelemetry.exporter.otlp": mod("opentelemetry.exporter.otlp"),
            "opentelemetry.exporter.otlp.proto": mod("opentelemetry.exporter.otlp.proto"),
            "opentelemetry.exporter.otlp.proto.grpc": mod("opentelemetry.exporter.otlp.proto.grpc"),
            "opentelemetry.exporter.otlp.proto.grpc.trace_exporter": mod("opentelemetry.exporter.otlp.proto.grpc.trace_exporter",
                                                                         OTLPSpanExporter=lambda: object()),
            "opentelemetry.sdk": mod("opentelemetry.sdk"),
            "opentelemetry.sdk.resources": mod("opentelemetry.sdk.resources",
                                               Resource=types.SimpleNamespace(create=lambda attrs: dict(attrs))),
            "opentelemetry.sdk.trace": mod("opentelemetry.sdk.trace", TracerProvider=Provider),
            "opentelemetry.sdk.trace.export": mod("opentelemetry.sdk.trace.export", BatchSpanProcessor=lambda e: object()),
            "opentelemetry.propagate": mod("opentelemetry.propagate", extract=lambda c: sdk.extracted.append(dict(c)) or ("ctx", dict(c))),
        }
        self.modules["opentelemetry"].trace = self.modules["opentelemetry.trace"]


@pytest.fixture
def fresh_shim(monkeypatch):
    monkeypatch.setattr(otel, "_tracer", None)
    monkeypatch.setattr(otel, "_enabled", False)
    for k in ("OTEL_EXPORTER_OTLP_TRACES_ENDPOINT", "OTEL_EXPORTER_OTLP_ENDPOINT", "TRACEPARENT"):
        monkeypatch.delenv(k, raising=False)
    return monkeypatch


def test_no_endpoint_means_no_sdk_and_no_span(fresh_shim):
    sdk = _FakeSdk()
    for k, v in sdk.modules.items():
        fresh_shim.setitem(sys.modules, k, v)
    with otel.start_as_current_span("fit") as span:
        assert span is None
    assert sdk.spans == [] and sdk.resources == []


def test_endpoint_configures_once_and_names_spans(fresh_shim):
    sdk = _FakeSdk()
    for k, v in sdk.modules.items():
        fresh_shim.setitem(sys.modules, k, v)
    fresh_shim.setenv("OTEL_EXPORTER_OTLP_ENDPOINT", "http://127.0.0.1:4317")
    fresh_shim.setenv("TRACEPARENT", "00-0af7651916cd43dd8448eb211c80319c-b7ad6b7169203331-01")
    with otel.start_as_current_span("fit") as a:
        with otel.start_as_current_span("train_on_batch") as b:
            assert (a, b) == ("fit", "train_on_batch")
    from tensornet_b200.version import VERSION
    assert sdk.resources == [{"service.name": "tensornet", "tensornet.version": VERSION}]        # configured once
    assert [s[0] for s in sdk.spans] == ["fit", "train_on_batch"]
    assert sdk.extracted[0] == {"traceparent": "00-0af7651916cd43dd8448eb211c80319c-b7ad6b7169203331-01"}
    assert sdk.spans[0][1] == ("ctx", sdk.extracted[0])


def test_endpoint_without_sdk_stays_silent(fresh_shim):
    fresh_shim.setenv("OTEL_EXPORTER_OTLP_TRACES_ENDPOINT", "http://127.0.0.1:4317")
    fresh_shim.setitem(sys.modules, "opentelemetry", None)          # import raises ImportError
    with otel.start_as_current_span("predict") as span:
        assert span is None
