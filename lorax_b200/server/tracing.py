"""Request tracing on the shard: one span per RPC, child of the router's batch span, exported as OTLP/HTTP JSON or, for a
`grpc://host:port` endpoint (or any endpoint on port 4317), as OTLP/gRPC protobuf through `TraceService/Export`.

The router puts its batch span's W3C `traceparent` in front of the framed message (`csrc/host/shard_client.hpp`); the shard
wraps the RPC in a span of service `lorax.server-{rank}` and posts finished spans to `{endpoint}/v1/traces` from a
background thread.  The reference does the same with the OpenTelemetry SDK: a UDS-aware server interceptor and an OTLP/gRPC
exporter (`server/lorax_server/tracing.py:15-62`), spans on `generate_token / filter / concatenate`
(`models/flash_causal_lm.py:391,582,1590`).

`LORAX_PROFILER_DIR` is the other half of the reference's profiling story (`models/model.py:121-131`, `server.py:114-118`):
a `torch.profiler` trace of the first prefills after warm-up, written for TensorBoard.
"""

from __future__ import annotations

import contextlib
import json
import os
import queue
import threading
import time
import urllib.request
from typing import Dict, List, Optional

TRACEPARENT_BYTES = 55
TRACE_FLAG = 0x80000000


def parse_traceparent(h: str):
    """-> (trace_id, span_id) or None."""
    parts = h.split("-") if h else []
    if len(parts) != 4 or len(parts[1]) != 32 or len(parts[2]) != 16:
        return None
    try:
        int(parts[1], 16), int(parts[2], 16)
    except ValueError:
        return None
    if set(parts[1]) == {"0"} or set(parts[2]) == {"0"}:
        return None
    return parts[1], parts[2]


def _any(v):
    if isinstance(v, bool):
        return {"boolValue": v}
    if isinstance(v, int):
        return {"intValue": str(v)}
    if isinstance(v, float):
        return {"doubleValue": v}
    return {"stringValue": str(v)}


# ---- protobuf wire format for opentelemetry.proto.collector.trace.v1.ExportTraceServiceRequest (field numbers of trace.proto)
def _varint(v: int) -> bytes:
    out = bytearray()
    while v >= 0x80:
        out.append((v & 0x7F) | 0x80)
        v >>= 7
    out.append(v)
    return bytes(out)


def _ld(field: int, payload: bytes) -> bytes:
    return _varint((field << 3) | 2) + _varint(len(payload)) + payload


def _vi(field: int, v: int) -> bytes:
    return _varint(field << 3) + _varint(v & 0xFFFFFFFFFFFFFFFF)


def _f64(field: int, v: int) -> bytes:
    return _varint((field << 3) | 1) + int(v).to_bytes(8, "little")


def _any_pb(v: dict) -> bytes:
    if "boolValue" in v:
        return _vi(2, int(v["boolValue"]))
    if "intValue" in v:
        return _vi(3, int(v["intValue"]))
    if "doubleValue" in v:
        import struct
        return _varint((4 << 3) | 1) + struct.pack("<d", v["doubleValue"])
    return _ld(1, str(v.get("stringValue", "")).encode())


def _kv_pb(key: str, value: dict) -> bytes:
    return _ld(1, key.encode()) + _ld(2, _any_pb(value))


def span_to_pb(span: dict) -> bytes:
    """One span in the JSON form used above -> an opentelemetry.proto.trace.v1.Span message."""
    out = _ld(1, bytes.fromhex(span["traceId"])) + _ld(2, bytes.fromhex(span["spanId"]))
    if span.get("parentSpanId"):
        out += _ld(4, bytes.fromhex(span["parentSpanId"]))
    out += _ld(5, span["name"].encode()) + _vi(6, int(span.get("kind", 1)))
    out += _f64(7, int(span["startTimeUnixNano"])) + _f64(8, int(span["endTimeUnixNano"]))
    for a in span.get("attributes", []):
        out += _ld(9, _kv_pb(a["key"], a["value"]))
    st = span.get("status") or {}
    if st.get("code"):
        out += _ld(15, _ld(2, str(st.get("message", "")).encode()) + _vi(3, int(st["code"])))
    return out


def export_request_pb(service: str, spans: List[dict]) -> bytes:
    scope_spans = _ld(1, _ld(1, b"lorax_b200")) + b"".join(_ld(2, span_to_pb(s)) for s in spans)
    resource = _ld(1, _kv_pb("service.name", {"stringValue": service}))
    return _ld(1, _ld(1, resource) + _ld(2, scope_spans))


def _grpc_target(endpoint: Optional[str]) -> Optional[str]:
    """host:port when the endpoint names an OTLP/gRPC collector, else None."""
    if not endpoint:
        return None
    for pre in ("grpc://", "http://"):
        if endpoint.startswith(pre):
            hp = endpoint[len(pre):].split("/", 1)[0]
            if pre == "grpc://":
                return hp if ":" in hp else hp + ":4317"
            return hp if hp.endswith(":4317") else None
    return None


class Tracer:
    def __init__(self, endpoint: Optional[str], service: str, flush_s: float = 0.5):
        self.service = service
        self.grpc_target = _grpc_target(endpoint)
        self.enabled = bool(endpoint) and (endpoint.startswith("http://") or self.grpc_target is not None)
        self.url = None
        self._export = None
        self.sent_batches = 0
        self.dropped = 0
        if self.enabled:
            base = endpoint.rstrip("/")
            self.url = base if base.endswith("/v1/traces") else base + "/v1/traces"
            if self.grpc_target is not None:
                import grpc
                self._channel = grpc.insecure_channel(self.grpc_target)
                self._export = self._channel.unary_unary("/opentelemetry.proto.collector.trace.v1.TraceService/Export",
                                                         request_serializer=None, response_deserializer=None)
            self._q: "queue.Queue[dict]" = queue.Queue(maxsize=8192)
            self._stop = threading.Event()
            self._flush_s = flush_s
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    @contextlib.contextmanager
    def span(self, name: str, traceparent: Optional[str] = None, attributes: Optional[Dict] = None):
        """Span around the body; a child of `traceparent` when given, else the root of a new trace.  Yields the attribute
        dict so the body can add to it."""
        attrs = dict(attributes or {})
        if not self.enabled:
            yield attrs
            return
        parent = parse_traceparent(traceparent) if traceparent else None
        trace_id = parent[0] if parent else os.urandom(16).hex()
        span = {"traceId": trace_id, "spanId": os.urandom(8).hex(), "name": name, "kind": 2, "startTimeUnixNano": str(time.time_ns())}
        if parent:
            span["parentSpanId"] = parent[1]
        status = {}
        try:
            yield attrs
        except Exception as e:
            status = {"code": 2, "message": f"{type(e).__name__}: {e}"}
            raise
        finally:
            span["endTimeUnixNano"] = str(time.time_ns())
            span["attributes"] = [{"key": k, "value": _any(v)} for k, v in attrs.items()]
            span["status"] = status
            try:
                self._q.put_nowait(span)
            except queue.Full:
                self.dropped += 1

    def _post(self, spans: List[dict]):
        if self._export is not None:
            for attempt in range(3):
                try:
                    self._export(export_request_pb(self.service, spans), timeout=2)
                    self.sent_batches += 1
                    return
                except Exception:
                    time.sleep(0.1 * (1 << attempt))
            self.dropped += len(spans)
            return
        body = json.dumps({"resourceSpans": [{"resource": {"attributes": [{"key": "service.name", "value": {"stringValue": self.service}}]},
                                              "scopeSpans": [{"scope": {"name": "lorax_b200"}, "spans": spans}]}]}).encode()
        req = urllib.request.Request(self.url, data=body, headers={"Content-Type": "application/json"}, method="POST")
        for attempt in range(3):
            try:
                with urllib.request.urlopen(req, timeout=2) as r:
                    if 200 <= r.status < 300:
                        self.sent_batches += 1
                        return
            except Exception:
                time.sleep(0.1 * (1 << attempt))
        self.dropped += len(spans)

    def _drain(self) -> List[dict]:
        out = []
        while len(out) < 256:
            try:
                out.append(self._q.get_nowait())
            except queue.Empty:
                break
        return out

    def _loop(self):
        while not self._stop.is_set():
            self._stop.wait(self._flush_s)
            spans = self._drain()
            if spans:
                self._post(spans)
        spans = self._drain()
        if spans:
            self._post(spans)

    def shutdown(self):
        if self.enabled:
            self._stop.set()
            self._thread.join(timeout=5)


class PrefillProfiler:
    """`LORAX_PROFILER_DIR=<dir>`: profile the first `steps` prefills (CPU + CUDA activities, stacks) and write a TensorBoard
    trace; `step()` is called once per Prefill RPC."""

    def __init__(self, directory: Optional[str], steps: int = 10):
        self.prof = None
        self.left = 0
        if directory:
            import torch
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            os.makedirs(directory, exist_ok=True)
            self.prof = torch.profiler.profile(activities=acts, with_stack=True,
                                               on_trace_ready=torch.profiler.tensorboard_trace_handler(directory, use_gzip=True))
            self.left = steps
            self.prof.start()

    def step(self):
        if self.prof is None:
            return
        self.prof.step()
        self.left -= 1
        if self.left <= 0:
            self.prof.stop()
            self.prof = None
