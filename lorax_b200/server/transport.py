"""Shard endpoints.

Two servers expose the same :class:`ShardRuntime`:

* `serve_framed`  the length-prefixed protobuf framing on `{uds_path}-{rank}.lx` that the C++ router speaks
  (`csrc/host/shard_client.hpp` documents the frame);
* `serve_grpc`    a regular gRPC `generate.v1.LoraxService` on `unix://{uds_path}-{rank}` (grpc.aio, message classes
  built at run time from the proto file), for any client of the original contract.  Exceptions become
  `INTERNAL` status, as the reference's interceptor does (`server/lorax_server/interceptor.py:11-48`).

Calls are serialised through one lock: the runtime drives a single CUDA stream.
"""

from __future__ import annotations

import json
import os
import socket
import struct
import threading
import traceback
from typing import Optional

import torch

from .proto import load_pb
from .tracing import TRACE_FLAG, TRACEPARENT_BYTES

HELPER_TOKENIZE, HELPER_TOKENIZE_JSON, HELPER_CHAT_TEMPLATE, HELPER_TOKENIZER_FILE, HELPER_CHAT_SETUP = 100, 101, 102, 103, 104


def _resolve_device(dev: torch.device) -> torch.device:
    """`cuda` without an index names the current device of the thread that built the runtime: pin it down once."""
    if dev.type == "cuda" and dev.index is None:
        return torch.device("cuda", torch.cuda.current_device())
    return dev


def _select_device(dev: torch.device):
    """Make `dev` the calling thread's current CUDA device."""
    if dev.type == "cuda" and dev.index is not None:
        torch.cuda.set_device(dev.index)


def _dispatch(runtime, name: str, request):
    fn = {
        "Info": lambda r: runtime.info(), "ServiceDiscovery": None, "ClearCache": runtime.clear_cache,
        "FilterBatch": runtime.filter_batch, "Warmup": runtime.warmup, "Prefill": runtime.prefill, "Embed": runtime.embed,
        "Classify": runtime.classify, "Decode": runtime.decode, "Health": lambda r: runtime.health(),
        "DownloadAdapter": runtime.download_adapter, "LoadAdapter": runtime.load_adapter, "OffloadAdapter": runtime.offload_adapter,
    }[name]
    with torch.inference_mode():
        return fn(request)


class FramedServer:
    def __init__(self, runtime, path: str, urls=None):
        self.rt = runtime
        self.device = _resolve_device(runtime.model.device)
        self.path = path
        self.pb = load_pb()
        self.ids = {v: k for k, v in self.pb.METHOD_IDS.items()}
        self.urls = urls or [path]
        self.lock = threading.Lock()
        self.sock: Optional[socket.socket] = None
        self._stop = threading.Event()
        self.thread: Optional[threading.Thread] = None

    def handle(self, method: int, payload: bytes) -> bytes:
        if method == HELPER_TOKENIZE:
            ids = self.rt.tokenize(payload[1:].decode("utf-8"), add_special=payload[:1] == b"\x01")
            return struct.pack(f"<{len(ids)}I", *ids)
        if method == HELPER_TOKENIZE_JSON:
            return json.dumps(self.rt.tokenize_detailed(json.loads(payload.decode("utf-8")))).encode()
        if method == HELPER_CHAT_TEMPLATE:
            return self.rt.apply_chat_template(json.loads(payload.decode("utf-8"))).encode("utf-8")
        if method == HELPER_CHAT_SETUP:        # what the router needs to render chat templates itself
            from .chat_template import DEFAULT_TEMPLATE
            plain = getattr(type(self.rt).apply_chat_template, "__qualname__", "").startswith("ShardRuntime.")
            return json.dumps({"chat_template": (getattr(self.rt, "chat_template", None) or DEFAULT_TEMPLATE) if plain else None,
                               "bos_token": getattr(self.rt, "bos_token", "") or "", "eos_token": getattr(self.rt, "eos_token", "") or ""}).encode()
        if method == HELPER_TOKENIZER_FILE:
            fn = getattr(self.rt, "router_tokenizer_json", None)
            return (fn() if fn is not None else "").encode("utf-8")
        name = self.ids.get(method)
        if name is None:
            raise ValueError(f"unknown method id {method}")
        req_cls, _ = self.pb.RPCS[name]
        req = req_cls.FromString(payload)
        if name == "ServiceDiscovery":
            return self.pb.ServiceDiscoveryResponse(urls=self.urls).SerializeToString()
        with self.lock:
            return _dispatch(self.rt, name, req).SerializeToString()

    def _serve_conn(self, conn: socket.socket):
        def read_exact(n):
            buf = bytearray()
            while len(buf) < n:
                chunk = conn.recv(n - len(buf))
                if not chunk:
                    raise ConnectionError
                buf += chunk
            return bytes(buf)
        # the CUDA "current device" is a per-thread setting and new threads start on device 0: the kernels of this library are
        # launched through the raw runtime API, so the handler thread must select the shard's GPU itself
        _select_device(self.device)
        try:
            while not self._stop.is_set():
                method, length = struct.unpack("<II", read_exact(8))
                payload = read_exact(length) if length else b""
                traceparent = None
                if method & TRACE_FLAG:                 # the router's span context in front of the message
                    method &= ~TRACE_FLAG
                    traceparent, payload = payload[:TRACEPARENT_BYTES].decode("ascii", "replace"), payload[TRACEPARENT_BYTES:]
                try:
                    tracer = getattr(self.rt, "tracer", None)
                    if tracer is not None and tracer.enabled and traceparent:
                        with tracer.span(self.ids.get(method, str(method)), traceparent, {"rpc.payload_bytes": len(payload)}):
                            out = self.handle(method, payload)
                    else:
                        out = self.handle(method, payload)
                    conn.sendall(struct.pack("<II", 0, len(out)) + out)
                except Exception as e:  # report, keep the connection
                    if self.rt.model.device.type == "cuda":
                        torch.cuda.empty_cache()
                    msg = f"{type(e).__name__}: {e}".encode()
                    if os.environ.get("LORAX_B200_DEBUG"):
                        traceback.print_exc()
                    conn.sendall(struct.pack("<II", 1, len(msg)) + msg)
        except (ConnectionError, OSError, struct.error):
            pass
        finally:
            conn.close()

    def start(self):
        if os.path.exists(self.path):
            os.unlink(self.path)
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self.sock.bind(self.path)
        self.sock.listen(64)
        self.sock.settimeout(0.2)

        def loop():
            while not self._stop.is_set():
                try:
                    conn, _ = self.sock.accept()
                except socket.timeout:
                    continue
                except OSError:
                    break
                threading.Thread(target=self._serve_conn, args=(conn,), daemon=True).start()
        self.thread = threading.Thread(target=loop, daemon=True)
        self.thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self.sock is not None:
            self.sock.close()
        if self.thread is not None:
            self.thread.join(timeout=2)
        if os.path.exists(self.path):
            os.unlink(self.path)


async def serve_grpc(runtime, uds_path: str, rank: int, world_size: int, lock: Optional[threading.Lock] = None):
    """Start the grpc.aio endpoint; returns the server (caller awaits `wait_for_termination`)."""
    import grpc
    pb = load_pb()
    lock = lock or threading.Lock()
    device = _resolve_device(runtime.model.device)
    urls = [f"unix://{uds_path}-{r}" for r in range(world_size)]

    def make(name, req_cls, resp_cls):
        async def handler(request, context):
            try:
                if name == "ServiceDiscovery":
                    return pb.ServiceDiscoveryResponse(urls=urls)
                with lock:
                    _select_device(device)                               # per-thread setting, see FramedServer._serve_conn
                    tracer = getattr(runtime, "tracer", None)
                    if tracer is not None and tracer.enabled:
                        # gRPC callers carry the W3C context as metadata (reference: tracing.py:15-53, grpc-metadata/src/lib.rs)
                        md = {k: v for k, v in (context.invocation_metadata() or ())}
                        if md.get("traceparent"):
                            with tracer.span(name, md["traceparent"]):
                                return _dispatch(runtime, name, request)
                    return _dispatch(runtime, name, request)
            except Exception as e:
                if runtime.model.device.type == "cuda":
                    torch.cuda.empty_cache()
                await context.abort(grpc.StatusCode.INTERNAL, f"{type(e).__name__}: {e}")
        return grpc.unary_unary_rpc_method_handler(handler, request_deserializer=req_cls.FromString,
                                                   response_serializer=resp_cls.SerializeToString)
    handlers = {name: make(name, rq, rs) for name, (rq, rs) in pb.RPCS.items()}
    server = grpc.aio.server(options=[("grpc.max_send_message_length", (1 << 31) - 1), ("grpc.max_receive_message_length", (1 << 31) - 1)])
    server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(pb.SERVICE, handlers),))
    server.add_insecure_port(f"unix://{uds_path}-{rank}")
    await server.start()
    return server
