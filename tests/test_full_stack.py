"""Launcher-less full stack on CPU: a Python shard (framed UDS transport + gRPC) serving a tiny Llama checkpoint
with PEFT adapters on disk, the C++ `lorax-router` binary in front of it, and HTTP clients."""
import json
import os
import socket
import subprocess
import time
import urllib.request

import pytest
import torch
from safetensors.torch import save_file

from lorax_b200.adapters.lora import random_adapter, save_peft_adapter
from lorax_b200.config import EngineConfig, tiny_llama
from lorax_b200.models.decoder import DecoderModel
from lorax_b200.models.loading import export_hf_state_dict

ROUTER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lorax_b200", "bin", "lorax-router")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _post(port, path, body, stream=False, headers=None):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json", **(headers or {})})
    try:
        with urllib.request.urlopen(req, timeout=60) as r:
            data = r.read().decode()
            return r.status, data, dict(r.headers)
    except urllib.error.HTTPError as e:
        return e.code, e.read().decode(), dict(e.headers)


@pytest.fixture(scope="module")
def stack(tmp_path_factory):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from lorax_b200.csrc import build
    build.build_host()
    root = tmp_path_factory.mktemp("stack")
    cfg = tiny_llama(vocab_size=512)
    cfg.eos_token_id = 1
    model = DecoderModel.random_init(cfg, "cpu", torch.float32, seed=0)
    mdir = root / "model"
    mdir.mkdir()
    save_file(export_hf_state_dict(model), str(mdir / "model.safetensors"), metadata={"format": "pt"})
    d = cfg.to_dict()
    d["architectures"] = ["LlamaForCausalLM"]
    (mdir / "config.json").write_text(json.dumps(d))
    vocab = {f"w{i}": i for i in range(511)}
    vocab["<unk>"] = 511
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(mdir / "tokenizer.json"))
    (mdir / "tokenizer_config.json").write_text(json.dumps({"chat_template": "{% for m in messages %}{{ m['content'] }} {% endfor %}"}))
    for i in range(2):
        c, mm = random_adapter(cfg, r=8, alpha=16, target_modules=["q_proj", "v_proj", "down_proj"], seed=50 + i, std_a=0.1, std_b=0.1)
        save_peft_adapter(root / f"adapter{i}", c, mm)

    from lorax_b200.server.runtime import build_runtime
    from lorax_b200.server.transport import FramedServer
    ecfg = EngineConfig(max_input_length=64, max_total_tokens=128, max_batch_prefill_tokens=256, compile=False)
    rt = build_runtime(str(mdir), ecfg, device="cpu", dtype=torch.float32, source="local", num_blocks=256, max_batch=16)
    uds = str(root / "shard")
    # a stand-in for an OTLP/HTTP collector and a request-log sink: records every JSON document posted to it
    import http.server
    import threading
    received = []

    class Sink(http.server.BaseHTTPRequestHandler):
        def do_POST(self):
            body = self.rfile.read(int(self.headers.get("Content-Length", "0")))
            received.append((self.path, json.loads(body.decode())))
            self.send_response(200)
            self.send_header("Content-Length", "2")
            self.end_headers()
            self.wfile.write(b"{}")

        def log_message(self, *a):
            pass
    sink = http.server.ThreadingHTTPServer(("127.0.0.1", 0), Sink)
    threading.Thread(target=sink.serve_forever, daemon=True).start()
    sink_url = f"http://127.0.0.1:{sink.server_address[1]}"
    from lorax_b200.server.tracing import Tracer
    rt.tracer = Tracer(sink_url, "lorax.server-0", flush_s=0.1)
    srv = FramedServer(rt, uds + "-0.lx").start()
    port = _free_port()
    proc = subprocess.Popen([ROUTER, "--port", str(port), "--hostname", "127.0.0.1", "--master-shard-uds-path", uds, "--num-shard", "1",
                             "--max-input-length", "64", "--max-total-tokens", "128", "--max-batch-prefill-tokens", "256",
                             "--model-id", "tiny", "--adapter-source", "local", "--waiting-served-ratio", "0.3", "--otlp-endpoint", sink_url],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env={**os.environ, "REQUEST_LOGGER_URL": sink_url + "/log"})
    ok = False
    for _ in range(100):
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                ok = r.status == 200
                break
        except Exception:
            time.sleep(0.1)
    if not ok:
        proc.kill()
        raise RuntimeError("router did not come up: " + proc.stdout.read().decode()[-2000:])
    yield dict(port=port, root=root, rt=rt, model=model, cfg=cfg, received=received, uds=uds)
    sink.shutdown()
    rt.tracer.shutdown()
    proc.terminate()
    try:
        proc.wait(timeout=10)
    except subprocess.TimeoutExpired:
        proc.kill()
    srv.stop()


def test_generate_base_and_adapters_match_engine(stack):
    port, root = stack["port"], stack["root"]
    prompt = " ".join(f"w{i}" for i in (5, 17, 200, 33, 8, 91))
    outs = {}
    for name, params in (("base", {}), ("a0", {"adapter_id": str(root / "adapter0"), "adapter_source": "local"}),
                         ("a1", {"adapter_id": str(root / "adapter1"), "adapter_source": "local"})):
        st, body, hdr = _post(port, "/generate", {"inputs": prompt, "parameters": {"max_new_tokens": 8, "details": True, "ignore_eos_token": True, **params}})
        assert st == 200, body
        j = json.loads(body)
        assert j["details"]["generated_tokens"] == 8 and j["details"]["finish_reason"] == "length"
        assert len(j["details"]["tokens"]) == 8 and j["details"]["prompt_tokens"] == 6
        assert "x-generated-tokens" in {k.lower() for k in hdr}
        outs[name] = [t["id"] for t in j["details"]["tokens"]]
    assert outs["base"] != outs["a0"] or outs["base"] != outs["a1"]
    # oracle: the in-process engine with the same model
    from lorax_b200.runtime.engine import Engine
    eng = Engine(stack["model"], EngineConfig(max_total_tokens=128, max_batch_prefill_tokens=256), num_blocks=64, max_batch=4)
    base = eng.generate([[5, 17, 200, 33, 8, 91]], max_new_tokens=8)[0]
    assert outs["base"] == base


def test_stream_and_openai_routes(stack):
    port = stack["port"]
    st, body, _ = _post(port, "/generate_stream", {"inputs": "w1 w2 w3", "parameters": {"max_new_tokens": 5, "ignore_eos_token": True, "details": True}})
    assert st == 200
    events = [json.loads(l[5:]) for l in body.replace("\r", "").split("\n") if l.startswith("data:")]
    assert len(events) == 5 and events[-1]["generated_text"] is not None and events[0]["generated_text"] is None
    assert events[-1]["details"]["generated_tokens"] == 5
    st, body, _ = _post(port, "/v1/chat/completions", {"model": "tiny", "messages": [{"role": "user", "content": "w4 w5"}], "max_tokens": 4})
    assert st == 200, body
    j = json.loads(body)
    assert j["object"] == "chat.completion" and j["choices"][0]["message"]["role"] == "assistant" and j["usage"]["completion_tokens"] <= 4
    # the router rendered the chat template itself (no helper call to the shard), and the prompt it built is the shard renderer's
    with urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5) as r:
        count = [l for l in r.read().decode().splitlines() if l.startswith("lorax_router_chat_templates ")]
    assert count and int(count[0].split()[1]) >= 1, count
    want_prompt = stack["rt"].apply_chat_template({"messages": [{"role": "user", "content": "w4 w5"}]})
    assert j["usage"]["prompt_tokens"] == len(stack["rt"].tokenize(want_prompt))
    st, body, _ = _post(port, "/v1/completions", {"model": "tiny", "prompt": "w4 w5", "max_tokens": 3, "stream": True})
    assert st == 200 and "[DONE]" in body


def test_errors_and_misc_routes(stack):
    port = stack["port"]
    st, body, _ = _post(port, "/generate", {"inputs": "w1", "parameters": {"max_new_tokens": 4, "top_p": 2.0}})
    assert st == 422 and json.loads(body)["error_type"] == "validation"
    st, body, _ = _post(port, "/generate", {"inputs": "w1", "parameters": {"max_new_tokens": 4, "adapter_id": "/nonexistent/adapter", "adapter_source": "local"}})
    assert st == 424 and "adapter" in json.loads(body)["error"]
    st, body, _ = _post(port, "/generate", {"inputs": "w1 w2", "parameters": {"max_new_tokens": 3}})     # still healthy afterwards
    assert st == 200
    with urllib.request.urlopen(f"http://127.0.0.1:{port}/info", timeout=5) as r:
        info = json.loads(r.read())
    assert info["max_total_tokens"] == 128 and info["block_size"] == 32
    with urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5) as r:
        m = r.read().decode()
    assert "lorax_request_success" in m and "lorax_batch_inference_duration_bucket" in m
    for name in ('lorax_batch_inference_success{method="prefill"}', 'lorax_batch_inference_success{method="decode"}',
                 "lorax_request_validation_duration_bucket", "lorax_request_max_new_tokens_bucket"):
        assert name in m, name
    # requests were tokenised by the router's own workers, not by a call to shard 0
    count = [l for l in m.splitlines() if l.startswith("lorax_router_tokenizations ")]
    assert count and int(count[0].split()[1]) >= 2, count
    st, body, _ = _post(port, "/tokenize", {"inputs": "w7 w8"})
    assert st == 200 and [t["id"] for t in json.loads(body)] == [7, 8]


def test_concurrent_heterogeneous_requests(stack):
    import concurrent.futures as cf
    port, root = stack["port"], stack["root"]

    def one(i):
        params = {"max_new_tokens": 4 + i % 4, "ignore_eos_token": True, "details": True}
        if i % 3:
            params.update(adapter_id=str(root / f"adapter{i % 3 - 1}"), adapter_source="local")
        return _post(port, "/generate", {"inputs": f"w{i} w{i + 1} w{i + 2}", "parameters": params})
    with cf.ThreadPoolExecutor(12) as ex:
        res = list(ex.map(one, range(12)))
    assert all(st == 200 for st, _, _ in res)
    assert [json.loads(b)["details"]["generated_tokens"] for _, b, _ in res] == [4 + i % 4 for i in range(12)]
    # staggered arrivals: prompts that arrive while others decode ride along with the decode step (one forward pass), and the
    # tokens equal those of the same requests sent alone
    import threading
    import time as _t
    prompts = [" ".join(f"w{(11 * i + j) % 500 + 2}" for j in range(5 + i % 5)) for i in range(6)]

    def gen(i):
        params = {"max_new_tokens": 12, "ignore_eos_token": True, "details": True}
        if i % 2:
            params.update(adapter_id=str(root / f"adapter{i % 2 - 1}"), adapter_source="local")
        st, body, _ = _post(port, "/generate", {"inputs": prompts[i], "parameters": params})
        assert st == 200, body
        return [t["id"] for t in json.loads(body)["details"]["tokens"]]
    alone = [gen(i) for i in range(6)]
    before = dict(stack["rt"].fused_stats)
    out = [None] * 6

    def worker(i):
        _t.sleep(0.03 * i)
        out[i] = gen(i)
    ths = [threading.Thread(target=worker, args=(i,)) for i in range(6)]
    [t.start() for t in ths]
    [t.join() for t in ths]
    assert out == alone
    assert stack["rt"].fused_stats["one_pass"] > before["one_pass"]


def test_sampling_and_seed(stack):
    port = stack["port"]
    p = {"max_new_tokens": 6, "ignore_eos_token": True, "do_sample": True, "temperature": 1.5, "top_k": 50, "seed": 7, "details": True}
    a = json.loads(_post(port, "/generate", {"inputs": "w9 w10", "parameters": p})[1])
    b = json.loads(_post(port, "/generate", {"inputs": "w9 w10", "parameters": p})[1])
    assert [t["id"] for t in a["details"]["tokens"]] == [t["id"] for t in b["details"]["tokens"]]
    assert a["details"]["seed"] == 7


def test_python_client_sync_and_async(stack):
    import asyncio
    from lorax_b200.client import AsyncClient, Client
    from lorax_b200.client.errors import ValidationError as ServerValidationError
    c = Client(f"http://127.0.0.1:{stack['port']}")
    assert c.health()
    r = c.generate("w1 w2 w3", max_new_tokens=4, ignore_eos_token=True)
    assert r.details.generated_tokens == 4 and len(r.details.tokens) == 4
    toks = list(c.generate_stream("w1 w2 w3", max_new_tokens=4, ignore_eos_token=True))
    assert [t.token.id for t in toks] == [t.id for t in r.details.tokens] and toks[-1].generated_text is not None
    with pytest.raises(ServerValidationError):
        c.generate("w1", max_new_tokens=100000)

    async def go():
        ac = AsyncClient(f"http://127.0.0.1:{stack['port']}")
        outs = await asyncio.gather(*[ac.generate(f"w{i} w2", max_new_tokens=3, ignore_eos_token=True) for i in range(4)])
        streamed = [t async for t in ac.generate_stream("w1 w2 w3", max_new_tokens=4, ignore_eos_token=True)]
        return outs, streamed
    outs, streamed = asyncio.run(go())
    assert all(o.details.generated_tokens == 3 for o in outs) and len(streamed) == 4


def test_tracing_and_request_logger(stack):
    """OTLP/HTTP JSON spans from the router and the shard, stitched together: the request span continues the caller's
    `traceparent`; the batch spans of the batching loop link to it and carry their own context to the shard, whose RPC spans are
    their children.  REQUEST_LOGGER_URL receives one JSON document per finished request."""
    received = stack["received"]
    trace_id, parent = "4bf92f3577b34da6a3ce929d0e0e4736", "00f067aa0ba902b7"
    status, data, _ = _post(stack["port"], "/generate", {"inputs": "w5 w6 w7 w8", "parameters": {"max_new_tokens": 4}},
                            headers={"traceparent": f"00-{trace_id}-{parent}-01"})
    assert status == 200
    want_text = json.loads(data)["generated_text"]

    def spans_of(service):
        out = []
        for path, doc in list(received):
            if path != "/v1/traces":
                continue
            for rs in doc["resourceSpans"]:
                attrs = {a["key"]: a["value"] for a in rs["resource"]["attributes"]}
                if attrs["service.name"]["stringValue"] == service:
                    for ss in rs["scopeSpans"]:
                        out += ss["spans"]
        return out
    req_span = None
    for _ in range(100):
        req_span = next((s for s in spans_of("lorax.router") if s["traceId"] == trace_id), None)
        shard_spans = spans_of("lorax.server-0")
        logged = [d for p, d in list(received) if p == "/log" and d.get("input") == "w5 w6 w7 w8"]
        if req_span is not None and any(s["name"] == "Decode" for s in shard_spans) and logged:
            break
        time.sleep(0.1)
    assert req_span is not None and req_span["parentSpanId"] == parent and req_span["name"] == "generate" and req_span["kind"] == 2
    attrs = {a["key"]: a["value"] for a in req_span["attributes"]}
    assert attrs["generated_tokens"]["intValue"] == "4" and attrs["prompt_tokens"]["intValue"] == "4" and "inference_time_ms" in attrs
    assert int(req_span["endTimeUnixNano"]) > int(req_span["startTimeUnixNano"])
    router_spans = spans_of("lorax.router")
    linked = [s for s in router_spans if any(l["traceId"] == trace_id and l["spanId"] == req_span["spanId"] for l in s.get("links", []))]
    assert {s["name"] for s in linked} >= {"prefill", "decode"}
    root = next(s for s in router_spans if s["name"] == "batching_task")
    assert all(s["traceId"] == root["traceId"] and s["parentSpanId"] == root["spanId"] for s in linked)
    by_id = {s["spanId"]: s for s in linked}
    children = [s for s in shard_spans if s.get("parentSpanId") in by_id]
    assert {s["name"] for s in children} >= {"Prefill", "Decode"}
    assert all(s["traceId"] == root["traceId"] for s in children)
    assert logged[0]["output"] == want_text and logged[0]["generated_tokens"] == 4 and logged[0]["model_id"] == "tiny"


def test_chunked_prefill_matches_unchunked(stack):
    """A second router on the same shard with `--chunked-prefill` and a prefill budget of 24 tokens: prompts of up to 60 tokens
    are prefilled in several steps (interleaved with the decode steps of running requests) and generate the same tokens."""
    import concurrent.futures as cf
    prompts = [" ".join(f"w{(7 * i + 3 * j) % 500 + 2}" for i in range(n)) for j, n in enumerate((60, 9, 47, 30))]
    bodies = [{"inputs": p, "parameters": {"max_new_tokens": 6, "details": True, **({"adapter_id": str(stack["root"] / "adapter0"),
                                                                                      "adapter_source": "local"} if j == 2 else {})}}
              for j, p in enumerate(prompts)]
    want = [json.loads(_post(stack["port"], "/generate", b)[1])["generated_text"] for b in bodies]
    port = _free_port()
    proc = subprocess.Popen([ROUTER, "--port", str(port), "--hostname", "127.0.0.1", "--master-shard-uds-path", stack["uds"], "--num-shard", "1",
                             "--max-input-length", "64", "--max-total-tokens", "128", "--max-batch-prefill-tokens", "24",
                             "--chunked-prefill", "true", "--model-id", "tiny", "--adapter-source", "local"],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    try:
        for _ in range(100):
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                    if r.status == 200:
                        break
            except Exception:
                time.sleep(0.1)
        seen = []
        inner = stack["rt"]._new_sequences

        def spy(batch):
            out = inner(batch)
            seen.append((len(out[1]), [len(c.token_ids) for c in out[2]]))
            return out
        stack["rt"]._new_sequences = spy
        with cf.ThreadPoolExecutor(4) as ex:
            got = list(ex.map(lambda b: _post(port, "/generate", b), bodies))
        stack["rt"]._new_sequences = inner
        assert [g[0] for g in got] == [200] * 4, got
        assert [json.loads(g[1])["generated_text"] for g in got] == want
        assert any(chunks for _, chunks in seen) and all(sum(c) <= 24 for _, c in seen)       # some steps carried prompt chunks
        assert not stack["rt"].seqs
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=10)
        except subprocess.TimeoutExpired:
            proc.kill()


def test_prefix_cache_holds_only_tokens_whose_kv_was_written(stack):
    """A second router with `--prefix-caching`.  A request whose prompt plus generated tokens end exactly on a KV block
    boundary leaves its last sampled token without keys / values (it was never fed back).  A follow-up prompt that extends
    that text must not reuse the boundary block: its output has to equal the answer of the router without a prefix cache."""
    bs = stack["rt"].runner.page
    words = [f"w{(11 * i) % 500 + 2}" for i in range(2 * bs - 3)]
    first = {"inputs": " ".join(words), "parameters": {"max_new_tokens": 3, "details": True, "ignore_eos_token": True}}
    port = _free_port()
    proc = subprocess.Popen([ROUTER, "--port", str(port), "--hostname", "127.0.0.1", "--master-shard-uds-path", stack["uds"], "--num-shard", "1",
                             "--max-input-length", "100", "--max-total-tokens", "128", "--max-batch-prefill-tokens", "256",
                             "--prefix-caching", "true", "--model-id", "tiny", "--adapter-source", "local"],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    try:
        for _ in range(100):
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                    if r.status == 200:
                        break
            except Exception:
                time.sleep(0.1)
        st, body, _ = _post(port, "/generate", first)
        assert st == 200, body
        toks = [t["id"] for t in json.loads(body)["details"]["tokens"]]
        assert len(toks) == 3                                            # prompt + generated = 2 whole blocks
        follow = {"inputs": " ".join(words + [f"w{t}" for t in toks] + ["w7", "w8", "w9"]),
                  "parameters": {"max_new_tokens": 6, "details": True, "ignore_eos_token": True}}
        from lorax_b200.runtime.engine import Engine
        eng = Engine(stack["model"], EngineConfig(max_total_tokens=128, max_batch_prefill_tokens=256), num_blocks=64, max_batch=4)
        want = eng.generate([[int(w[1:]) for w in follow["inputs"].split()]], max_new_tokens=6)[0]
        seen = []
        inner = stack["rt"]._new_sequences

        def spy(batch):
            seen.extend(int(r.cache_len) for r in batch.requests)
            return inner(batch)
        stack["rt"]._new_sequences = spy
        st, body, _ = _post(port, "/generate", follow)
        stack["rt"]._new_sequences = inner
        assert st == 200, body
        assert [t["id"] for t in json.loads(body)["details"]["tokens"]] == want
        assert seen and seen[0] == bs                                    # the first block is reused, the boundary block is not
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=10)
        except subprocess.TimeoutExpired:
            proc.kill()


def test_openapi_document_is_served(stack):
    """`/api-doc/openapi.json` (and `/docs`) serve the OpenAPI document of docs/reference/openapi.json."""
    with urllib.request.urlopen(f"http://127.0.0.1:{stack['port']}/api-doc/openapi.json", timeout=5) as r:
        doc = json.loads(r.read().decode())
    assert doc["openapi"].startswith("3.") and {"/generate", "/generate_stream", "/v1/chat/completions", "/classify", "/metrics"} <= set(doc["paths"])
    assert "GenerateParameters" in doc["components"]["schemas"] and "merged_adapters" in doc["components"]["schemas"]["GenerateParameters"]["properties"]


def test_startup_probe_runs_a_real_request_and_health_runs_a_step(stack):
    """`/startup` sends one real one-token generation through router, scheduler and shard (router/src/server.rs:488-588 of the
    reference does the same); the shard's Health answers only after a one-token prefill into the reserved block 0 has run."""
    port, rt = stack["port"], stack["rt"]
    calls = {"prefill": 0}
    inner = rt.runner.prefill

    def counting(items):
        calls["prefill"] += 1
        if len(items) == 1 and list(items[0].blocks) == [0]:
            calls["probe"] = calls.get("probe", 0) + 1
        return inner(items)
    rt.runner.prefill = counting
    try:
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/startup", timeout=20) as r:
                assert r.status == 200
        except urllib.error.HTTPError as e:
            raise AssertionError(f"/startup answered {e.code}: {e.read().decode()}")
        assert calls["prefill"] >= 1                       # the probe request reached the model
        rt.health()
        assert calls.get("probe", 0) >= 1                  # Health itself runs a step on block 0
    finally:
        rt.runner.prefill = inner


def test_health_turns_false_after_a_device_side_failure(stack):
    """A step that finds the kernels' status word set (a bounded wait that ran out on the device) fails its batch: the client
    gets 424, the router drops the batch, and /health, which probes the shard after a failed generation as the reference does
    (router/src/health.rs:150-178), stays 503 until the shard is healthy again."""
    from lorax_b200.ops.native import NativeError
    port, rt = stack["port"], stack["rt"]
    inner = rt.runner.wait

    def failing_wait(k):
        rt.runner.device_failed = "device status 5 (peer flag timeout), detail 4007"
        raise NativeError(rt.runner.device_failed)
    rt.runner.wait = failing_wait
    try:
        st, body, _ = _post(port, "/generate", {"inputs": "w5 w6 w7", "parameters": {"max_new_tokens": 4}})
        assert st == 424 and "peer flag timeout" in body, (st, body)
        with pytest.raises(urllib.error.HTTPError) as ei:
            urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=5)
        assert ei.value.code == 503
    finally:
        rt.runner.wait = inner
        rt.runner.device_failed = None
    assert not rt.seqs                                                   # the failed batch was cleared on the shard
    with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=5) as r:
        assert r.status == 200
    st, body, _ = _post(port, "/generate", {"inputs": "w5 w6 w7", "parameters": {"max_new_tokens": 4}})
    assert st == 200, body


def test_merge_adapter_weights_equals_the_adapter_applied_at_run_time(stack):
    """`--merge-adapter-weights`: the adapter folded into the base weights at load time generates what the same adapter applied
    per request generates."""
    from lorax_b200.server.runtime import build_runtime
    root = stack["root"]
    ecfg = EngineConfig(max_input_length=64, max_total_tokens=128, max_batch_prefill_tokens=256, compile=False)
    merged = build_runtime(str(root / "model"), ecfg, device="cpu", dtype=torch.float32, source="local", num_blocks=64, max_batch=4,
                           merge_adapter=str(root / "adapter1"), merge_adapter_source="local")
    pb = merged.pb
    ids = [7, 99, 12, 300, 45, 6]

    def gen(rt, adapter_index):
        req = pb.Request(id=1, tokenized_inputs=pb.TokenizedInputs(ids=ids), truncate=64, adapter_index=adapter_index, blocks=[1, 2, 3],
                         parameters=pb.NextTokenChooserParameters(temperature=1.0, top_p=1.0, typical_p=1.0, repetition_penalty=1.0),
                         stopping_parameters=pb.StoppingCriteriaParameters(max_new_tokens=8, ignore_eos_token=True))
        resp = rt.prefill(pb.PrefillRequest(batch=pb.Batch(id=900, requests=[req], size=1, max_tokens=64)))
        out = list(resp.generations[0].next_tokens.ids)
        cached = resp.batch
        while True:
            d = rt.decode(pb.DecodeRequest(batches=[cached]))
            out += list(d.generations[0].next_tokens.ids)
            if not d.HasField("batch"):
                return out
            cached = d.batch
    rt = stack["rt"]
    params = pb.AdapterParameters(adapter_ids=[str(root / "adapter1")])
    rt.load_adapter(pb.LoadAdapterRequest(adapter_parameters=params, adapter_source=2, adapter_index=77))
    want = gen(rt, 77)
    assert gen(merged, 0) == want and gen(rt, 0) != want
    rt.offload_adapter(pb.OffloadAdapterRequest(adapter_parameters=params, adapter_source=2, adapter_index=77))


def _pb_fields(buf: bytes):
    """Protobuf wire format -> list of (field, wire type, value); enough to read an OTLP export request."""
    out, i = [], 0
    while i < len(buf):
        key = shift = 0
        while True:
            b = buf[i]; i += 1
            key |= (b & 0x7F) << shift; shift += 7
            if b < 0x80:
                break
        field, wire = key >> 3, key & 7
        if wire == 0:
            v = shift = 0
            while True:
                b = buf[i]; i += 1
                v |= (b & 0x7F) << shift; shift += 7
                if b < 0x80:
                    break
        elif wire == 1:
            v = int.from_bytes(buf[i:i + 8], "little"); i += 8
        elif wire == 2:
            n = shift = 0
            while True:
                b = buf[i]; i += 1
                n |= (b & 0x7F) << shift; shift += 7
                if b < 0x80:
                    break
            v = buf[i:i + n]; i += n
        else:
            raise ValueError(f"wire type {wire}")
        out.append((field, wire, v))
    return out


def test_tracing_over_otlp_grpc(stack):
    """A router whose `--otlp-endpoint` is a gRPC collector (`grpc://host:port`, or any URL on port 4317): spans arrive as
    protobuf `ExportTraceServiceRequest`s through `TraceService/Export`, which is the transport the reference's exporter speaks
    (router/src/main.rs:492-541).  The collector here is a grpcio server that keeps the raw request bytes."""
    import grpc
    from concurrent import futures
    got = []

    class Collector(grpc.GenericRpcHandler):
        def service(self, details):
            if details.method != "/opentelemetry.proto.collector.trace.v1.TraceService/Export":
                return None
            return grpc.unary_unary_rpc_method_handler(lambda req, ctx: (got.append(req), b"")[1],
                                                       request_deserializer=None, response_serializer=None)
    server = grpc.server(futures.ThreadPoolExecutor(2))
    server.add_generic_rpc_handlers((Collector(),))
    cport = server.add_insecure_port("127.0.0.1:0")
    server.start()
    port = _free_port()
    proc = subprocess.Popen([ROUTER, "--port", str(port), "--hostname", "127.0.0.1", "--master-shard-uds-path", stack["uds"], "--num-shard", "1",
                             "--max-input-length", "64", "--max-total-tokens", "128", "--model-id", "tiny", "--adapter-source", "local",
                             "--otlp-endpoint", f"grpc://127.0.0.1:{cport}"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    try:
        for _ in range(100):
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                    if r.status == 200:
                        break
            except Exception:
                time.sleep(0.1)
        trace_id, parent = "0af7651916cd43dd8448eb211c80319c", "b7ad6b7169203331"
        status, _, _ = _post(port, "/generate", {"inputs": "w5 w6 w7", "parameters": {"max_new_tokens": 3}},
                             headers={"traceparent": f"00-{trace_id}-{parent}-01"})
        assert status == 200

        def spans():
            out = []
            for req in list(got):
                for f, _, rs in _pb_fields(req):
                    assert f == 1
                    rsf = _pb_fields(rs)
                    resource = next(v for k, _, v in rsf if k == 1)
                    kv = _pb_fields(next(v for k, _, v in _pb_fields(resource) if k == 1))
                    assert kv[0][2] == b"service.name" and _pb_fields(kv[1][2])[0][2] == b"lorax.router"
                    for k, _, ss in rsf:
                        if k == 2:
                            out += [dict((ff, vv) for ff, _, vv in _pb_fields(v) if ff != 9) | {"attrs": [vv for ff, _, vv in _pb_fields(v) if ff == 9]}
                                    for kk, _, v in _pb_fields(ss) if kk == 2]
            return out
        mine = None
        for _ in range(100):
            mine = next((s for s in spans() if s[1] == bytes.fromhex(trace_id)), None)
            if mine is not None:
                break
            time.sleep(0.1)
        assert mine is not None, "no span of the request reached the collector"
        assert mine[5] == b"generate" and mine[4] == bytes.fromhex(parent) and mine[6] == 2 and len(mine[2]) == 8
        assert mine[8] > mine[7] > 1_600_000_000 * 10 ** 9          # fixed64 start / end in unix nanoseconds
        attrs = {}
        for a in mine["attrs"]:
            f = _pb_fields(a)
            attrs[f[0][2].decode()] = _pb_fields(f[1][2])[0]
        assert attrs["generated_tokens"][0] == 3 and attrs["generated_tokens"][2] == 3       # AnyValue.int_value
        assert any(s[5] in (b"prefill", b"decode") for s in spans())
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=10)
        except subprocess.TimeoutExpired:
            proc.kill()
        server.stop(0)


def test_shard_tracer_exports_over_otlp_grpc():
    """The shard's tracer against the same kind of collector: a span with a parent, attributes of every type and an error
    status, read back from the protobuf request."""
    import grpc
    from concurrent import futures
    from lorax_b200.server.tracing import Tracer
    got = []

    class Collector(grpc.GenericRpcHandler):
        def service(self, details):
            return grpc.unary_unary_rpc_method_handler(lambda req, ctx: (got.append((details.method, req)), b"")[1])
    server = grpc.server(futures.ThreadPoolExecutor(2))
    server.add_generic_rpc_handlers((Collector(),))
    cport = server.add_insecure_port("127.0.0.1:0")
    server.start()
    try:
        tr = Tracer(f"grpc://127.0.0.1:{cport}", "lorax.server-0", flush_s=0.05)
        assert tr.enabled and tr.grpc_target == f"127.0.0.1:{cport}"
        tp = "00-0af7651916cd43dd8448eb211c80319c-b7ad6b7169203331-01"
        with pytest.raises(RuntimeError):
            with tr.span("Prefill", tp, {"batch": 3, "ratio": 0.5, "ok": True, "who": "x"}):
                raise RuntimeError("boom")
        for _ in range(100):
            if got:
                break
            time.sleep(0.05)
        tr.shutdown()
        assert got and got[0][0] == "/opentelemetry.proto.collector.trace.v1.TraceService/Export" and tr.sent_batches >= 1
        rs = _pb_fields(_pb_fields(got[0][1])[0][2])
        span = _pb_fields(next(v for k, _, v in _pb_fields(next(v for k, _, v in rs if k == 2)) if k == 2))
        d = {k: v for k, _, v in span if k != 9}
        assert d[1] == bytes.fromhex("0af7651916cd43dd8448eb211c80319c") and d[4] == bytes.fromhex("b7ad6b7169203331") and d[5] == b"Prefill"
        assert d[8] >= d[7] and dict((k, v) for k, _, v in _pb_fields(d[15]))[3] == 2
        attrs = {}
        for k, _, v in span:
            if k == 9:
                f = _pb_fields(v)
                attrs[f[0][2]] = _pb_fields(f[1][2])[0]
        import struct
        assert attrs[b"batch"][::2] == (3, 3) and attrs[b"ok"][::2] == (2, 1) and attrs[b"who"][::2] == (1, b"x")
        assert attrs[b"ratio"][0] == 4 and struct.unpack("<d", attrs[b"ratio"][2].to_bytes(8, "little"))[0] == 0.5
        assert Tracer("http://collector:4317", "s").grpc_target == "collector:4317" and Tracer("http://c:4318", "s").grpc_target is None
    finally:
        server.stop(0)


def test_chat_template_tools_guideline_and_echo(stack):
    """Chat-template inputs as the reference applies them (router/src/infer.rs:97-147): tools reach the prompt even when the
    template has no `tools` variable (as JSON behind the last message, followed by the tool prompt), a template that names
    `guideline` refuses a request without one, and `/v1/completions` with `echo` returns the prompt in front of the completion."""
    from lorax_b200.server.chat_template import DEFAULT_TOOL_PROMPT, TemplateError, render_chat
    plain = "{% for m in messages %}<{{ m.role }}>{{ m.content }}{% endfor %}"
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "weather in Paris?"}]
    out = render_chat(msgs, plain, tools=tools)
    assert out.startswith("<system>be brief<user>weather in Paris?\n---\n[{\"type\":\"function\"") and out.endswith(DEFAULT_TOOL_PROMPT)
    assert msgs[1]["content"] == "weather in Paris?"                       # the caller's messages are left alone
    aware = plain + "{% if tools %}[TOOLS {{ tools | length }}]{% endif %}"
    out = render_chat(msgs, aware, tools=tools, tool_prompt="pick one")
    assert out == "<system>be brief<user>weather in Paris?\n---\npick one[TOOLS 1]"
    assert render_chat(msgs, plain) == "<system>be brief<user>weather in Paris?"
    guided = "{{ guideline }}|" + plain
    assert render_chat(msgs, guided, guideline="G").startswith("G|<system>")
    with pytest.raises(TemplateError):
        render_chat(msgs, guided)
    # through the router
    status, data, _ = _post(stack["port"], "/v1/completions", {"model": "tiny", "prompt": "w5 w6 w7", "max_tokens": 3, "echo": True})
    assert status == 200
    echoed = json.loads(data)["choices"][0]["text"]
    status, data, _ = _post(stack["port"], "/v1/completions", {"model": "tiny", "prompt": "w5 w6 w7", "max_tokens": 3})
    assert status == 200 and echoed == "w5 w6 w7" + json.loads(data)["choices"][0]["text"]
    status, data, _ = _post(stack["port"], "/v1/chat/completions", {"model": "tiny", "max_tokens": 3, "guideline": "g", "tool_prompt": "p",
                                                                     "messages": [{"role": "user", "content": "w5 w6"}]})
    assert status == 200 and json.loads(data)["choices"][0]["message"]["role"] == "assistant"


def test_router_leaves_tokenisation_and_templates_to_the_shard_when_told_to(stack):
    """`--router-tokenizer off --router-chat-template off`: a second router on the same shard serves the same answers with shard 0
    doing both (the path a tokenizer file or a template outside the router's subset takes by itself)."""
    port2 = _free_port()
    proc = subprocess.Popen([ROUTER, "--port", str(port2), "--hostname", "127.0.0.1", "--master-shard-uds-path", stack["uds"], "--num-shard", "1",
                             "--max-input-length", "64", "--max-total-tokens", "128", "--max-batch-prefill-tokens", "256", "--model-id", "tiny",
                             "--adapter-source", "local", "--router-tokenizer", "off", "--router-chat-template", "off"],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    try:
        for _ in range(100):
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port2}/health", timeout=1) as r:
                    if r.status == 200:
                        break
            except Exception:
                time.sleep(0.1)
        else:
            raise RuntimeError("second router did not come up")
        body = {"model": "tiny", "messages": [{"role": "user", "content": "w4 w5"}], "max_tokens": 4}
        st1, b1, _ = _post(stack["port"], "/v1/chat/completions", body)
        st2, b2, _ = _post(port2, "/v1/chat/completions", body)
        assert st1 == 200 and st2 == 200
        j1, j2 = json.loads(b1), json.loads(b2)
        assert j1["choices"][0]["message"]["content"] == j2["choices"][0]["message"]["content"] and j1["usage"] == j2["usage"]
        with urllib.request.urlopen(f"http://127.0.0.1:{port2}/metrics", timeout=5) as r:
            m = r.read().decode()
        assert "lorax_router_tokenizations" not in m and "lorax_router_chat_templates 0" in m
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=10)
        except subprocess.TimeoutExpired:
            proc.kill()
