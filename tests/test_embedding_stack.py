"""Embedding / token-classification model behind the C++ router on CPU: `/embed`, `/v1/embeddings`, `/classify`,
`/classify_batch`, and the generation routes refusing politely."""
import json
import os
import subprocess
import time
import urllib.request

import pytest
import torch
from safetensors.torch import save_file

from test_full_stack import ROUTER, _free_port, _post


@pytest.fixture(scope="module")
def emb_stack(tmp_path_factory):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from lorax_b200.csrc import build
    from lorax_b200.models.encoder import EncoderConfig, random_encoder_state_dict
    build.build_host()
    root = tmp_path_factory.mktemp("emb")
    raw = {"model_type": "distilbert", "vocab_size": 512, "dim": 64, "n_layers": 2, "n_heads": 4, "hidden_dim": 128,
           "max_position_embeddings": 64, "id2label": {str(i): f"TAG{i}" for i in range(4)}}

    cfg = EncoderConfig.from_dict(raw)
    sd = random_encoder_state_dict(cfg, seed=11, num_labels=4)
    mdir = root / "model"
    mdir.mkdir()
    save_file({("distilbert." + k if not k.startswith("classifier") else k): v for k, v in sd.items()}, str(mdir / "model.safetensors"),
              metadata={"format": "pt"})
    (mdir / "config.json").write_text(json.dumps(raw))
    vocab = {f"w{i}": i for i in range(512)}
    vocab["<unk>"] = 0
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(mdir / "tokenizer.json"))

    from lorax_b200.config import EngineConfig
    from lorax_b200.server.runtime import EncoderRuntime, build_runtime
    from lorax_b200.server.transport import FramedServer
    rt = build_runtime(str(mdir), EngineConfig(max_input_length=32, max_total_tokens=64, max_batch_prefill_tokens=128, compile=False),
                       device="cpu", dtype=torch.float32, source="local")
    assert isinstance(rt, EncoderRuntime)
    uds = str(root / "shard")
    srv = FramedServer(rt, uds + "-0.lx").start()
    port = _free_port()
    proc = subprocess.Popen([ROUTER, "--port", str(port), "--hostname", "127.0.0.1", "--master-shard-uds-path", uds, "--num-shard", "1",
                             "--max-input-length", "32", "--max-total-tokens", "64", "--max-batch-prefill-tokens", "128",
                             "--model-id", "tiny-distilbert"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    ok = False
    for _ in range(100):
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/info", timeout=1) as r:
                ok = r.status == 200
                break
        except Exception:
            time.sleep(0.1)
    if not ok:
        proc.kill()
        raise RuntimeError("router did not come up: " + proc.stdout.read().decode()[-2000:])
    yield dict(port=port, rt=rt)
    proc.terminate()
    try:
        proc.wait(timeout=10)
    except subprocess.TimeoutExpired:
        proc.kill()
    srv.stop()


def test_embed_and_classify_routes(emb_stack):
    port, rt = emb_stack["port"], emb_stack["rt"]
    text = "w5 w9 w77 w3"
    want = rt.model.embed([rt.tokenize(text)])[0]
    st, body, _ = _post(port, "/embed", {"inputs": text})
    assert st == 200, body
    got = json.loads(body)["embeddings"]
    assert len(got) == 64 and max(abs(a - b) for a, b in zip(got, want)) < 1e-4

    st, body, _ = _post(port, "/v1/embeddings", {"input": [text, "w1 w2"], "model": "x"})
    assert st == 200, body
    data = json.loads(body)["data"]
    assert [d["index"] for d in data] == [0, 1] and len(data[1]["embedding"]) == 64
    assert max(abs(a - b) for a, b in zip(data[0]["embedding"], want)) < 1e-4

    labels, scores = rt.model.classify([rt.tokenize(text)])
    st, body, _ = _post(port, "/classify", {"inputs": text})
    assert st == 200, body
    ents = json.loads(body)
    assert [e["entity_group"] for e in ents] == labels[0]
    assert max(abs(e["score"] - s) for e, s in zip(ents, scores[0])) < 1e-4

    st, body, _ = _post(port, "/classify_batch", {"inputs": [text, "w8"]})
    assert st == 200, body
    out = json.loads(body)
    assert len(out) == 2 and len(out[1]) == 1

    st, body, _ = _post(port, "/generate", {"inputs": text, "parameters": {"max_new_tokens": 2}})
    assert st in (422, 424), body
    import urllib.request
    with urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5) as r:
        m = r.read().decode()
    for name in ('lorax_batch_inference_success{method="classify"}', 'lorax_batch_inference_success{method="embed"}',
                 "lorax_request_input_count_bucket", "lorax_request_classify_output_count_bucket"):
        assert name in m, name


def test_metrics_as_json(emb_stack):
    """`/metrics?format=json` (and `Accept: application/json`): the Prometheus families as {type, data: [{key, value}]}."""
    port = emb_stack["port"]
    _post(port, "/embed", {"inputs": "w1 w2"})
    with urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics?format=json", timeout=5) as r:
        assert r.status == 200
        m = json.loads(r.read().decode())
    fam = m["lorax_batch_inference_success"]
    assert fam["type"] == "counter" and any(d["key"].endswith('{method="embed"}') and d["value"] >= 1 for d in fam["data"])
    hist = m["lorax_request_input_count"]
    assert hist["type"] == "histogram" and {"sum", "count"} <= {d["key"] for d in hist["data"]}
    req = urllib.request.Request(f"http://127.0.0.1:{port}/metrics", headers={"Accept": "application/json"})
    with urllib.request.urlopen(req, timeout=5) as r:
        assert "lorax_batch_inference_success" in json.loads(r.read().decode())
    with urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5) as r:
        assert r.read().decode().startswith("# TYPE")


def test_token_classes_become_entities(emb_stack):
    """Labels in the B- / I- scheme are aggregated into entities with character offsets, as the reference's router does
    (router/src/infer.rs:1765-1819): the same rule restated in Python over the shard's per-token output."""
    port, rt = emb_stack["port"], emb_stack["rt"]
    saved = dict(rt.model.config.id2label)
    rt.model.config.id2label = {i: n for i, n in enumerate(["O", "B-PER", "I-PER", "B-LOC"])}
    try:
        text = "w5 w9 w77 w3 w300 w12 w8 w41 w6"
        labels, scores = rt.model.classify([rt.tokenize(text)])
        labels, scores = labels[0], scores[0]
        assert any("-" in l for l in labels)
        words = text.split()
        offs, p0 = [], 0
        for wd in words:
            a = text.index(wd, p0)
            offs.append((a, a + len(wd)))
            p0 = a + len(wd)
        want, cur, sc = [], None, []
        for (a, b), cls, s_ in zip(offs, labels, scores):
            parts = cls.split("-")
            bi, tag = (parts[0], parts[1]) if len(parts) == 2 else ("0", "0")
            if bi == "B" or (cur is not None and tag != cur["entity_group"]):
                if cur is not None:
                    want.append(cur)
                    sc = [s_]
                cur = {"entity_group": tag, "score": s_, "start": a, "end": b}
            elif cur is not None:
                sc.append(s_)
                cur["score"] = sum(sc) / len(sc)
                cur["end"] = b
        if cur is not None:
            want.append(cur)
        st, body, _ = _post(port, "/classify", {"inputs": text})
        assert st == 200, body
        got = json.loads(body)
        assert [(e["entity_group"], e["start"], e["end"]) for e in got] == [(e["entity_group"], e["start"], e["end"]) for e in want]
        assert all(abs(g["score"] - w["score"]) < 1e-4 for g, w in zip(got, want))
        assert all(g["word"] == text[g["start"]:g["end"]].lower() for g in got)
    finally:
        rt.model.config.id2label = saved


def test_python_clients_classify_and_embed(emb_stack):
    """The synchronous and the asyncio client against the routes of an embedding / token-classification deployment."""
    import asyncio
    from lorax_b200.client import AsyncClient, Client
    url = f"http://127.0.0.1:{emb_stack['port']}"
    c = Client(url)
    one = c.classify("w5 w9 w77")
    many = c.classify_batch(["w5 w9 w77", "w8"])
    assert len(one.entities) == 3 and len(many) == 2 and many[0].entities == one.entities
    assert len(c.embed("w5 w9").embeddings) == 64

    async def run():
        ac = AsyncClient(url)
        a = await ac.classify("w5 w9 w77")
        b = await ac.classify_batch(["w5 w9 w77", "w8"])
        e = await ac.embed("w5 w9")
        return a, b, e, await ac.health(), await ac.info()
    a, b, e, ok, info = asyncio.run(run())
    assert a.entities == one.entities and [x.entities for x in b] == [x.entities for x in many]
    assert len(e.embeddings) == 64 and ok and info["model_id"] == "tiny-distilbert"


def test_concurrent_inputs_share_shard_batches(emb_stack):
    """Embed / classify inputs go through a queue and a batching thread in the router: while one batch is on the shard the
    next one fills up, so concurrent HTTP calls end up in shared batches, each input still gets its own answer, and the queue
    and batch metrics of the generation path are reported for them (the reference schedules these entries through its batching
    task as well)."""
    import concurrent.futures as cf
    port, rt = emb_stack["port"], emb_stack["rt"]
    sizes = []
    real = rt.embed

    def slow_embed(req):
        sizes.append(len(req.batch.requests))
        time.sleep(0.05)                      # long enough for the other calls to queue up behind the first batch
        return real(req)
    rt.embed = slow_embed
    try:
        texts = [f"w{i} w{i + 1} w{(i * 7) % 500}" for i in range(24)]
        with cf.ThreadPoolExecutor(24) as pool:
            outs = list(pool.map(lambda t: _post(port, "/embed", {"inputs": t}), texts))
    finally:
        rt.embed = real
    assert all(st == 200 for st, _, _ in outs)
    for t, (_, body, _) in zip(texts, outs):
        want = rt.model.embed([rt.tokenize(t)])[0]
        got = json.loads(body)["embeddings"]
        assert max(abs(a - b) for a, b in zip(got, want)) < 1e-4
    assert sum(sizes) == 24 and len(sizes) < 24 and max(sizes) > 1, sizes
    with urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=5) as r:
        m = r.read().decode()
    for name in ("lorax_batch_next_size_bucket", "lorax_request_queue_duration_bucket", 'lorax_queue_length{kind="encoder"}',
                 'lorax_batch_inference_duration_bucket{method="embed"', "lorax_router_tokenizations"):
        assert name in m, name
    # a failing batch answers every input of it with an error and the route keeps working
    def broken(req):
        raise RuntimeError("encoder exploded")
    rt.embed = broken
    try:
        st, body, _ = _post(port, "/embed", {"inputs": "w1"})
    finally:
        rt.embed = real
    assert st == 424 and "error" in json.loads(body)
    st, _, _ = _post(port, "/embed", {"inputs": "w1"})
    assert st == 200
