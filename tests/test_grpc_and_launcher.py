"""The gRPC face of the shard (generate.v1.LoraxService over a unix socket, runtime-built descriptors) and the
C++ launcher supervising a shard + router."""
import asyncio
import json
import os
import signal
import socket
import subprocess
import sys
import time
import urllib.request

import pytest
import torch
from safetensors.torch import save_file

from lorax_b200.config import EngineConfig, tiny_llama
from lorax_b200.models.decoder import DecoderModel
from lorax_b200.models.loading import export_hf_state_dict

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LAUNCHER = os.path.join(REPO, "lorax_b200", "bin", "lorax-launcher")


def _model_dir(root):
    from tokenizers import Tokenizer, models, pre_tokenizers
    cfg = tiny_llama(vocab_size=512)
    model = DecoderModel.random_init(cfg, "cpu", torch.float32, seed=0)
    mdir = root / "model"
    mdir.mkdir()
    save_file(export_hf_state_dict(model), str(mdir / "model.safetensors"), metadata={"format": "pt"})
    (mdir / "config.json").write_text(json.dumps(cfg.to_dict()))
    vocab = {f"w{i}": i for i in range(512)}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="w0"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(mdir / "tokenizer.json"))
    return mdir


def test_grpc_contract(tmp_path):
    import grpc
    from lorax_b200.server.proto import load_pb
    from lorax_b200.server.runtime import build_runtime
    from lorax_b200.server.transport import serve_grpc
    pb = load_pb()
    mdir = _model_dir(tmp_path)
    rt = build_runtime(str(mdir), EngineConfig(max_input_length=64, max_total_tokens=128, max_batch_prefill_tokens=256, compile=False),
                       device="cpu", dtype=torch.float32, source="local", num_blocks=64, max_batch=8)
    uds = str(tmp_path / "s")

    async def run():
        server = await serve_grpc(rt, uds, 0, 1)
        async with grpc.aio.insecure_channel(f"unix://{uds}-0") as ch:
            def call(name, req):
                rq, rs = pb.RPCS[name]
                return ch.unary_unary(f"/{pb.SERVICE}/{name}", request_serializer=rq.SerializeToString, response_deserializer=rs.FromString)(req)
            info = await call("Info", pb.InfoRequest())
            assert info.block_size == 32 and info.supports_generation and info.requires_block_allocator
            sd = await call("ServiceDiscovery", pb.ServiceDiscoveryRequest())
            assert list(sd.urls) == [f"unix://{uds}-0"]
            req = pb.Request(id=0, inputs="w1 w2 w3", truncate=64, adapter_index=0, blocks=[1, 2],
                             parameters=pb.NextTokenChooserParameters(temperature=1.0, top_p=1.0, typical_p=1.0, repetition_penalty=1.0),
                             stopping_parameters=pb.StoppingCriteriaParameters(max_new_tokens=3, ignore_eos_token=True))
            resp = await call("Prefill", pb.PrefillRequest(batch=pb.Batch(id=7, requests=[req], size=1, max_tokens=6)))
            assert len(resp.generations) == 1 and resp.batch.id == 7 and list(resp.batch.request_ids) == [0]
            toks = [resp.generations[0].next_tokens.ids[0]]
            cached = resp.batch
            while True:
                d = await call("Decode", pb.DecodeRequest(batches=[cached]))
                toks.append(d.generations[0].next_tokens.ids[0])
                if d.generations[0].HasField("generated_text"):
                    assert d.generations[0].generated_text.generated_tokens == 3
                    assert not d.HasField("batch")
                    break
                cached = d.batch
            assert len(toks) == 3
            # an unknown batch is an INTERNAL error, and the server keeps working
            with pytest.raises(grpc.aio.AioRpcError) as ei:
                await call("Decode", pb.DecodeRequest(batches=[pb.CachedBatch(id=99)]))
            assert ei.value.code() == grpc.StatusCode.INTERNAL
            await call("Health", pb.HealthRequest())
        await server.stop(0)
    asyncio.run(run())


@pytest.mark.parametrize("num_shard", [1, 2])
def test_launcher_supervises_shard_and_router(tmp_path, num_shard):
    """`lorax-launcher` end to end on CPU: one shard, and two tensor-parallel shards (Gloo) behind one router."""
    from lorax_b200.csrc import build
    build.build_host()
    mdir = _model_dir(tmp_path)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, PYTHONPATH=REPO, CUDA_VISIBLE_DEVICES="", LORAX_COMPILE="0")
    proc = subprocess.Popen([LAUNCHER, "--model-id", str(mdir), "--source", "local", "--port", str(port), "--hostname", "127.0.0.1",
                             "--shard-uds-path", str(tmp_path / "uds"), "--python", sys.executable, "--max-input-length", "64",
                             "--max-total-tokens", "128", "--json-output", "--master-port", str(29611 + num_shard), "--num-shard", str(num_shard)],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    try:
        ok = False
        for _ in range(600):
            if proc.poll() is not None:
                break
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                    ok = r.status == 200
                    break
            except Exception:
                time.sleep(0.2)
        if not ok:
            proc.kill()
            raise AssertionError("deployment did not come up:\n" + proc.stdout.read().decode()[-9000:])
        req = urllib.request.Request(f"http://127.0.0.1:{port}/generate", data=json.dumps({"inputs": "w1 w2", "parameters": {"max_new_tokens": 3}}).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=60) as r:
            text = json.loads(r.read())["generated_text"]
        # tensor parallelism must not change the tokens: compare with the single-process model
        from lorax_b200.config import EngineConfig
        from lorax_b200.server.runtime import build_runtime
        rt = build_runtime(str(mdir), EngineConfig(max_input_length=64, max_total_tokens=128, compile=False), device="cpu",
                           dtype=torch.float32, source="local", num_blocks=64, max_batch=4)
        ids = rt.tokenize("w1 w2")
        from lorax_b200.runtime.engine import Engine
        eng = Engine(rt.model, EngineConfig(max_total_tokens=128, max_batch_prefill_tokens=256), num_blocks=64, max_batch=2)
        want = eng.generate([ids], max_new_tokens=3, eos_token_ids=frozenset(rt.eos_ids))[0]
        assert text.strip() == rt.tokenizer.decode(want, skip_special_tokens=True).strip(), (text, want)
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
            raise
    out = proc.stdout.read().decode()
    assert "shard 0 ready" in out and proc.returncode == 0, out[-2000:]
    if num_shard == 2:
        assert "shard 1 ready" in out


@pytest.mark.gpu
def test_launcher_two_gpu_shards(tmp_path):
    """Two CUDA shards (NCCL + the in-kernel NVLink collectives) behind the router, started by the launcher."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from lorax_b200.csrc import build
    build.build_host()
    mdir = _model_dir(tmp_path)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, PYTHONPATH=REPO, NCCL_NVLS_ENABLE="0", LORAX_B200_DEBUG="1")
    proc = subprocess.Popen([LAUNCHER, "--model-id", str(mdir), "--source", "local", "--port", str(port), "--hostname", "127.0.0.1",
                             "--shard-uds-path", str(tmp_path / "uds"), "--python", sys.executable, "--max-input-length", "64",
                             "--max-total-tokens", "128", "--json-output", "--master-port", "29631", "--num-shard", "2", "--dtype", "bfloat16"],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    try:
        ok = False
        for _ in range(900):
            if proc.poll() is not None:
                break
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                    ok = r.status == 200
                    break
            except Exception:
                time.sleep(0.2)
        if not ok:
            proc.kill()
            raise AssertionError("deployment did not come up:\n" + proc.stdout.read().decode()[-9000:])
        outs = []
        for n in (3, 9):
            req = urllib.request.Request(f"http://127.0.0.1:{port}/generate",
                                         data=json.dumps({"inputs": "w1 w2 w7 w9", "parameters": {"max_new_tokens": n, "ignore_eos_token": True, "details": True}}).encode(),
                                         headers={"Content-Type": "application/json"})
            try:
                with urllib.request.urlopen(req, timeout=120) as r:
                    j = json.loads(r.read())
            except urllib.error.HTTPError as e:
                proc.send_signal(signal.SIGTERM)
                raise AssertionError(f"HTTP {e.code}: {e.read().decode()[:600]}\n" + proc.stdout.read().decode()[-9000:])
            assert j["details"]["generated_tokens"] == n
            outs.append([t["id"] for t in j["details"]["tokens"]])
        assert outs[1][:3] == outs[0]
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.wait(timeout=60)
        except subprocess.TimeoutExpired:
            proc.kill()
            raise
    out = proc.stdout.read().decode()
    assert "shard 1 ready" in out and proc.returncode == 0, out[-2000:]


def test_launcher_accepts_the_reference_flag_set(tmp_path):
    """Flags of the reference launcher beyond the core set (launcher/src/main.rs:273-655): the ones that configure something
    reach the shard or the router (CORS headers, validation workers, eager mode, shard count), the ones that choose between code
    paths that do not exist here are accepted with a warning, `--download-only` stops after the download, and invalid
    combinations are refused before anything is spawned."""
    from lorax_b200.csrc import build
    build.build_host()
    mdir = _model_dir(tmp_path)
    base = [LAUNCHER, "--model-id", str(mdir), "--source", "local", "--python", sys.executable, "--json-output",
            "--shard-uds-path", str(tmp_path / "uds"), "--hostname", "127.0.0.1"]
    env = dict(os.environ, PYTHONPATH=REPO, CUDA_VISIBLE_DEVICES="", LORAX_COMPILE="0")
    r = subprocess.run(base + ["--ngrok"], capture_output=True, env=env, timeout=60)
    assert r.returncode == 2 and b"ngrok" in r.stdout
    r = subprocess.run(base + ["--sharded", "true"], capture_output=True, env=env, timeout=60)
    assert r.returncode == 2 and b"sharded" in r.stdout
    r = subprocess.run(base + ["--validation-workers", "0"], capture_output=True, env=env, timeout=60)
    assert r.returncode == 2 and b"validation_workers" in r.stdout
    r = subprocess.run(base + ["--download-only"], capture_output=True, env=env, timeout=300)
    assert r.returncode == 0 and b"--download-only: not starting shards" in r.stdout and b"shard 0 ready" not in r.stdout
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    proc = subprocess.Popen(base + ["--port", str(port), "--max-input-length", "64", "--max-total-tokens", "128", "--sharded", "false", "--eager",
                                    "--validation-workers", "3", "--cors-allow-origin", "*", "--cors-allow-credentials", "true",
                                    "--cors-expose-header", "x-compute-time", "--cors-allow-method", "GET, POST", "--compile-max-batch-size", "8",
                                    "--compile-max-rank", "16", "--disable-sgmv", "--trust-remote-code", "--backend", "flashinfer",
                                    "--default-adapter-source", "local", "--memory-wiggle-room", "0.9", "--skip-download"],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    try:
        ok = False
        for _ in range(600):
            if proc.poll() is not None:
                break
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as resp:
                    ok = resp.status == 200
                    break
            except Exception:
                time.sleep(0.2)
        if not ok:
            proc.kill()
            raise AssertionError("deployment did not come up:\n" + proc.stdout.read().decode()[-9000:])
        req = urllib.request.Request(f"http://127.0.0.1:{port}/info", headers={"Origin": "http://app.example"})
        with urllib.request.urlopen(req, timeout=30) as resp:
            info = json.loads(resp.read())
            hdr = {k.lower(): v for k, v in resp.headers.items()}
        assert info["validation_workers"] == 3
        assert hdr["access-control-allow-origin"] == "http://app.example" and hdr["access-control-allow-credentials"] == "true"
        assert hdr["access-control-expose-headers"] == "x-compute-time"
        req = urllib.request.Request(f"http://127.0.0.1:{port}/generate", method="OPTIONS", headers={"Origin": "http://app.example"})
        with urllib.request.urlopen(req, timeout=30) as resp:
            assert resp.status == 204 and resp.headers["Access-Control-Allow-Methods"] == "GET, POST"
        req = urllib.request.Request(f"http://127.0.0.1:{port}/generate", data=json.dumps({"inputs": "w1 w2", "parameters": {"max_new_tokens": 2}}).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=60) as resp:
            assert "generated_text" in json.loads(resp.read())
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
            raise
    out = proc.stdout.read().decode()
    assert proc.returncode == 0 and "starting 1 shard(s)" in out, out[-2000:]
    for flag in ("--backend", "--disable-sgmv", "--trust-remote-code"):
        assert f"{flag} is accepted for compatibility" in out


def test_download_weights_fetches_the_default_adapter(tmp_path, capsys):
    """`lorax-server download-weights <model> --adapter-id <adapter>`: the step the launcher runs before the shards start makes
    the base weights and the default adapter available, and fails when either is missing."""
    from lorax_b200.adapters.lora import random_adapter, save_peft_adapter
    from lorax_b200.server import cli
    mdir = _model_dir(tmp_path)
    c, mm = random_adapter(tiny_llama(vocab_size=512), r=8, alpha=16, target_modules=["q_proj", "v_proj"], seed=1)
    save_peft_adapter(tmp_path / "ad", c, mm)
    cli.main(["download-weights", str(mdir), "--source", "local", "--adapter-id", str(tmp_path / "ad"), "--adapter-source", "local",
              "--json-output", "--logger-level", "INFO"])
    out = capsys.readouterr().out
    assert "1 weight file(s) ready" in out and f"adapter {tmp_path / 'ad'} ready" in out
    with pytest.raises(Exception):
        cli.main(["download-weights", str(mdir), "--source", "local", "--adapter-id", str(tmp_path / "nope"), "--adapter-source", "local"])


def test_router_speaks_grpc_to_the_shard(tmp_path):
    """`lorax-router --shard-transport grpc`: the router's own HTTP/2 client reaches the shard's grpcio endpoint on
    `unix://{uds}-0` for the service's RPCs (the tokenizer helpers stay on the framed socket).  A generation gives the tokens the
    framed transport gives, a prompt longer than one flow-control window goes through, and a shard-side exception reaches the
    HTTP client as text."""
    import asyncio
    import json
    import subprocess
    import threading
    import time
    import urllib.error
    import urllib.request
    from lorax_b200.csrc import build
    from lorax_b200.server.runtime import build_runtime
    from lorax_b200.server.transport import FramedServer, serve_grpc
    from test_full_stack import ROUTER, _free_port, _post
    build.build_host()
    mdir = _model_dir(tmp_path)
    rt = build_runtime(str(mdir), EngineConfig(max_input_length=1900, max_total_tokens=1964, max_batch_prefill_tokens=2000, compile=False),
                       device="cpu", dtype=torch.float32, source="local", num_blocks=128, max_batch=8)
    uds = str(tmp_path / "s")
    framed = FramedServer(rt, uds + "-0.lx").start()
    loop = asyncio.new_event_loop()
    started = threading.Event()
    holder = {}

    def grpc_thread():
        asyncio.set_event_loop(loop)

        async def main():
            holder["server"] = await serve_grpc(rt, uds, 0, 1, lock=framed.lock)
            started.set()
            await holder["server"].wait_for_termination()
        loop.run_until_complete(main())
    th = threading.Thread(target=grpc_thread, daemon=True)
    th.start()
    assert started.wait(20)
    outs = {}
    procs = []
    try:
        for transport in ("framed", "grpc"):
            port = _free_port()
            proc = subprocess.Popen([ROUTER, "--port", str(port), "--hostname", "127.0.0.1", "--master-shard-uds-path", uds, "--num-shard", "1",
                                     "--max-input-length", "1900", "--max-total-tokens", "1964", "--max-batch-prefill-tokens", "2000",
                                     "--model-id", "tiny", "--shard-transport", transport], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
            procs.append(proc)
            for _ in range(100):
                try:
                    with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                        if r.status == 200:
                            break
                except Exception:
                    time.sleep(0.1)
            else:
                proc.kill()
                raise RuntimeError("router did not come up: " + proc.stdout.read().decode()[-2000:])
            st, body, _ = _post(port, "/generate", {"inputs": "w1 w2 w3 w4", "parameters": {"max_new_tokens": 5, "details": True}})
            assert st == 200, body
            outs[transport] = [t["id"] for t in json.loads(body)["details"]["tokens"]]
            if transport == "grpc":
                # 1500 long (unknown) words: the request message is larger than HTTP/2's default 65535-byte windows
                long_prompt = " ".join("x" * 60 + str(i) for i in range(1500))
                assert len(long_prompt) > 90000
                st, body, _ = _post(port, "/generate", {"inputs": long_prompt, "parameters": {"max_new_tokens": 2}})
                assert st == 200, body[:300]
                # a failing shard call: the message travels in the trailers
                inner = rt.prefill

                def boom(req):
                    raise RuntimeError("the shard says no: 100% sure")
                rt.prefill = boom
                try:
                    st, body, _ = _post(port, "/generate", {"inputs": "w1 w2", "parameters": {"max_new_tokens": 2}})
                finally:
                    rt.prefill = inner
                assert st == 424 and "the shard says no: 100% sure" in body, (st, body)
                st, body, _ = _post(port, "/generate", {"inputs": "w1 w2 w3 w4", "parameters": {"max_new_tokens": 5, "details": True}})
                assert st == 200 and [t["id"] for t in json.loads(body)["details"]["tokens"]] == outs["grpc"]
        assert outs["framed"] == outs["grpc"] and len(outs["grpc"]) == 5
    finally:
        for proc in procs:
            proc.terminate()
            try:
                proc.wait(timeout=10)
            except subprocess.TimeoutExpired:
                proc.kill()
        loop.call_soon_threadsafe(lambda: asyncio.ensure_future(holder["server"].stop(0)))
        framed.stop()
