"""Throughput of the SERVED path: HTTP clients -> C++ router -> shard runtime -> kernels, on one GPU.

    python benchmarks/bench_served.py [--model mistral-7b] [--adapters 100] [--concurrency 256] [--seconds 30]

Builds a random-weight model of the named architecture in this process, parks random rank-r adapters in the pinned
host tier, starts the framed-socket shard server and the `lorax-router` binary, then runs a closed-loop load generator
in a child process (so that it does not share the interpreter lock with the shard): `concurrency` clients, each sending
`POST /generate` with a random prompt of token ids, a Zipf-distributed adapter and a fixed number of new tokens.
Prints one JSON line: generated tokens per second in the measured window and latency percentiles from the router's
timing headers.
"""

from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import argparse
import asyncio
import json
import os
import random
import statistics
import subprocess
import sys
import time


# ---------------------------------------------------------------------------------------------- load generator (child)
async def _client_main(a):
    import aiohttp
    rng = random.Random(1234)
    weights = [1.0 / (i + 1) ** 1.1 for i in range(max(a.adapters, 1))]
    done = []
    t_start = time.perf_counter()
    t_measure = t_start + a.warmup_seconds
    t_end = t_measure + a.seconds

    async def worker(session):
        while time.perf_counter() < t_end:
            n = rng.randint(a.min_prompt, a.max_prompt)
            prompt = " ".join(str(rng.randrange(2, a.vocab)) for _ in range(n))
            params = {"max_new_tokens": a.new_tokens, "ignore_eos_token": True}
            if a.adapters:
                ad = rng.choices(range(a.adapters), weights)[0]
                params.update(adapter_id=f"synthetic-{ad}", adapter_source="local")
            t0 = time.perf_counter()
            try:
                async with session.post(a.url + "/generate", json={"inputs": prompt, "parameters": params}) as r:
                    await r.read()
                    t1 = time.perf_counter()
                    done.append(dict(status=r.status, t0=t0, t1=t1, tokens=int(r.headers.get("x-generated-tokens", 0)),
                                     tpt=float(r.headers.get("x-time-per-token", 0)), queue=float(r.headers.get("x-queue-time", 0)),
                                     infer=float(r.headers.get("x-inference-time", 0))))
            except Exception as e:
                done.append(dict(status=0, t0=t0, t1=time.perf_counter(), tokens=0, error=str(e)))

    conn = aiohttp.TCPConnector(limit=0)
    async with aiohttp.ClientSession(connector=conn, timeout=aiohttp.ClientTimeout(total=600)) as s:
        await asyncio.gather(*[worker(s) for _ in range(a.concurrency)])
    ok = [d for d in done if d["status"] == 200]
    # tokens of a request are credited to the window in proportion to the part of its life that falls into it
    toks = 0.0
    for d in ok:
        lo, hi = max(d["t0"], t_measure), min(d["t1"], t_end)
        if hi > lo:
            toks += d["tokens"] * (hi - lo) / max(d["t1"] - d["t0"], 1e-9)
    inwin = [d for d in ok if d["t1"] >= t_measure]
    med = lambda xs: statistics.median(xs) if xs else None
    print(json.dumps({"tokens_per_s": toks / a.seconds, "requests": len(ok), "failures": len(done) - len(ok),
                      "p50_time_per_token_ms": med([d["tpt"] for d in inwin]), "p50_queue_ms": med([d["queue"] for d in inwin]),
                      "p50_latency_s": med([d["t1"] - d["t0"] for d in inwin])}))


# ---------------------------------------------------------------------------------------------- server side (parent)
def _free_port() -> int:
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mistral-7b", choices=["mistral-7b", "llama3-8b", "tiny"])
    ap.add_argument("--adapters", type=int, default=100)
    ap.add_argument("--rank", type=int, default=16)
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--seconds", type=float, default=30.0)
    ap.add_argument("--warmup-seconds", type=float, default=15.0)
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=1024)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--client", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--url", default="")
    ap.add_argument("--vocab", type=int, default=32000)
    a = ap.parse_args()
    if a.client:
        asyncio.run(_client_main(a))
        return

    import tempfile
    import torch
    from lorax_b200 import config as cfgs
    from lorax_b200.adapters.lora import BlobLayout, pad_rank
    from lorax_b200.config import EngineConfig
    from lorax_b200.models.decoder import DecoderModel
    from lorax_b200.server.runtime import ShardRuntime
    from lorax_b200.server.transport import FramedServer

    on_gpu = torch.cuda.is_available()
    dev = torch.device("cuda", 0) if on_gpu else torch.device("cpu")
    dt = torch.bfloat16 if on_gpu else torch.float32
    mc = {"mistral-7b": cfgs.mistral_7b, "llama3-8b": cfgs.llama3_8b, "tiny": cfgs.tiny_llama}[a.model]()
    if a.model == "tiny" and on_gpu:
        mc.torch_dtype = "bfloat16"
    max_total = a.max_prompt + a.new_tokens + 32
    if on_gpu:
        model = DecoderModel.random_init_on_device(mc, dev, dt, seed=0, max_positions=max_total + 64)
    else:
        model = DecoderModel.random_init(mc, dev, dt, seed=0)
    rp = pad_rank(a.rank)
    units = BlobLayout(model, with_lm_head=False).units
    blob_elems = rp * units
    esz = 2 if on_gpu else 4
    ecfg = EngineConfig(max_input_length=a.max_prompt, max_total_tokens=max_total, max_batch_prefill_tokens=4096, compile=on_gpu,
                        host_adapter_cache_gb=blob_elems * esz * (a.adapters + 4) / (1 << 30) + 1)
    rt = ShardRuntime(model, None, ecfg, model_id=a.model, max_batch=a.concurrency,
                      adapter_arena_bytes=int(blob_elems * esz * (a.adapters + 2) * 1.02) + (64 << 20))
    g = torch.Generator(device=dev).manual_seed(99)
    units_rt = rt.adapters.layout.units
    for i in range(a.adapters):
        blob = torch.randn(rp * units_rt, generator=g, device=dev, dtype=torch.float32).mul_(0.02).to(dt)
        host = torch.empty(rp * units_rt, dtype=dt, pin_memory=on_gpu)
        host.copy_(blob)
        rt.adapters.register_blob(f"2:synthetic-{i}", host, rp)
    if on_gpu:
        torch.cuda.synchronize()

    tmp = tempfile.mkdtemp(prefix="lx-served-")
    uds = os.path.join(tmp, "shard")
    srv = FramedServer(rt, uds + "-0.lx").start()
    port = _free_port()
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    router = subprocess.Popen([os.path.join(here, "lorax_b200", "bin", "lorax-router"), "--port", str(port), "--hostname", "127.0.0.1",
                               "--master-shard-uds-path", uds, "--num-shard", "1", "--max-input-length", str(a.max_prompt),
                               "--max-total-tokens", str(max_total), "--max-batch-prefill-tokens", "4096", "--model-id", a.model,
                               "--adapter-source", "local", "--max-concurrent-requests", str(4 * a.concurrency),
                               "--max-active-adapters", str(max(a.adapters, 1) + 8)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    import urllib.request
    for _ in range(300):
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                if r.status == 200:
                    break
        except Exception:
            time.sleep(0.2)
    else:
        router.kill()
        raise RuntimeError("router did not come up: " + router.stdout.read().decode()[-2000:])
    try:
        out = subprocess.run([sys.executable, os.path.abspath(__file__), "--client", "--url", f"http://127.0.0.1:{port}",
                              "--adapters", str(a.adapters), "--concurrency", str(a.concurrency), "--seconds", str(a.seconds),
                              "--warmup-seconds", str(a.warmup_seconds), "--min-prompt", str(a.min_prompt), "--max-prompt", str(a.max_prompt),
                              "--new-tokens", str(a.new_tokens), "--vocab", str(mc.vocab_size)], capture_output=True, text=True, timeout=1800)
        line = out.stdout.strip().splitlines()[-1] if out.stdout.strip() else "{}"
        res = json.loads(line)
        res.update(model=a.model, adapters=a.adapters, concurrency=a.concurrency, fused_passes=rt.fused_stats,
                   metric="generated tokens/s over HTTP (router + shard), closed loop")
        print(json.dumps(res))
        if out.returncode != 0:
            print(out.stderr[-2000:], file=sys.stderr)
    finally:
        router.terminate()
        try:
            router.wait(timeout=10)
        except subprocess.TimeoutExpired:
            router.kill()
        srv.stop()
    os._exit(0)


if __name__ == "__main__":
    main()
