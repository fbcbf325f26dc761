"""Per-operator device-time breakdown of one prefill step and one decode step of the serving engine.

    python benchmarks/profile_step.py [--model mistral-7b] [--batch 256] [--ctx 700] [--prefill 1024] [--adapters 100]

Runs the steps eagerly (no CUDA graph) with every operator bracketed by CUDA events, so the numbers include the
launch gap of each kernel; the shares tell where a step spends its time.  With `--graph-steps N` the decode step is captured
in a CUDA graph and replayed N times instead (the serving path); a launch list taken over that run gives each kernel's own time.
"""

from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import argparse
import json

import torch

from lorax_b200 import config as cfgs
from lorax_b200.adapters.lora import BlobLayout, pad_rank
from lorax_b200.adapters.manager import AdapterManager
from lorax_b200.models.decoder import DecoderModel
from lorax_b200.ops import native
from lorax_b200.runtime.kv_cache import KVCache
from lorax_b200.runtime.runner import ModelRunner, PrefillItem


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mistral-7b")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=700)
    ap.add_argument("--prefill", type=int, default=1024)
    ap.add_argument("--adapters", type=int, default=100)
    ap.add_argument("--rank", type=int, default=16)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--json", default=None)
    ap.add_argument("--graph-steps", type=int, default=0,
                    help="instead of the eager breakdown, replay the captured decode graph this many times and print the mean step "
                         "time; under `ncu --metrics gpu__time_duration.sum` this lists every kernel of a decode step")
    a = ap.parse_args()
    mc = {"mistral-7b": cfgs.mistral_7b, "llama3-8b": cfgs.llama3_8b, "tiny": cfgs.tiny_llama}[a.model]()
    if a.layers:
        mc.num_hidden_layers = a.layers
    dev = torch.device("cuda", 0)
    model = DecoderModel.random_init_on_device(mc, dev, torch.bfloat16, max_positions=4096)
    rp = pad_rank(a.rank)
    units = BlobLayout(model, with_lm_head=False).units
    n = rp * units
    mgr = AdapterManager(model, arena_bytes=(a.adapters + 1) * n * 2 + (64 << 20), host_bytes=(a.adapters + 2) * n * 2)
    for i in range(a.adapters):
        blob = (torch.randn(n, device=dev) * 0.02).to(torch.bfloat16)
        host = torch.empty(n, dtype=torch.bfloat16, pin_memory=True)
        host.copy_(blob)
        mgr.register_blob(f"a{i}", host, rp)
        mgr.load(i + 1, f"a{i}")
    mgr.fence()
    page = 32
    blocks_per = (a.ctx + 64 + page - 1) // page
    kv = KVCache(mc.num_hidden_layers, a.batch * blocks_per + 64, model.nkv, model.d, torch.bfloat16, dev)
    runner = ModelRunner(model, kv, max_batch=a.batch, max_seq_tokens=a.ctx + 64, max_prefill_tokens=max(a.prefill, 4096), use_graphs=a.graph_steps > 0)
    g = torch.Generator().manual_seed(0)
    rows = [runner.state.take_row(i) for i in range(a.batch)]
    blocks = [[1 + i * blocks_per + j for j in range(blocks_per)] for i in range(a.batch)]
    ads = [int(torch.randint(0, a.adapters + 1, (1,), generator=g)) for _ in range(a.batch)] if a.adapters else [0] * a.batch
    runner.install(rows, [1] * a.batch, [a.ctx] * a.batch, blocks, ads)
    runner.resort()
    results = {}
    if a.graph_steps:
        for _ in range(3):
            runner.decode()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.graph_steps):
            runner.decode()
        e1.record()
        torch.cuda.synchronize()
        native.workspace().check_status()
        key = next(iter(runner.graph_kernels))
        print(json.dumps(dict(batch=a.batch, ctx=a.ctx, layers=mc.num_hidden_layers, graph_steps=a.graph_steps,
                              kernels_per_step=runner.graph_kernels[key], step_ms=round(e0.elapsed_time(e1) / a.graph_steps, 3))))
        return
    # ---- decode
    for _ in range(2):
        runner.decode()
    torch.cuda.synchronize()
    native.enable_timing()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    runner.decode()
    e1.record()
    rep = native.timing_report()
    results["decode"] = dict(batch=a.batch, ctx=a.ctx, step_ms=round(e0.elapsed_time(e1), 3), ops=rep)
    # ---- prefill (two sequences with different adapters)
    native.disable_timing()
    half = a.prefill // 2
    items = [PrefillItem(torch.randint(0, mc.vocab_size, (half,), generator=g).tolist(), 0, blocks[i], adapter_index=ads[i]) for i in range(2)]
    runner.prefill(items)
    torch.cuda.synchronize()
    native.enable_timing()
    e0.record()
    runner.prefill(items)
    e1.record()
    rep = native.timing_report()
    results["prefill"] = dict(tokens=2 * half, step_ms=round(e0.elapsed_time(e1), 3), ops=rep)
    native.workspace().check_status()
    for phase, r in results.items():
        print(f"== {phase}: {json.dumps({k: v for k, v in r.items() if k != 'ops'})}")
        tot = sum(o["total_ms"] for o in r["ops"])
        for o in r["ops"]:
            print(f"  {o['op']:16s} {o['shapes']:44s} calls {o['calls']:4d}  total {o['total_ms']:8.3f} ms ({100 * o['total_ms'] / tot:5.1f}%)  mean {o['mean_us']:8.2f} us")
    if a.json:
        with open(a.json, "w") as f:
            json.dump(results, f, indent=1)


if __name__ == "__main__":
    main()
