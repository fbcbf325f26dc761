#!/usr/bin/env python
"""Headline benchmark: output tokens/s while serving 100 LoRA adapters on the Mistral-7B architecture.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched with torch.distributed.run)
    python bench.py --impl reference ...                     (the unmodified reference, if it could be installed)

Workload (synthetic, random-init weights): Mistral-7B, bf16, tensor parallel over N GPUs, 100 random LoRA
adapters of rank 16 on q,k,v,o,gate,up,down, adapter per request ~ Zipf(1.1), prompts of uniform-random token
ids with length uniform in [128, 1024], 256 new tokens, greedy.  By default 2000 requests arrive as a Poisson
stream at 400 requests/s, more than the engine serves, so a queue builds and the batch stays full
(`--arrivals closed` keeps `--batch` requests in flight instead).  Before the timed window a ramp fills the
decode batch, so the window measures the steady state.  A "step" is one iteration of the serving engine:
admission + prefill of newly arrived requests when the scheduler decides to, then one decode step over the
running batch.

Numbers reported.  `value` is device-timed with CUDA events over exactly K steps.  `p50_ttft_ms` (arrival to first
token, for every request admitted in the window), `p50_tpot_ms` and `p99_tpot_ms` (intervals between consecutive
tokens of running requests) come from the CUDA events the engine records with every step's results.  `e2e.value`
runs K more steps through the same public API (`Engine.add_request` / `Engine.step`) timed on the host clock; in
both windows every step copies the new requests' token ids from pinned host memory to the device and reads the
sampled tokens back, and the bytes of those copies are counted from the tensors.

Other configurations: `--model mixtral-8x7b` (experts on the device path), `--model llama3-8b --quantize fp8
--min-prompt 8192 --max-prompt 8192` (block-scaled fp8 weights, long prompts), `--ranks 8,16,32,64 --resident 32`
(mixed ranks, fewer HBM slots than adapters), `--kv-cache-dtype fp8` (e4m3 KV pages; named in `dtype`).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def reference_arm(args):
    """Tries the unmodified reference: its Python shard package as copied into baseline/_ref by
    baseline/install_reference.py (the package directory plus the protobuf stubs its Makefile would generate).  The
    stock Mistral path is imported in this process on this machine; when an import fails the JSON line names the
    module, the importing file and the other native modules of that path that are missing here."""
    import importlib
    import traceback
    if int(os.environ.get("RANK", "0")) != 0:        # launched one process per GPU: rank 0 prints the one line
        return 0
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "lorax_server")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/lorax_server is absent: run baseline/install_reference.py "
                          "<reference checkout> (pip cannot install the reference offline: no poetry-core backend)"}))
        return 0
    sys.path.insert(0, ref_root)
    try:
        import torch  # noqa: F401  (CUDA extensions link against torch's libraries)
    except Exception:
        pass
    missing = []
    # third-party modules the stock FlashMistral path imports (file:line in the reference's server/lorax_server)
    for mod, where in (("peft", "utils/adapter.py:13"), ("dropout_layer_norm", "models/custom_modeling/flash_mistral_modeling.py:24"),
                       ("rotary_emb", "layers/rotary.py:10"), ("flash_attn_2_cuda", "utils/flash_attn.py"),
                       ("punica_kernels", "utils/punica.py"), ("grpc_interceptor", "interceptor.py")):
        try:
            importlib.import_module(mod)
        except BaseException as e:      # a CUDA extension built for another torch raises ImportError/OSError
            missing.append(f"{mod} ({where}): {type(e).__name__}: {str(e)[:80]}")
    try:
        import torch  # noqa: F401
        importlib.import_module("lorax_server.models.flash_mistral")
        first = None
    except BaseException as e:
        tb = traceback.extract_tb(e.__traceback__)
        site = next((f"{fr.filename.split('_ref/')[-1]}:{fr.lineno}" for fr in reversed(tb) if "_ref/" in fr.filename), "?")
        first = f"{type(e).__name__}: {e} at {site}"
    if first is None and not missing:
        why = ("the reference's FlashMistral stack imports on this machine, but its router and launcher are Rust (no cargo) and no "
               "in-process driver for it ships with this benchmark")
    else:
        why = ("importing the reference's stock lorax_server.models.flash_mistral fails on this machine: " + (first or "ok") +
               "; modules of that path missing here: " + ("; ".join(missing) if missing else "none") +
               ". None is in the offline wheelhouse; dropout_layer_norm / rotary_emb / punica_kernels are CUDA extensions the "
               "reference builds from network-fetched sources for sm_80")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int, period_s: float = 0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def zipf_sampler(n: int, s: float, gen):
    import torch
    w = torch.tensor([1.0 / (k ** s) for k in range(1, n + 1)], dtype=torch.float64)
    w /= w.sum()
    cdf = w.cumsum(0)

    def draw():
        u = torch.rand(1, generator=gen, dtype=torch.float64)
        return int(torch.searchsorted(cdf, u).clamp(max=n - 1))
    return draw


def _finish(tp, eng=None):
    """World 1 returns to the interpreter.  With several ranks the NCCL communicator is not torn down (destroying a process
    group whose collectives were captured in CUDA graphs can block at interpreter exit): the graphs are dropped, the ranks
    meet at a barrier, the interpreter's exit handlers run, and the process leaves."""
    sys.stdout.flush()
    sys.stderr.flush()
    if tp.world_size == 1:
        return 0
    try:
        if eng is not None:
            eng.runner.graphs.clear()
        tp.barrier()
    except Exception:
        pass
    import atexit
    try:
        atexit._run_exitfuncs()
    except Exception:
        pass
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="mistral-7b", choices=["mistral-7b", "llama3-8b", "llama3-70b", "mixtral-8x7b", "tiny"])
    ap.add_argument("--batch", type=int, default=256, help="requests kept in flight")
    ap.add_argument("--adapters", type=int, default=100)
    ap.add_argument("--ranks", default="16", help="LoRA rank, or a comma list of ranks dealt round-robin over the adapters")
    ap.add_argument("--arrivals", default="poisson", choices=["poisson", "closed"])
    ap.add_argument("--requests", type=int, default=2000, help="poisson: number of arrivals")
    ap.add_argument("--rate", type=float, default=400.0, help="poisson: arrivals per second")
    ap.add_argument("--quantize", default=None, choices=[None, "fp8"], help="base linear weights in block-scaled fp8 e4m3")
    ap.add_argument("--kv-cache-dtype", default=None, choices=[None, "fp8"],
                    help="e4m3 KV pages (scale 1); a reduced-precision cache, never the headline configuration")
    ap.add_argument("--resident", type=int, default=None,
                    help="adapters that fit the HBM arena (default: all). Fewer makes the engine exchange adapters with the pinned host tier")
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=1024)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--layers", type=int, default=None, help="debug only: the reported config names the change")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--waiting-served-ratio", type=float, default=None, help="scheduler knob (default: the engine's)")
    ap.add_argument("--baseline-mode", action="store_true", help="NCCL collectives instead of the fused NVLink kernels")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    from lorax_b200 import config as cfgs
    from lorax_b200.adapters.manager import AdapterManager
    from lorax_b200.config import EngineConfig
    from lorax_b200.models.decoder import DecoderModel
    from lorax_b200.parallel.tp import TensorParallel
    from lorax_b200.runtime.engine import Engine, GenRequest

    if not torch.cuda.is_available():
        print(json.dumps({"error": "bench.py needs a CUDA device"}))
        return 1
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(json.dumps({"error": f"--gpus {args.gpus} must be launched with torch.distributed.run --nproc-per-node {args.gpus}"}))
            return 1
    tp = TensorParallel.init_from_env()
    dev = tp.device
    rank0 = tp.rank == 0

    mc = {"mistral-7b": cfgs.mistral_7b, "llama3-8b": cfgs.llama3_8b, "llama3-70b": cfgs.llama3_70b, "mixtral-8x7b": cfgs.mixtral_8x7b,
          "tiny": cfgs.tiny_llama}[args.model]()
    if args.model == "tiny":
        mc.torch_dtype = "bfloat16"
    if args.layers:
        mc.num_hidden_layers = args.layers
    max_total = args.max_prompt + args.new_tokens + 32
    t_setup = time.perf_counter()
    model = DecoderModel.random_init_on_device(mc, dev, torch.bfloat16, seed=0, tp=tp, max_positions=max_total + 64)
    if args.quantize == "fp8":
        model.quantize_fp8()
    if tp.world_size > 1 and not args.baseline_mode:
        try:
            from lorax_b200.parallel import fused
            fused.enable(tp, model)
        except Exception as e:  # fall back to NCCL, and say so
            if rank0:
                print(f"[bench] fused NVLink path unavailable ({e}); using NCCL", file=sys.stderr)

    # ---- adapters: random blobs generated on the device, parked in the pinned host tier, loaded through the exchange path
    esize = 2
    from lorax_b200.adapters.lora import BlobLayout, pad_rank
    layout_units = BlobLayout(model, with_lm_head=False).units
    ranks = [int(x) for x in str(args.ranks).split(",")]
    rps = [pad_rank(r) for r in ranks]
    elems = [rp * layout_units for rp in rps]                     # adapter a has rank ranks[a % len(ranks)]
    mean_elems = sum(elems) / len(elems)
    resident = args.adapters if args.resident is None else max(1, min(args.resident, args.adapters))
    arena_bytes = int(mean_elems * esize * (resident + 2) * 1.02) + int(max(elems) * esize) + (64 << 20)
    mgr = AdapterManager(model, arena_bytes=arena_bytes, host_bytes=int(mean_elems * esize * (args.adapters + 4)) + (64 << 20))
    g_dev = torch.Generator(device=dev).manual_seed(1234 + tp.rank)
    for a in range(args.adapters):
        n_el = elems[a % len(elems)]
        blob = torch.randn(n_el, generator=g_dev, device=dev, dtype=torch.float32).mul_(0.02).to(torch.bfloat16)
        host = torch.empty(n_el, dtype=torch.bfloat16, pin_memory=True)
        host.copy_(blob)
        mgr.register_blob(f"adapter-{a}", host, rps[a % len(rps)])
        del blob
    torch.cuda.synchronize(dev)
    for a in range(resident):
        assert mgr.load(a + 1, f"adapter-{a}"), "adapter arena too small"
    mgr.fence()
    torch.cuda.synchronize(dev)

    ecfg = EngineConfig(max_total_tokens=max_total, max_batch_prefill_tokens=max(4096, args.max_prompt), max_input_length=args.max_prompt,
                        compile=not args.no_graphs, kv_cache_dtype=args.kv_cache_dtype)
    if args.waiting_served_ratio is not None:
        ecfg.waiting_served_ratio = args.waiting_served_ratio
    eng = Engine(model, ecfg, max_batch=args.batch)
    for a in range(args.adapters):
        eng.register_adapter(a + 1, f"adapter-{a}")

    gen = torch.Generator().manual_seed(42)          # identical on every rank: ranks schedule in lockstep
    draw_adapter = zipf_sampler(args.adapters, 1.1, gen) if args.adapters > 0 else (lambda: -1)
    next_id = [1]
    meta = {}                                        # request id -> (arrival time, counts for latency stats)

    def new_request(ramp: bool = False, arrival: float = 0.0):
        n = int(torch.randint(args.min_prompt, args.max_prompt + 1, (1,), generator=gen))
        ids = torch.randint(0, mc.vocab_size, (n,), generator=gen).tolist()
        new = args.new_tokens
        if ramp:       # requests of the ramp start "mid flight" so that the batch is a steady-state mix of progress
            new = int(torch.randint(1, args.new_tokens + 1, (1,), generator=gen))
        r = GenRequest(next_id[0], ids, max_new_tokens=new, adapter_index=draw_adapter() + 1, ignore_eos_token=True,
                       arrival_time=arrival)
        next_id[0] += 1
        return r

    # ---- arrivals.  "poisson": `--requests` arrivals with exponential gaps at `--rate` requests/s on the wall clock that
    # starts when the ramp ends (every rank draws the same gaps and follows rank 0's clock through the step barrier of the
    # collectives; admission itself is deterministic given the queue).  "closed": a finished request is replaced at once.
    lat = {"ttft": [], "ttft_sched": [], "itl": []}
    last_tok = {}
    poisson = args.arrivals == "poisson"
    gaps = (torch.empty(args.requests, dtype=torch.float64).exponential_(args.rate, generator=gen).cumsum(0).tolist()
            if poisson else [])
    arr = {"next": 0, "t0": None, "admitted": 0}

    def feed(now: float):
        """Hand the engine every request whose arrival time has passed."""
        if not poisson:
            return
        if tp.world_size > 1:                        # one clock for all ranks: rank 0's
            now = tp.broadcast_scalar(now)
        while arr["next"] < len(gaps) and arr["t0"] + gaps[arr["next"]] <= now:
            r = new_request(arrival=arr["t0"] + gaps[arr["next"]])
            meta[r.request_id] = r.arrival_time
            eng.add_request(r)
            arr["next"] += 1

    ramping = [True]

    def harvest(events, record: bool = False):
        n = 0
        for ev in events:
            n += 1
            rid = ev.request_id
            if record:
                if ev.index == 0 and rid in meta:
                    lat["ttft"].append(ev.device_time - meta[rid])
                elif ev.index > 0 and rid in last_tok:
                    lat["itl"].append(ev.device_time - last_tok[rid])
            last_tok[rid] = ev.device_time
            if ev.finished:
                eng.finished.pop(rid, None)
                last_tok.pop(rid, None)
                meta.pop(rid, None)
                if not poisson or ramping[0]:        # closed loop (and the ramp of either mode): replace at once
                    r = new_request(arrival=time.perf_counter())
                    meta[r.request_id] = r.arrival_time
                    eng.add_request(r)
        return n

    # ---- ramp: fill the batch with requests that are "mid flight" and keep it full (finished requests are replaced at once)
    # until every row is taken, so that the timed windows see the steady-state mix of progress (not part of warm-up or timing)
    for _ in range(args.batch):
        eng.add_request(new_request(ramp=True))
    ramp_steps = 0
    while (len(eng.waiting) > 0 or len(eng.running) < args.batch - 8) and ramp_steps < 600:
        harvest(eng.step())
        ramp_steps += 1
    ramping[0] = False
    arr["t0"] = time.perf_counter()
    for _ in range(args.warmup):
        feed(time.perf_counter())
        harvest(eng.step())
    torch.cuda.synchronize(dev)
    setup_s = time.perf_counter() - t_setup

    def window(n_steps: int, device_timed: bool):
        runner = eng.runner
        h0, d0, l0 = runner.h2d_bytes, runner.d2h_bytes, runner.kernel_launches()
        p0 = dict(eng.stats)
        tp.barrier()
        torch.cuda.synchronize(dev)
        sampler = ClockSampler(dev.index or 0)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        toks = 0
        for _ in range(n_steps):
            feed(time.perf_counter())
            toks += harvest(eng.step(), record=True)
        e1.record()
        tp.barrier()
        torch.cuda.synchronize(dev)
        t1 = time.perf_counter()
        clocks = sampler.stop()
        dev_s = e0.elapsed_time(e1) / 1e3
        secs = tp.max_scalar(dev_s if device_timed else (t1 - t0))
        return dict(tokens=toks, seconds=secs, h2d=(runner.h2d_bytes - h0) / n_steps, d2h=(runner.d2h_bytes - d0) / n_steps,
                    launches=runner.kernel_launches() - l0, clocks=clocks,
                    prefill_tokens=eng.stats["prefill_tokens"] - p0["prefill_tokens"],
                    prefill_steps=eng.stats["prefill_steps"] - p0["prefill_steps"],
                    decode_steps=eng.stats["decode_steps"] - p0["decode_steps"],
                    adapter_loads=eng.stats.get("adapter_loads", 0) - p0.get("adapter_loads", 0))

    w1 = window(args.steps, device_timed=True)
    n_lat = {k: len(v) for k, v in lat.items()}
    w2 = window(args.steps, device_timed=False)
    if not rank0:
        return _finish(tp, eng)
    value = w1["tokens"] / w1["seconds"]
    e2e = w2["tokens"] / w2["seconds"]
    pct = lambda xs, q: (round(1e3 * sorted(xs)[min(len(xs) - 1, int(q * len(xs)))], 3) if xs else None)
    out = {
        "metric": "output tok/s at 100 adapters, Mistral-7B arch, TP1-8; p50 TTFT/TPOT",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": tp.world_size, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(1e3 * w1["seconds"] / args.steps, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": ("bf16" if not args.quantize else f"bf16 activations, {args.quantize} base weights")
                                     + (f", {args.kv_cache_dtype} KV cache" if args.kv_cache_dtype else ""),
        "data": "synthetic (random token ids, random-init base and adapter weights)",
        "impl": "ours",
        "config": {
            "model": args.model + (f"-{args.layers}layers-DEBUG" if args.layers else ""), "global_batch": args.batch,
            "seq_len": f"prompt U[{args.min_prompt},{args.max_prompt}] + {args.new_tokens} new",
            "parallelism": f"tp{tp.world_size}", "adapters": args.adapters, "resident_adapters": resident,
            "adapter_loads_in_window": w1["adapter_loads"], "lora_rank": args.ranks,
            "lora_targets": "q,k,v,o,gate,up,down", "adapter_choice": "zipf(1.1)",
            "arrivals": (f"poisson, {args.requests} requests at {args.rate:g}/s (more than the engine serves: the queue never empties), after a ramp "
                         f"that fills {args.batch} decode rows" if poisson else "closed loop (saturated)"),
            "requests_arrived": arr["next"] if poisson else None, "waiting_at_end": len(eng.waiting),
            "l2": "inputs larger than L2: each step streams >14 GB of weights, adapters and KV cache",
            "cuda_graphs": not args.no_graphs, "collectives": "nccl" if (args.baseline_mode or tp.fused is None) else "fused-nvlink",
            "prefill_tokens_in_window": w1["prefill_tokens"], "prefill_steps": w1["prefill_steps"], "decode_steps": w1["decode_steps"],
        },
        # device timestamps (CUDA events of the steps that produced the tokens) of both windows.  TTFT = first token - arrival, which
        # under saturating arrivals is mostly time in the queue; TPOT = gap between consecutive tokens of a running request.
        "p50_ttft_ms": pct(lat["ttft"], 0.5), "p50_tpot_ms": pct(lat["itl"], 0.5),
        "p99_tpot_ms": pct(lat["itl"], 0.99), "latency_samples": {"ttft": len(lat["ttft"]), "tpot": len(lat["itl"])},
        "clocks": {k: w1["clocks"][k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": round(w2["h2d"], 1),
                "d2h_bytes_per_step": round(w2["d2h"], 1), "timing": "host wall clock around Engine.step()",
                "clocks": {k: w2["clocks"][k] for k in ("sm_mhz", "sm_max_mhz", "reasons")}},
        "gpu_launches": int(w1["launches"]),
        "setup_s": round(setup_s, 1),
    }
    print(json.dumps(out))
    return _finish(tp, eng)


if __name__ == "__main__":
    sys.exit(main())
