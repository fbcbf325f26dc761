"""`lorax-server` command line: `serve`, `download-weights`, `quantize` (same commands as the reference's
`server/lorax_server/cli.py:34-176`)."""

from __future__ import annotations

import argparse
import asyncio
import json
import os
import signal
import sys
import threading
import time

QUANTIZE_CHOICES = ["bitsandbytes", "bitsandbytes-nf4", "bitsandbytes-fp4", "gptq", "awq", "eetq", "hqq-4bit", "hqq-3bit", "hqq-2bit", "fp8", "fp8-kv"]


def _log(level: str, msg: str, as_json: bool):
    if as_json:
        print(json.dumps({"level": level, "target": "lorax_server", "message": msg}), flush=True)
    else:
        print(f"{level} {msg}", flush=True)


def serve(args):
    import torch
    from ..config import EngineConfig
    from ..parallel.tp import TensorParallel
    from .runtime import build_runtime
    from .transport import FramedServer, serve_grpc

    if args.dtype and args.quantize:
        raise SystemExit("Only 1 can be set between `dtype` and `quantize`, as they both decide how the final model is loaded")
    cfg = EngineConfig.from_env(model_id=args.model_id, max_input_length=args.max_input_length, max_total_tokens=args.max_total_tokens,
                                max_batch_prefill_tokens=args.max_batch_prefill_tokens, adapter_memory_fraction=args.adapter_memory_fraction,
                                compile=not args.no_compile, prefix_caching=args.prefix_caching, chunked_prefill=args.chunked_prefill,
                                speculative_tokens=args.speculative_tokens, quantize=args.quantize)
    tp = TensorParallel.init_from_env()
    dtype = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32, None: None}[args.dtype]
    _log("INFO", f"loading {args.model_id} on rank {tp.rank}/{tp.world_size}", args.json_output)
    merge = dict(merge_adapter=args.adapter_id, merge_adapter_source=args.adapter_source) if (args.merge_adapter_weights and args.adapter_id) else {}
    rt = build_runtime(args.model_id, cfg, tp=tp, dtype=dtype, source=args.source, revision=args.revision, device=args.device, **merge)
    if merge:
        args.adapter_id = ""                                # it is part of the base weights now
    if args.preloaded_adapter_ids:
        rt.preload_adapters([a.strip() for a in args.preloaded_adapter_ids.split(",")], {"hub": 0, "s3": 1, "local": 2, "pbase": 3}[args.preloaded_adapter_source or args.adapter_source])
    if args.adapter_id:
        rt.load_default_adapter(args.adapter_id, {"hub": 0, "s3": 1, "local": 2, "pbase": 3}[args.preloaded_adapter_source or args.adapter_source])
    from .tracing import PrefillProfiler, Tracer
    rt.tracer = Tracer(args.otlp_endpoint or os.environ.get("OTLP_ENDPOINT"), f"lorax.server-{tp.rank}")
    rt.profiler = PrefillProfiler(cfg.profiler_dir)
    framed = FramedServer(rt, f"{args.uds_path}-{tp.rank}.lx").start()
    _log("INFO", f"Server started at unix://{args.uds_path}-{tp.rank}", args.json_output)

    async def main():
        server = await serve_grpc(rt, args.uds_path, tp.rank, tp.world_size, lock=framed.lock)
        stop = asyncio.Event()
        loop = asyncio.get_running_loop()
        for s in (signal.SIGINT, signal.SIGTERM):
            loop.add_signal_handler(s, stop.set)
        await stop.wait()
        await server.stop(2)
    try:
        asyncio.run(main())
    finally:
        framed.stop()
        _log("INFO", "Signal received. Shutting down", args.json_output)


def download_weights(args):
    from ..utils.sources import resolve_model
    from ..utils.weights import weight_files
    d = resolve_model(args.model_id, args.source, args.revision)
    files = weight_files(d, args.extension)
    _log("INFO", f"{len(files)} weight file(s) ready under {d}", args.json_output)
    if args.adapter_id:              # the default adapter is fetched with the base model (cli.py:113-143 of the reference)
        from ..utils.sources import resolve_adapter
        a = resolve_adapter(args.adapter_id, args.adapter_source, args.api_token)
        _log("INFO", f"adapter {args.adapter_id} ready under {a}", args.json_output)


def quantize(args):
    from ..utils.quantize import quantize_checkpoint
    extra = {}
    if args.scheme == "gptq":
        extra = dict(bits=args.bits, group=args.groupsize, nsamples=args.nsamples, seqlen=args.seqlen, dataset=args.dataset,
                     damp=args.percdamp, act_order=args.act_order)
    stats = quantize_checkpoint(args.model_id, args.output_dir, method=args.scheme, **extra)
    _log("INFO", f"quantised checkpoint written to {args.output_dir}: {stats['quantized']} of {stats['tensors']} tensors in {args.scheme}",
         args.json_output)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="lorax-server")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve")
    s.add_argument("model_id")
    s.add_argument("--adapter-id", default="")
    s.add_argument("--revision", default=None)
    s.add_argument("--sharded", action="store_true")
    s.add_argument("--quantize", default=None, choices=QUANTIZE_CHOICES)
    s.add_argument("--dtype", default=None, choices=["float16", "bfloat16", "float32"])
    s.add_argument("--device", default=None)
    s.add_argument("--source", default="hub")
    s.add_argument("--adapter-source", default="hub")
    s.add_argument("--uds-path", default="/tmp/lorax-server")
    s.add_argument("--max-input-length", type=int, default=1024)
    s.add_argument("--max-total-tokens", type=int, default=2048)
    s.add_argument("--max-batch-prefill-tokens", type=int, default=4096)
    s.add_argument("--adapter-memory-fraction", type=float, default=0.1)
    s.add_argument("--speculative-tokens", type=int, default=0)
    s.add_argument("--preloaded-adapter-ids", default="")
    s.add_argument("--preloaded-adapter-source", default=None, help="source of --preloaded-adapter-ids (default: --adapter-source)")
    s.add_argument("--otlp-endpoint", default=None)
    s.add_argument("--merge-adapter-weights", action="store_true", help="fold --adapter-id into the base weights at load time")
    s.add_argument("--no-compile", action="store_true")
    s.add_argument("--prefix-caching", action="store_true")
    s.add_argument("--chunked-prefill", action="store_true")
    s.add_argument("--json-output", action="store_true")
    # options of the reference's shard CLI that select nothing here: graphs are on unless --no-compile, no remote code is ever
    # run, encoders report their own width, and log lines carry their level
    s.add_argument("--compile", action="store_true", help=argparse.SUPPRESS)
    s.add_argument("--trust-remote-code", action="store_true", help=argparse.SUPPRESS)
    s.add_argument("--embedding-dim", type=int, default=None, help=argparse.SUPPRESS)
    s.add_argument("--logger-level", default="INFO", help=argparse.SUPPRESS)
    s.set_defaults(fn=serve)
    d = sub.add_parser("download-weights")
    d.add_argument("model_id")
    d.add_argument("--revision", default=None)
    d.add_argument("--source", default="hub")
    d.add_argument("--extension", default=".safetensors")
    d.add_argument("--adapter-id", default="")
    d.add_argument("--adapter-source", default="hub")
    d.add_argument("--api-token", default=None)
    d.add_argument("--auto-convert", default="true", help=argparse.SUPPRESS)      # .bin checkpoints are always converted
    d.add_argument("--logger-level", default="INFO", help=argparse.SUPPRESS)
    d.add_argument("--embedding-dim", type=int, default=None, help=argparse.SUPPRESS)
    d.add_argument("--json-output", action="store_true")
    d.set_defaults(fn=download_weights)
    q = sub.add_parser("quantize")
    q.add_argument("model_id")
    q.add_argument("output_dir")
    q.add_argument("--scheme", default="gptq", choices=["fp8", "gptq"])
    q.add_argument("--bits", type=int, default=4, choices=[2, 4, 8])
    q.add_argument("--groupsize", type=int, default=128)
    q.add_argument("--nsamples", type=int, default=128)
    q.add_argument("--seqlen", type=int, default=2048)
    q.add_argument("--percdamp", type=float, default=0.01)
    q.add_argument("--act-order", action="store_true", help="quantise the most active input channels first (desc_act checkpoints)")
    q.add_argument("--dataset", default="", help="UTF-8 text file with one calibration sample per line (default: random token ids)")
    q.add_argument("--json-output", action="store_true")
    q.set_defaults(fn=quantize)
    args = ap.parse_args(argv)
    args.fn(args)


if __name__ == "__main__":
    main()
