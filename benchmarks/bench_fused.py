"""Fused row-parallel GEMM + all-reduce kernel against the NCCL baseline (GEMM kernel, then `all_reduce`), with the
roofline of the fused path: the slower of FLOPs / measured GEMM peak and NVLink bytes / measured link bandwidth.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_fused.py

Both arms are captured in a CUDA graph (20 calls rotating through >126 MB of weights) and device-timed; the number
reported is the maximum over ranks.  With `--allreduce` the two-shot all-reduce kernel is timed against NCCL's instead.
"""

from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import json
import math
import os

import torch
import torch.distributed as dist

from lorax_b200.ops import native
from lorax_b200.parallel.tp import TensorParallel

NVLINK_GBS = 770.0         # measured peer copy bandwidth per direction on this machine class
PEAK_TFLOPS = 1640.9


def gtime(fn, n_rot, reps=20):
    for i in range(3):
        fn(i % n_rot)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            fn(i % n_rot)
    g.replay()
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(5):
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        torch.cuda.synchronize()
        best = min(best, s.elapsed_time(e) * 1e3 / reps)
    t = torch.tensor([best], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bench_allreduce(tp):
    """Two-shot all-reduce kernel against NCCL's all-reduce on bf16 [T, 4096]; results are compared bit for bit."""
    from lorax_b200.parallel import fused
    fc = fused.FusedCollectives(tp, n_max=4096, max_rows=512)
    fc.setup_all_reduce(4352, 4096)
    for T in (16, 256, 1216, 4096):
        x = torch.randn(T, 4096, device="cuda", dtype=torch.bfloat16)
        src = fc.all_reduce_input(T, 4096)
        src.copy_(x)
        want = x.clone()
        dist.all_reduce(want)
        got = fc.all_reduce(src).clone()
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        t_nccl = gtime(lambda i: dist.all_reduce(x), 1)
        t_mine = gtime(lambda i: fc.all_reduce(src), 1)
        fc.check()
        if tp.rank == 0:
            print(json.dumps(dict(op="all_reduce", T=T, mbytes=round(T * 4096 * 2 / 1e6, 1), world=tp.world_size, nccl_us=round(t_nccl, 1),
                                  two_shot_us=round(t_mine, 1), max_abs_diff=err)), flush=True)
    dist.barrier()
    os._exit(0)


def main():
    import sys
    tp = TensorParallel.init_from_env()
    ws = tp.world_size
    if "--allreduce" in sys.argv:
        bench_allreduce(tp)
    from lorax_b200.parallel import fused

    class _M:
        hidden = 4096
    fc = fused.FusedCollectives(tp, n_max=4096, max_rows=512)
    results = []
    for name, N, Kfull in (("o_proj", 4096, 4096), ("down_proj", 4096, 14336)):
        K = Kfull // ws
        n_rot = max(2, int(math.ceil(300e6 / (N * K * 2))))
        wts = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / K ** 0.5 for _ in range(n_rot)]
        for T in (8, 32, 64, 128, 256):
            x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
            out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)

            def base(i):
                native.gemm(x, wts[i], out=out)
                dist.all_reduce(out)
            t_fused = gtime(lambda i: fc.gemm_allreduce(x, wts[i]), n_rot)
            t_base = gtime(base, n_rot)
            t_gemm = gtime(lambda i: native.gemm(x, wts[i], out=out), n_rot)
            fc.check()
            flops = 2.0 * T * N * K
            link_bytes = (ws - 1) / ws * T * N * (4 + 2)
            roof_us = max(flops / (PEAK_TFLOPS * 1e12), link_bytes / (NVLINK_GBS * 1e9), N * K * 2 / 6.5389e12) * 1e6
            results.append(dict(op=name, T=T, N=N, K_per_rank=K, world=ws, fused_us=round(t_fused, 2), gemm_plus_nccl_us=round(t_base, 2),
                                gemm_only_us=round(t_gemm, 2), roofline_us=round(roof_us, 2), fused_frac_of_roofline=round(roof_us / t_fused, 3)))
            if tp.rank == 0:
                print(json.dumps(results[-1]), flush=True)
    if tp.rank == 0 and os.environ.get("LX_BENCH_OUT"):
        with open(os.environ["LX_BENCH_OUT"], "w") as f:
            json.dump(results, f, indent=1)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
