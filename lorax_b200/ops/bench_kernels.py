"""Micro-benchmarks of the CUDA kernels against their roofline (and cuBLAS for the GEMM).

``python -m lorax_b200.ops.bench_kernels [--json out.json]`` times each kernel with CUDA events after a
warm-up, rotating through enough distinct buffers that the working set exceeds the 126 MB L2.
"""

from __future__ import annotations

import argparse
import json
import math

import torch

from lorax_b200.ops import native


def _time(fn, n_rot: int, iters: int = 20, warmup: int = 3) -> float:
    """Median milliseconds per call; fn(i) uses buffer set i % n_rot."""
    for i in range(warmup):
        fn(i % n_rot)
    torch.cuda.synchronize()
    times = []
    for i in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn(i % n_rot)
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def bench_gemm(results, peaks):
    shapes = [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336), ("lm_head", 32000, 4096)]
    for T in (1, 16, 64, 128, 256, 1024, 4096):
        for name, N, K in shapes:
            wbytes = N * K * 2
            n_rot = max(2, int(math.ceil(300e6 / wbytes)))
            ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(n_rot)]
            x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
            out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
            ms = _time(lambda i: native.gemm(x, ws[i], out=out), n_rot)
            ms_cublas = _time(lambda i: torch.matmul(x, ws[i].t(), out=out), n_rot)
            native.workspace().check_status()
            flops = 2.0 * T * N * K
            bytes_ = wbytes + T * K * 2 + T * N * 2
            results.append({
                "kernel": "gemm_bf16_tcgen05", "shape": f"{name} T={T} N={N} K={K}", "ms": round(ms, 4),
                "cublas_ms": round(ms_cublas, 4), "tflops": round(flops / ms / 1e9, 1), "gbs": round(bytes_ / ms / 1e6, 1),
                "frac_of_measured_hbm": round(bytes_ / ms / 1e6 / peaks["hbm_gbs"], 3),
                "frac_of_measured_bf16": round(flops / ms / 1e9 / peaks["bf16_tflops"], 3),
            })
            print(results[-1], flush=True)
            del ws


def bench_attn_decode(results, peaks):
    nh, nkv, d, page = 32, 8, 128, 32
    for B, ctx in ((16, 1024), (64, 1024), (256, 700), (256, 2048), (8, 8192)):
        blocks_per = (ctx + page - 1) // page
        nblocks = B * blocks_per + 1
        cache = torch.randn(nblocks, nkv, 2, page, d, device="cuda", dtype=torch.bfloat16)
        bt = (torch.randperm(nblocks - 1, device="cuda")[: B * blocks_per] + 1).view(B, blocks_per).to(torch.int32)
        cl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
        q = torch.randn(B, nh * d, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(B, nh * d, device="cuda", dtype=torch.bfloat16)
        for nsplit in (1, 4):
            ms = _time(lambda i: native.attn_decode(q, cache, bt, cl, nh, nkv, d, d ** -0.5, nsplit=nsplit, out=out), 1)
            bytes_ = B * ctx * nkv * d * 2 * 2
            results.append({"kernel": "attn_decode_paged", "shape": f"B={B} ctx={ctx} nsplit={nsplit}", "ms": round(ms, 4),
                            "gbs": round(bytes_ / ms / 1e6, 1), "frac_of_measured_hbm": round(bytes_ / ms / 1e6 / peaks["hbm_gbs"], 3)})
            print(results[-1], flush=True)


def bench_attn_prefill(results, peaks):
    from lorax_b200.ops import reference as ref
    nh, nkv, d, page = 32, 8, 128, 32
    for B, L in ((8, 512), (4, 1024), (1, 8192)):
        blocks_per = (L + page - 1) // page
        cache = torch.randn(B * blocks_per + 1, nkv, 2, page, d, device="cuda", dtype=torch.bfloat16)
        bt = (torch.arange(B * blocks_per, device="cuda") + 1).view(B, blocks_per).to(torch.int32)
        q = torch.randn(B * L, nh * d, device="cuda", dtype=torch.bfloat16)
        cu = torch.arange(0, (B + 1) * L, L, device="cuda", dtype=torch.int32)
        cl = torch.zeros(B, device="cuda", dtype=torch.int32)
        ts, tq = ref.prefill_tiles([L] * B)
        ts = torch.tensor(ts, device="cuda", dtype=torch.int32)
        tq = torch.tensor(tq, device="cuda", dtype=torch.int32)
        out = torch.empty_like(q)
        ms = _time(lambda i: native.attn_prefill(q, cache, bt, cu, cl, ts, tq, nh, nkv, d, d ** -0.5, out=out), 1)
        flops = 4.0 * B * L * L * nh * d / 2
        results.append({"kernel": "attn_prefill", "shape": f"B={B} L={L}", "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1)})
        print(results[-1], flush=True)


def bench_small(results, peaks):
    for T in (256, 4096):
        H = 4096
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(H, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(x)
        ms = _time(lambda i: native.norm_residual(x, r, w, 1e-5, out=out), 1)
        results.append({"kernel": "norm_residual", "shape": f"T={T} H={H}", "ms": round(ms, 4), "gbs": round(4 * T * H * 2 / ms / 1e6, 1)})
        print(results[-1], flush=True)
        gu = torch.randn(T, 2 * 14336, device="cuda", dtype=torch.bfloat16)
        o2 = torch.empty(T, 14336, device="cuda", dtype=torch.bfloat16)
        ms = _time(lambda i: native.act_mul(gu, 14336, out=o2), 1)
        results.append({"kernel": "act_mul", "shape": f"T={T} I=14336", "ms": round(ms, 4), "gbs": round(3 * T * 14336 * 2 / ms / 1e6, 1)})
        print(results[-1], flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", default=None)
    a = ap.parse_args()
    peaks = {"hbm_gbs": 6538.9, "bf16_tflops": 1640.9}
    try:
        with open("MEASURED_PEAKS.json") as f:
            peaks.update(json.load(f))
    except OSError:
        pass
    results = []
    for name, fn in (("gemm", bench_gemm), ("attn_decode", bench_attn_decode), ("attn_prefill", bench_attn_prefill), ("small", bench_small)):
        if a.only and a.only != name:
            continue
        fn(results, peaks)
    if a.json:
        with open(a.json, "w") as f:
            json.dump(results, f, indent=1)


if __name__ == "__main__":
    main()
