"""Micro-benchmarks of the CUDA kernels against their roofline (and cuBLAS for the GEMM).

``python benchmarks/bench_kernels.py [--json out.json]`` times each kernel with CUDA events after a
warm-up, rotating through enough distinct buffers that the working set exceeds the 126 MB L2.
"""

from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

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


def bench_lora(results, peaks):
    """One projection with 100 rank-16 adapters over the rows (Zipf 1.1, rows grouped by adapter): the GEMM that carries LoRA in
    its own launch against shrink + GEMM + expand as three launches, and against the base GEMM alone."""
    from lorax_b200.ops import reference
    r, S, G = 16, 100, 5
    sites = [("qkv", [4096, 1024, 1024], 4096), ("o", [4096], 4096), ("gate_up", [14336, 14336], 4096), ("down", [4096], 14336)]
    wz = torch.tensor([1.0 / (k ** 1.1) for k in range(1, S + 1)], dtype=torch.float64)
    for T in (64, 256, 1024, 4096):
        rows = sorted(int(v) for v in torch.multinomial(wz / wz.sum(), T, replacement=True, generator=torch.Generator().manual_seed(T)))
        tl = reference.build_lora_tiles(rows, 32)
        tiles = torch.full((len(tl) + 16, 4), -1, device="cuda", dtype=torch.int32)
        tiles[: len(tl)] = torch.tensor(tl, device="cuda", dtype=torch.int32)
        for name, parts, K in sites:
            N, nparts = sum(parts), len(parts)
            units = nparts * K + N
            arena = (torch.randn(S * r * units, device="cuda") * 0.02).to(torch.bfloat16)
            slot_base = torch.arange(S, device="cuda", dtype=torch.int64) * r * units
            slot_rank = torch.full((S,), r, device="cuda", dtype=torch.int32)
            tm = torch.zeros(S * 2 * G * 128, dtype=torch.uint8).pin_memory()
            for s_ in range(S):
                base = arena.data_ptr() + s_ * r * units * 2
                native.lora_encode_tmap(tm[(s_ * 2 * G) * 128:], base, K, nparts * r, r * units, 1)
                native.lora_encode_tmap_b(tm[(s_ * 2 * G + G) * 128:], base + r * nparts * K * 2, r, N, r * units, 1)
            tmaps = tm.cuda()
            n_rot = max(2, int(math.ceil(300e6 / (N * K * 2))))
            ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / math.sqrt(K) for _ in range(n_rot)]
            x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
            out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
            n0 = parts[0] if nparts > 1 else N
            n1 = parts[0] + parts[1] if nparts > 2 else N
            lf = native.LoraFused(tiles, tiles.shape[0], len(tl), tmaps, 2 * G, 0, G, slot_rank, slot_base, nparts, n0, n1, 0, r, arena, 0, nparts * K)

            def separate(i):
                v = native.lora_shrink_tiles(x, tiles, tiles.shape[0], 32, tmaps, 2 * G, 0, slot_rank, nparts, 0, r, live_tiles=len(tl))
                native.gemm(x, ws[i], out=out)
                native.lora_expand_tiles(v[:T], tiles, tiles.shape[0], 32, arena, slot_base, slot_rank, nparts * K, out, n0, n1)
            ms_f = _time(lambda i: native.gemm_lora_fused(x, ws[i], lf, out=out), n_rot)
            ms_s = _time(separate, n_rot)
            ms_b = _time(lambda i: native.gemm(x, ws[i], out=out), n_rot)
            native.workspace().check_status()
            results.append({"kernel": "gemm_bf16_tcgen05<lora>", "shape": f"{name} T={T} N={N} K={K} entries={len(tl)}",
                            "ms_one_launch": round(ms_f, 4), "ms_three_launches": round(ms_s, 4), "ms_base_gemm": round(ms_b, 4)})
            print(results[-1], flush=True)
            del ws, arena


def bench_moe(results, peaks):
    """Mixtral-8x7B expert block (8 experts, top 2) on one GPU: the device path (grouped tcgen05 GEMMs) against the bytes it must
    stream (every expert's weights once when each expert has at least one row) and the FLOPs of the routed rows."""
    E, k, H, I = 8, 2, 4096, 14336
    wr = (torch.randn(E, H, device="cuda") * 0.3).to(torch.bfloat16)
    w13 = torch.randn(E, 2 * I, H, device="cuda", dtype=torch.bfloat16) / math.sqrt(H)
    w2 = torch.randn(E, H, I, device="cuda", dtype=torch.bfloat16) / math.sqrt(I)
    for T in (16, 256, 2048, 4096):
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        ms = _time(lambda i: native.moe_ffn(x, wr, w13, w2, k, 0, "silu"), 1, iters=10)
        native.workspace().check_status()
        wbytes = (w13.numel() + w2.numel()) * 2
        flops = 2.0 * T * k * 3 * H * I
        results.append({"kernel": "moe_ffn (route, gather, 2 grouped GEMMs, act, combine)", "shape": f"T={T} E={E} top{k} H={H} I={I}",
                        "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "weight_gbs": round(wbytes / ms / 1e6, 1),
                        "frac_of_measured_hbm": round(wbytes / ms / 1e6 / peaks["hbm_gbs"], 3),
                        "frac_of_measured_bf16": round(flops / ms / 1e9 / peaks["bf16_tflops"], 3)})
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
    for name, fn in (("gemm", bench_gemm), ("lora", bench_lora), ("moe", bench_moe), ("attn_decode", bench_attn_decode), ("attn_prefill", bench_attn_prefill),
                     ("small", bench_small)):
        if a.only and a.only != name:
            continue
        fn(results, peaks)
    if a.json:
        with open(a.json, "w") as f:
            json.dump(results, f, indent=1)


if __name__ == "__main__":
    main()
