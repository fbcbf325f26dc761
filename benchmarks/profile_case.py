"""Small, self-terminating workloads for `ncu` captures of single kernels.

    python benchmarks/profile_case.py --case gemm_decode|gemm_mid|gemm_prefill|gemm_fp8_decode|gemm_fp8_prefill|gemm_lora_decode|gemm_lora_decode_gateup|gemm_lora_prefill|gemm_lora_prefill_gateup|attn_decode|attn_prefill|lora_shrink|lora_expand|moe_decode|moe_prefill

Each case launches the kernel a handful of times on inputs larger than the 126 MB L2 but at most a few GB, and
exits 0; run it plain first, then under
`ncu --set full --clock-control none -k regex:<kernel> -c 2 -o <report> python benchmarks/profile_case.py --case ...`.
"""

from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import argparse

import torch

from lorax_b200.ops import native, reference


def gemm_case(T):
    N, K = 28672, 4096
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    for i in range(4):
        native.gemm(x, ws[i % 2], out=out)


def attn_decode_case():
    nh, nkv, d, page, B, ctx = 32, 8, 128, 32, 128, 2048
    bp = ctx // page
    cache = torch.randn(B * bp + 1, nkv, 2, page, d, device="cuda", dtype=torch.bfloat16)
    bt = (torch.randperm(B * bp, device="cuda") + 1).view(B, bp).to(torch.int32)
    cl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    q = torch.randn(B, nh * d, device="cuda", dtype=torch.bfloat16)
    for _ in range(4):
        native.attn_decode(q, cache, bt, cl, nh, nkv, d, d ** -0.5)


def attn_prefill_case():
    nh, nkv, d, page, B, L = 32, 8, 128, 32, 4, 2048
    bp = L // page
    cache = torch.randn(B * bp + 1, nkv, 2, page, d, device="cuda", dtype=torch.bfloat16)
    bt = (torch.arange(B * bp, device="cuda") + 1).view(B, bp).to(torch.int32)
    q = torch.randn(B * L, nh * d, device="cuda", dtype=torch.bfloat16)
    cu = torch.arange(0, (B + 1) * L, L, device="cuda", dtype=torch.int32)
    cl = torch.zeros(B, device="cuda", dtype=torch.int32)
    ts, tq = reference.prefill_tiles([L] * B)
    ts = torch.tensor(ts, device="cuda", dtype=torch.int32)
    tq = torch.tensor(tq, device="cuda", dtype=torch.int32)
    for _ in range(3):
        native.attn_prefill(q, cache, bt, cu, cl, ts, tq, nh, nkv, d, d ** -0.5)


def lora_case(which):
    """100 rank-16 adapters, one layer's QKV group (A_cat [48, 4096], B_cat [6144, 16]), 256 decode rows."""
    K, parts, r, S, T = 4096, [4096, 1024, 1024], 16, 100, 256
    N = sum(parts)
    units = 3 * K + N
    arena = (torch.randn(S * r * units, device="cuda") * 0.02).to(torch.bfloat16)
    slot_base = (torch.arange(S, device="cuda", dtype=torch.int64) * r * units)
    slot_rank = torch.full((S,), r, device="cuda", dtype=torch.int32)
    G = 5
    tm = torch.zeros(S * G * 128, dtype=torch.uint8).pin_memory()
    for s in range(S):
        native.lora_encode_tmap(tm[(s * G) * 128:], arena.data_ptr() + s * r * units * 2, K, 3 * r, r * units, 1)
    tmaps = tm.cuda()
    rows = sorted(int(x) for x in torch.randint(0, S, (T,)))
    tl = reference.build_lora_tiles(rows, 32)
    tiles = torch.full((T, 4), -1, device="cuda", dtype=torch.int32)
    tiles[: len(tl)] = torch.tensor(tl, device="cuda", dtype=torch.int32)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    y = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
    for _ in range(4):
        v = native.lora_shrink_tiles(x, tiles, T, 32, tmaps, G, 0, slot_rank, 3, 0, r)
        if which == "expand":
            native.lora_expand_tiles(v[:T], tiles, T, 32, arena, slot_base, slot_rank, 3 * K, y, parts[0], parts[0] + parts[1])


def gemm_lora_case(T, parts=(4096, 1024, 1024)):
    """QKV (or gate_up) projection with the multi-adapter LoRA in the same launch: 100 rank-16 adapters drawn like the
    benchmark does (Zipf 1.1), rows sorted by adapter, weights rotating over more than L2."""
    import math
    K, r, S = 4096, 16, 100
    N = sum(parts)
    nparts = len(parts)
    units = nparts * K + N
    arena = (torch.randn(S * r * units, device="cuda") * 0.02).to(torch.bfloat16)
    slot_base = torch.arange(S, device="cuda", dtype=torch.int64) * r * units
    slot_rank = torch.full((S,), r, device="cuda", dtype=torch.int32)
    G = 5
    tm = torch.zeros(S * 2 * G * 128, dtype=torch.uint8).pin_memory()
    for s_ in range(S):
        base = arena.data_ptr() + s_ * r * units * 2
        native.lora_encode_tmap(tm[(s_ * 2 * G) * 128:], base, K, nparts * r, r * units, 1)
        native.lora_encode_tmap_b(tm[(s_ * 2 * G + G) * 128:], base + r * nparts * K * 2, r, N, r * units, 1)
    tmaps = tm.cuda()
    w_ = torch.tensor([1.0 / (k ** 1.1) for k in range(1, S + 1)], dtype=torch.float64)
    rows = sorted(int(x) for x in torch.multinomial(w_ / w_.sum(), T, replacement=True))
    tl = reference.build_lora_tiles(rows, 32)
    tiles = torch.full((min(max(T, len(tl)), len(tl) + 16), 4), -1, device="cuda", dtype=torch.int32)
    tiles[: len(tl)] = torch.tensor(tl, device="cuda", dtype=torch.int32)
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / math.sqrt(K) for _ in range(4)]
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    n0 = parts[0] if nparts > 1 else N
    n1 = parts[0] + parts[1] if nparts > 2 else N
    lf = native.LoraFused(tiles, tiles.shape[0], len(tl), tmaps, 2 * G, 0, G, slot_rank, slot_base, nparts, n0, n1, 0, r, arena, 0, nparts * K)
    for i in range(4):
        assert native.gemm_lora_fused(x, ws[i], lf, out=out) is not None


def gemm_fp8_case(T):
    """Block-scaled fp8 GEMM, gate_up shape, weights rotating over > L2."""
    N, K = 28672, 4096
    ws = []
    for _ in range(3):
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / 64
        ws.append(reference.quantize_weight_fp8_block128(w))
        del w
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    for i in range(4):
        native.gemm_fp8(x, ws[i % 3][0].view(torch.uint8), ws[i % 3][1], out=out)


def gemm_int4_case(T):
    """Weight-only 4-bit GEMM straight from the packed codes, gate_up shape, three weight sets (> L2 in total)."""
    from lorax_b200.utils import quant_formats as qf
    N, K = 28672, 4096
    base = qf.quantize_rtn(torch.randn(N, K) * 0.02, 4, 128).to("cuda")
    ws = [qf.GroupQuantWeight(base.codes.clone(), base.sz.clone(), 4, 128, (N, K)) for _ in range(3)]
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    for i in range(4):
        native.gemm_wq(x, ws[i % 3], out=out)


def moe_case(T):
    """Mixtral-8x7B expert shapes (8 experts, top 2, hidden 4096, intermediate 14336) on one GPU: routing, gather, grouped w1|w3
    GEMM, act * up, grouped w2 GEMM, combine.  2.8 GB of expert weights: every launch streams them from HBM."""
    import math
    E, k, H, I = 8, 2, 4096, 14336
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    wr = (torch.randn(E, H, device="cuda") * 0.3).to(torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, device="cuda", dtype=torch.bfloat16) / math.sqrt(H))
    w2 = (torch.randn(E, H, I, device="cuda", dtype=torch.bfloat16) / math.sqrt(I))
    for _ in range(3):
        native.moe_ffn(x, wr, w13, w2, k, 0, "silu")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    a = ap.parse_args()
    native.load()
    {"gemm_decode": lambda: gemm_case(64), "gemm_prefill": lambda: gemm_case(4096), "attn_decode": attn_decode_case,
     "attn_prefill": attn_prefill_case, "gemm_lora_decode": lambda: gemm_lora_case(256), "gemm_lora_decode_gateup": lambda: gemm_lora_case(256, (14336, 14336)), "gemm_lora_prefill": lambda: gemm_lora_case(576),
     "gemm_lora_prefill_gateup": lambda: gemm_lora_case(4096, (14336, 14336)),
     "gemm_fp8_decode": lambda: gemm_fp8_case(64), "gemm_fp8_prefill": lambda: gemm_fp8_case(2048), "gemm_mid": lambda: gemm_case(256),
     "gemm_int4_decode": lambda: gemm_int4_case(8),
     "lora_shrink": lambda: lora_case("shrink"), "lora_expand": lambda: lora_case("expand"),
     "moe_decode": lambda: moe_case(256), "moe_prefill": lambda: moe_case(2048)}[a.case]()
    torch.cuda.synchronize()
    native.workspace().check_status()
    print("ok", a.case)


if __name__ == "__main__":
    main()
