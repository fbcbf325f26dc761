"""Numerics of every CUDA kernel against the fp32 PyTorch statement of the same operator."""
import math

import pytest
import torch

from lorax_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
    from lorax_b200.ops import native
    native.load()
    return native


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-6)).item()


@pytest.mark.parametrize("T,N,K", [(1, 512, 256), (7, 384, 512), (16, 4096, 4096), (33, 1024, 14336), (100, 6144, 4096),
                                   (128, 4096, 4096), (200, 1000, 520), (256, 2048, 1024)])
def test_gemm_small_t(nat, T, N, K):
    torch.manual_seed(T * 7 + N)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / math.sqrt(K)
    out = nat.gemm(x, w)
    torch.cuda.synchronize()
    nat.workspace().check_status()
    want = x.float() @ w.float().t()
    assert _rel_err(out, want) < 6e-3
    # deterministic (split-K reduces in a fixed order)
    out2 = nat.gemm(x, w)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("T,N,K", [(257, 512, 512), (1000, 4096, 4096), (4096, 6144, 4096), (300, 1000, 520)])
def test_gemm_large_t(nat, T, N, K):
    torch.manual_seed(T + N)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / math.sqrt(K)
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    out = nat.gemm(x, w, bias=b)
    torch.cuda.synchronize()
    nat.workspace().check_status()
    want = x.float() @ w.float().t() + b.float()
    assert _rel_err(out, want) < 6e-3


@pytest.mark.parametrize("mode", [1, 2])
def test_gemm_modes_bias_split(nat, mode):
    torch.manual_seed(3)
    T, N, K = 48, 640, 2048
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / math.sqrt(K)
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    want = x.float() @ w.float().t() + b.float()
    for split in ([1, 2, 4] if mode == 1 else [0]):
        out = nat.gemm(x, w, bias=b, mode=mode, force_split=split)
        torch.cuda.synchronize()
        nat.workspace().check_status()
        assert _rel_err(out, want) < 6e-3, (mode, split)


@pytest.mark.parametrize("T,N,K,bn", [(16, 4096, 4096, 0), (64, 28672, 4096, 0), (256, 6144, 4096, 64), (256, 4096, 14336, 256),
                                      (200, 1000, 520, 0), (576, 4096, 4096, 0), (700, 28672, 1024, 0), (1000, 4096, 14336, 0)])
def test_gemm_stream_k(nat, T, N, K, bn):
    """The partly filled last wave is cut along K across all SMs (policy 2 forces it); policy 1 computes whole tiles."""
    torch.manual_seed(T + N + K)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / math.sqrt(K)
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    want = x.float() @ w.float().t() + b.float()
    base = 1 if T <= 256 else 2
    outs = []
    for policy in (1, 2, 2):
        out = nat.gemm(x, w, bias=b, mode=base | (policy << 8), force_split=bn << 16)
        torch.cuda.synchronize()
        nat.workspace().check_status()
        assert _rel_err(out, want) < 6e-3, policy
        outs.append(out)
    assert torch.equal(outs[1], outs[2])          # fixed reduction order
    assert _rel_err(outs[1], outs[0]) < 2e-3


def test_gemm_strided_views(nat):
    torch.manual_seed(4)
    big = torch.randn(40, 3 * 1024, device="cuda", dtype=torch.bfloat16)
    x = big[:, 1024:2048]
    w = torch.randn(256, 1024, device="cuda", dtype=torch.bfloat16) / 32
    outbuf = torch.zeros(40, 512, device="cuda", dtype=torch.bfloat16)
    nat.gemm(x, w, out=outbuf[:, 256:])
    torch.cuda.synchronize()
    assert _rel_err(outbuf[:, 256:], x.float() @ w.float().t()) < 6e-3
    assert outbuf[:, :256].abs().max().item() == 0


@pytest.mark.parametrize("T,H,layernorm", [(5, 4096, False), (64, 8192, False), (3, 256, False), (9, 1024, True)])
def test_norm_residual(nat, T, H, layernorm):
    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(H, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(H, device="cuda", dtype=torch.bfloat16) if layernorm else None
    r_ref = r.clone()
    want = ref.norm_residual(x, r_ref, w, 1e-5, bias=b, layernorm=layernorm, weight_offset=1.0 if not layernorm else 0.0)
    got = nat.norm_residual(x, r, w, 1e-5, bias=b, layernorm=layernorm, weight_offset=1.0 if not layernorm else 0.0)
    assert torch.equal(r, r_ref)
    assert _rel_err(got, want) < 5e-3
    got2 = nat.norm_residual(x, None, w, 1e-5, bias=b, layernorm=layernorm)
    want2 = ref.norm_residual(x, None, w, 1e-5, bias=b, layernorm=layernorm)
    assert _rel_err(got2, want2) < 5e-3


@pytest.mark.parametrize("nh,nkv,d,rot", [(32, 8, 128, 128), (4, 2, 64, 64), (8, 8, 64, 32)])
def test_rope_kvwrite(nat, nh, nkv, d, rot):
    torch.manual_seed(1)
    T, page, blocks = 37, 32, 12
    qkv = torch.randn(T, (nh + 2 * nkv) * d, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (T,), device="cuda", dtype=torch.int32)
    cs = ref.rope_cache(rot, 512, 10000.0, device="cuda")
    slots = torch.randperm(blocks * page, device="cuda")[:T].to(torch.int32)
    slots[3] = -1
    cache = torch.zeros(blocks, nkv, 2, page, d, device="cuda", dtype=torch.bfloat16)
    cache_ref = cache.clone()
    qkv_ref = qkv.clone()
    ref.rope_kvwrite(qkv_ref, pos, cs, cache_ref, slots, nh, nkv, d, rot)
    nat.rope_kvwrite(qkv, pos, cs, cache, slots, nh, nkv, d, rot)
    assert _rel_err(qkv, qkv_ref) < 4e-3
    assert _rel_err(cache, cache_ref) < 4e-3


def test_prefill_metadata(nat):
    """Per-token positions, cache slots and adapter slots of a ragged prefill, computed on the device from the per-sequence arrays."""
    q_lens, cache_lens, slots_of = [5, 64, 1, 130, 33], [0, 7, 99, 32, 0], [-1, 3, 3, 0, -1]
    B, page, max_blocks = len(q_lens), 32, 9
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device="cuda", dtype=torch.int32)
    cl = torch.tensor(cache_lens, device="cuda", dtype=torch.int32)
    ss = torch.tensor(slots_of, device="cuda", dtype=torch.int32)
    bt = torch.randint(1, 500, (B, max_blocks), device="cuda", dtype=torch.int32)
    T = sum(q_lens)
    got = nat.prefill_metadata(cu, cl, ss, bt, page, T)
    want = ref.prefill_metadata(cu, cl, ss, bt, page, T)
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    # against the definition
    t = 5 + 64 + 1 + 17                     # token 17 of sequence 3
    assert int(got[0][t]) == 32 + 17 and int(got[1][t]) == int(bt[3, (32 + 17) // page]) * page + (32 + 17) % page and int(got[2][t]) == 0


@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_pytorch_tanh"])
def test_act_mul(nat, act):
    x = torch.randn(19, 2 * 1376, device="cuda", dtype=torch.bfloat16)
    assert _rel_err(nat.act_mul(x, 1376, act), ref.act_mul(x, 1376, act)) < 4e-3
    assert _rel_err(nat.act_mul(x, 1376, act, gated=False), ref.act_mul(x, 1376, act, gated=False)) < 4e-3


def test_embed_argmax_advance(nat):
    table = torch.randn(1000, 256, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 2000, (50,), device="cuda", dtype=torch.int32)
    got = nat.embed(ids, table, v0=500, v1=1500, mult=2.0)
    want = ref.embed(ids, table, v0=500, v1=1500, mult=2.0)
    assert torch.equal(got, want)
    logits = torch.randn(33, 32000, device="cuda", dtype=torch.bfloat16)
    i, lp = nat.argmax_logprob(logits)
    wi, wlp = ref.argmax_logprob(logits)
    assert torch.equal(i.long(), wi.long())
    assert torch.allclose(lp, wlp, atol=2e-3)
    B, page = 9, 32
    bt = torch.randint(1, 100, (B, 8), device="cuda", dtype=torch.int32)
    state = [torch.randint(0, 100, (B,), device="cuda", dtype=torch.int32) for _ in range(2)]
    inp, pos = state
    ctx = pos + 1
    ctx[2] = 0
    slots = torch.zeros(B, device="cuda", dtype=torch.int32)
    nxt = torch.randint(0, 100, (B,), device="cuda", dtype=torch.int32)
    a = [t.clone() for t in (inp, pos, ctx, slots)]
    b = [t.clone() for t in (inp, pos, ctx, slots)]
    nat.advance_decode(a[0], nxt, a[1], a[2], a[3], bt, page)
    ref.advance_decode(b[0], nxt, b[1], b[2], b[3], bt, page)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def _make_cache(B, max_len, nkv, d, page=32, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    max_blocks = (max_len + page - 1) // page
    nblocks = B * max_blocks + 1
    cache = torch.randn(nblocks, nkv, 2, page, d, device="cuda", dtype=torch.bfloat16, generator=g)
    perm = torch.randperm(nblocks - 1, device="cuda", generator=g)[: B * max_blocks] + 1
    bt = perm.view(B, max_blocks).to(torch.int32)
    return cache, bt


@pytest.mark.parametrize("nh,nkv,d,window,softcap,nsplit", [(32, 8, 128, 0, 0.0, 1), (32, 8, 128, 100, 0.0, 1),
                                                             (4, 2, 64, 0, 0.0, 1), (8, 8, 128, 0, 30.0, 1),
                                                             (32, 8, 128, 0, 0.0, 4), (32, 1, 128, 0, 0.0, 2)])
def test_attn_decode(nat, nh, nkv, d, window, softcap, nsplit):
    torch.manual_seed(5)
    B, max_len = 11, 700
    cache, bt = _make_cache(B, max_len, nkv, d)
    ctx = torch.randint(1, max_len, (B,), device="cuda", dtype=torch.int32)
    ctx[0] = 1
    ctx[1] = max_len
    ctx[2] = 0
    q = torch.randn(B, nh * d, device="cuda", dtype=torch.bfloat16)
    scale = d ** -0.5
    got = nat.attn_decode(q, cache, bt, ctx, nh, nkv, d, scale, window, softcap, nsplit)
    want = ref.attn_decode(q, cache, bt, ctx, nh, nkv, d, scale, window, softcap)
    assert _rel_err(got, want) < 1e-2


@pytest.mark.parametrize("nh,nkv,d,window,cached", [(32, 8, 128, 0, False), (4, 2, 64, 0, True), (8, 2, 128, 70, True)])
def test_attn_prefill(nat, nh, nkv, d, window, cached):
    torch.manual_seed(6)
    q_lens = [5, 64, 130, 257, 1]
    B = len(q_lens)
    cache_lens = [0, 3, 64, 100, 31] if cached else [0] * B
    max_len = max(a + b for a, b in zip(q_lens, cache_lens))
    cache, bt = _make_cache(B, max_len, nkv, d, seed=1)
    T = sum(q_lens)
    q = torch.randn(T, nh * d, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device="cuda", dtype=torch.int32)
    cl = torch.tensor(cache_lens, device="cuda", dtype=torch.int32)
    ts, tq = ref.prefill_tiles(q_lens)
    ts = torch.tensor(ts, device="cuda", dtype=torch.int32)
    tq = torch.tensor(tq, device="cuda", dtype=torch.int32)
    scale = d ** -0.5
    got = nat.attn_prefill(q, cache, bt, cu, cl, ts, tq, nh, nkv, d, scale, window)
    want = ref.attn_prefill(q, cache, bt, cu, cl, ts, tq, nh, nkv, d, scale, window)
    assert _rel_err(got, want) < 1e-2


@pytest.mark.parametrize("nh,nkv,d,rot", [(32, 8, 128, 128), (4, 2, 64, 32)])
def test_fp8_kv_cache(nat, nh, nkv, d, rot):
    """e4m3 KV pages with a K and a V scale: `rope_kvwrite` stores value / scale (saturating), decode and prefill attention read
    stored value * scale.  The bytes written match the fp32 reference bit for bit (up to the rounding of the rotated bf16 value),
    and attention over the same fp8 cache matches fp32 attention over its dequantised values; against the bf16 cache the error is
    the quantisation's."""
    torch.manual_seed(21)
    page, ks, vs = 32, 0.05, 0.02
    # ---- writes
    T, blocks = 41, 12
    qkv = torch.randn(T, (nh + 2 * nkv) * d, device="cuda", dtype=torch.bfloat16) * 3
    pos = torch.randint(0, 500, (T,), device="cuda", dtype=torch.int32)
    cs = ref.rope_cache(rot, 512, 10000.0, device="cuda")
    slots = torch.randperm(blocks * page, device="cuda")[:T].to(torch.int32)
    slots[5] = -1
    cache = torch.zeros(blocks, nkv, 2, page, d, device="cuda", dtype=torch.float8_e4m3fn)
    cache_ref = torch.zeros_like(cache)
    qkv_ref = qkv.clone()
    ref.rope_kvwrite(qkv_ref, pos, cs, cache_ref, slots, nh, nkv, d, rot, kv_scale=(ks, vs))
    nat.rope_kvwrite(qkv, pos, cs, cache, slots, nh, nkv, d, rot, kv_scale=(ks, vs))
    a, b = cache.float(), cache_ref.float()
    assert (a != b).float().mean() < 0.02                  # a rotated value that rounds differently in bf16 may land one e4m3 step away
    assert _rel_err(a, b) < 2e-2
    assert a.abs().max() <= 448 and torch.isfinite(a).all()        # 3 * N(0,1) / 0.02 saturates instead of overflowing
    # ---- reads
    B, max_len = 9, 600
    wide, bt = _make_cache(B, max_len, nkv, d, seed=3)
    kq = torch.empty_like(wide, dtype=torch.float8_e4m3fn)
    kq.view(torch.uint8)[:, :, 0] = ref._to_e4m3_bytes(wide[:, :, 0], ks)
    kq.view(torch.uint8)[:, :, 1] = ref._to_e4m3_bytes(wide[:, :, 1], vs)
    ctx = torch.randint(1, max_len, (B,), device="cuda", dtype=torch.int32)
    ctx[0], ctx[1] = 1, max_len
    q = torch.randn(B, nh * d, device="cuda", dtype=torch.bfloat16)
    scale = d ** -0.5
    for nsplit in (1, 4):
        got = nat.attn_decode(q, kq, bt, ctx, nh, nkv, d, scale, 0, 0.0, nsplit, kv_scale=(ks, vs))
        want = ref.attn_decode(q, kq, bt, ctx, nh, nkv, d, scale, 0, 0.0, kv_scale=(ks, vs))
        assert _rel_err(got, want) < 1e-2, nsplit
    assert _rel_err(got, ref.attn_decode(q, wide, bt, ctx, nh, nkv, d, scale)) < 8e-2        # quantisation error only
    q_lens, cache_lens = [70, 200, 33], [0, 150, 64]
    Tq = sum(q_lens)
    qp = torch.randn(Tq, nh * d, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device="cuda", dtype=torch.int32)
    cl = torch.tensor(cache_lens, device="cuda", dtype=torch.int32)
    ts, tq = ref.prefill_tiles(q_lens)
    ts, tq = torch.tensor(ts, device="cuda", dtype=torch.int32), torch.tensor(tq, device="cuda", dtype=torch.int32)
    got = nat.attn_prefill(qp, kq, bt[:3], cu, cl, ts, tq, nh, nkv, d, scale, 0, kv_scale=(ks, vs))
    want = ref.attn_prefill(qp, kq, bt[:3], cu, cl, ts, tq, nh, nkv, d, scale, 0, kv_scale=(ks, vs))
    assert _rel_err(got, want) < 1e-2
    nat.workspace().check_status()


@pytest.mark.parametrize("nh,nkv,window,softcap,q_lens,cache_lens", [
    (32, 8, 0, 0.0, [700, 1300, 3], [0, 0, 0]),                # several key blocks per tile: both TMEM buffers and both K/V stages cycle
    (8, 2, 0, 0.0, [200, 64, 129], [900, 37, 128]),            # chunks that continue a cached prefix (chunked prefill, prefix cache)
    (16, 4, 300, 0.0, [1000, 50], [0, 2000]),                  # sliding window: key blocks left of the window are skipped
    (8, 4, 0, 30.0, [333], [5])])                              # soft-capped scores
def test_attn_prefill_tensor_core(nat, nh, nkv, window, softcap, q_lens, cache_lens):
    """tcgen05 flash prefill (two heads of a KV group per CTA, K / V pages by TMA from the paged cache) against fp32 attention."""
    torch.manual_seed(16)
    d = 128
    assert nat.load().lx_attn_prefill_tc_supported(nh, nkv, d, nh * d, nh * d) == 1
    B = len(q_lens)
    max_len = max(a + b for a, b in zip(q_lens, cache_lens))
    cache, bt = _make_cache(B, max_len, nkv, d, seed=4)
    T = sum(q_lens)
    q = torch.randn(T, nh * d, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device="cuda", dtype=torch.int32)
    cl = torch.tensor(cache_lens, device="cuda", dtype=torch.int32)
    ts, tq = ref.prefill_tiles(q_lens)
    ts = torch.tensor(ts, device="cuda", dtype=torch.int32)
    tq = torch.tensor(tq, device="cuda", dtype=torch.int32)
    scale = d ** -0.5
    for _ in range(2):
        got = nat.attn_prefill(q, cache, bt, cu, cl, ts, tq, nh, nkv, d, scale, window, softcap)
        torch.cuda.synchronize()
        nat.workspace().check_status()
        want = ref.attn_prefill(q, cache, bt, cu, cl, ts, tq, nh, nkv, d, scale, window, softcap)
        assert _rel_err(got, want) < 1e-2
        assert torch.isfinite(got.float()).all()


@pytest.mark.parametrize("nh,nkv,d,nsplit", [(12, 12, 64, 1), (32, 8, 128, 3), (6, 6, 128, 1)])
def test_attn_alibi(nat, nh, nkv, d, nsplit):
    """ALiBi slopes in both attention kernels (BLOOM, MPT): bias -slope_h * (query position - key position)."""
    from lorax_b200.models.decoder import alibi_slopes
    torch.manual_seed(15)
    slopes = alibi_slopes(nh).cuda()
    scale = d ** -0.5
    B, max_len = 7, 500
    cache, bt = _make_cache(B, max_len, nkv, d, seed=2)
    ctx = torch.randint(1, max_len, (B,), device="cuda", dtype=torch.int32)
    ctx[0], ctx[1] = 1, max_len
    q = torch.randn(B, nh * d, device="cuda", dtype=torch.bfloat16)
    got = nat.attn_decode(q, cache, bt, ctx, nh, nkv, d, scale, 0, 0.0, nsplit, alibi=slopes)
    want = ref.attn_decode(q, cache, bt, ctx, nh, nkv, d, scale, alibi=slopes)
    plain = ref.attn_decode(q, cache, bt, ctx, nh, nkv, d, scale)
    assert _rel_err(got, want) < 1e-2 and _rel_err(plain, want) > 0.1
    q_lens, cache_lens = [9, 150, 64], [0, 70, 33]
    cache, bt = _make_cache(3, 256, nkv, d, seed=3)
    T = sum(q_lens)
    q = torch.randn(T, nh * d, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device="cuda", dtype=torch.int32)
    cl = torch.tensor(cache_lens, device="cuda", dtype=torch.int32)
    ts, tq = ref.prefill_tiles(q_lens)
    ts = torch.tensor(ts, device="cuda", dtype=torch.int32)
    tq = torch.tensor(tq, device="cuda", dtype=torch.int32)
    got = nat.attn_prefill(q, cache, bt, cu, cl, ts, tq, nh, nkv, d, scale, alibi=slopes)
    want = ref.attn_prefill(q, cache, bt, cu, cl, ts, tq, nh, nkv, d, scale, alibi=slopes)
    assert _rel_err(got, want) < 1e-2


@pytest.mark.parametrize("T", [3, 100, 700])
def test_lora_shrink_expand(nat, T):
    torch.manual_seed(8)
    K, parts = 1024, [512, 128, 128]
    N = sum(parts)
    ranks = [8, 16, 64, 32]
    unit_a, unit_b = 0, 3 * K        # per-unit-rank offsets of A_cat and B_cat inside a blob
    unit_total = 3 * K + N
    bases, off = [], 0
    for r in ranks:
        bases.append(off)
        off += r * unit_total
    arena = (torch.randn(off, device="cuda") * 0.05).to(torch.bfloat16)
    slot_base = torch.tensor(bases + [-1], device="cuda", dtype=torch.int64)
    slot_rank = torch.tensor(ranks + [0], device="cuda", dtype=torch.int32)
    # runs of equal slots plus base-model tokens
    tok_slot = torch.randint(-1, len(ranks), (T,), device="cuda", dtype=torch.int32)
    if T > 64:
        tok_slot = tok_slot[torch.arange(T, device="cuda") // 37 % tok_slot.numel()].contiguous()
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    v = torch.zeros(T, 3 * 64, device="cuda", dtype=torch.float32)
    v_ref = v.clone()
    nat.lora_shrink(x, tok_slot, arena, slot_base, slot_rank, unit_a, 3, 64, v)
    ref.lora_shrink(x, tok_slot, arena, slot_base, slot_rank, unit_a, 3, 64, v_ref)
    torch.cuda.synchronize()
    assert _rel_err(v, v_ref) < 2e-3
    y = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
    y_ref = y.clone()
    nat.lora_expand(v_ref, tok_slot, arena, slot_base, slot_rank, unit_b, y, parts[0], parts[0] + parts[1])
    ref.lora_expand(v_ref, tok_slot, arena, slot_base, slot_rank, unit_b, y_ref, parts[0], parts[0] + parts[1])
    nat.workspace().check_status()
    assert _rel_err(y, y_ref) < 5e-3


@pytest.mark.parametrize("T,max_rows", [(40, 32), (300, 32), (700, 128)])
def test_lora_tiled_tensor_core(nat, T, max_rows):
    """Tile-table LoRA: tcgen05 shrink through per-slot tensor maps + tiled expand, against the PyTorch loop."""
    torch.manual_seed(9)
    K, parts, L = 1024, [512, 128, 128], 3
    N = sum(parts)
    ranks = [8, 16, 64, 32]
    layer_units = 3 * K + N                    # A_cat (3 parts) then B_cat, per unit rank
    bases, off = [], 0
    for r in ranks:
        bases.append(off)
        off += r * layer_units * L
        off = (off + 63) // 64 * 64
    arena = (torch.randn(off, device="cuda") * 0.05).to(torch.bfloat16)
    slot_base = torch.tensor(bases, device="cuda", dtype=torch.int64)
    slot_rank = torch.tensor(ranks, device="cuda", dtype=torch.int32)
    G = 5
    tm_host = torch.zeros(len(ranks) * G * 128, dtype=torch.uint8).pin_memory()
    for s, r in enumerate(ranks):
        nat.lora_encode_tmap(tm_host[(s * G + 0) * 128:], arena.data_ptr() + bases[s] * 2, K, 3 * r, r * layer_units, L)
    tmaps = tm_host.cuda()
    # rows grouped by slot, with base-model rows in between
    seg = [(-1, 3), (0, 5), (2, T // 3), (1, 1), (3, T // 4)]
    rows = []
    for sl, n in seg:
        rows += [sl] * n
    rows = (rows + [1] * T)[:T]
    tl = ref.build_lora_tiles(rows, max_rows)
    tiles = torch.tensor(tl, device="cuda", dtype=torch.int32).view(-1, 4)
    pad = torch.full((7, 4), -1, device="cuda", dtype=torch.int32)
    tiles_padded = torch.cat([tiles, pad])
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    layer = 2
    offA = layer * layer_units
    offB = layer * layer_units + 3 * K
    nat.workspace().lora_v.zero_()      # columns past a slot's rank are never written; other tests leave values there
    vf = nat.lora_shrink_tiles(x, tiles_padded, tiles_padded.shape[0], max_rows, tmaps, G, 0, slot_rank, 3, layer, 64)
    torch.cuda.synchronize()
    nat.workspace().check_status()
    v = vf[:T].clone()
    v_ref = torch.zeros_like(v)
    ref.lora_shrink_tiles(x, tiles.cpu(), len(tl), max_rows, arena, slot_base, slot_rank, offA, 3, 64, v_ref)
    live = torch.tensor([s >= 0 for s in rows], device="cuda")
    assert _rel_err(v[live], v_ref[live]) < 4e-3
    y = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
    y_ref = y.clone()
    nat.lora_expand_tiles(vf[:T], tiles_padded, tiles_padded.shape[0], max_rows, arena, slot_base, slot_rank, offB, y, parts[0], parts[0] + parts[1])
    ref.lora_expand_tiles(v_ref, tiles.cpu(), len(tl), max_rows, arena, slot_base, slot_rank, offB, y_ref, parts[0], parts[0] + parts[1])
    nat.workspace().check_status()
    assert _rel_err(y, y_ref) < 5e-3
    # rows without a tile are untouched
    untouched = [i for i, s in enumerate(rows) if s < 0]
    assert torch.equal(y[untouched], y_ref[untouched])


@pytest.mark.parametrize("T,K,parts,ranks,layout", [(40, 1024, [512, 128, 128], [16, 48, 64, 32], "blocks"),
                                                    (256, 4096, [1024, 256, 256], [16, 16, 32, 64], "blocks"),
                                                    (700, 2048, [768, 768], [16, 32, 16, 64], "blocks"),
                                                    (300, 14336, [512], [16, 64, 32, 16], "blocks"),
                                                    # a prefill-sized step: every CTA walks several token tiles and rebuilds its unit list
                                                    (2304, 2048, [1536, 768], [16, 32, 16, 64], "runs"),
                                                    # another adapter on every row: more expand units per token tile than the list holds
                                                    (200, 1024, [512, 256], [16, 64, 32, 64], "alternating"),
                                                    # the same in a long step: one-row entries in the shrink units of four row groups
                                                    (600, 1024, [512, 256], [16, 64, 32, 64], "alternating")])
def test_gemm_with_lora_in_the_same_launch(nat, T, K, parts, ranks, layout):
    """Shrink items, base tiles and expand UMMAs in ONE launch of the GEMM kernel against fp32 PyTorch:
    x W^T + b + (x A_slot^T) B_slot^T per row, several adapters and ranks, base-model rows in between, rows of one adapter
    crossing 16-row and 256-row boundaries, rank 48 (a part that straddles two 128-row chunks of A_cat), two calls in a row."""
    torch.manual_seed(T + K)
    nparts, L = len(parts), 2
    N = sum(parts)
    layer_units = nparts * K + N
    bases, off = [], 0
    for r in ranks:
        bases.append(off)
        off += r * layer_units * L
        off = (off + 63) // 64 * 64
    arena = (torch.randn(off, device="cuda") * 0.05).to(torch.bfloat16)
    slot_base = torch.tensor(bases, device="cuda", dtype=torch.int64)
    slot_rank = torch.tensor(ranks, device="cuda", dtype=torch.int32)
    G = 5
    tm_host = torch.zeros(len(ranks) * 2 * G * 128, dtype=torch.uint8).pin_memory()
    for s, r in enumerate(ranks):
        nat.lora_encode_tmap(tm_host[(s * 2 * G + 0) * 128:], arena.data_ptr() + bases[s] * 2, K, nparts * r, r * layer_units, L)
        nat.lora_encode_tmap_b(tm_host[(s * 2 * G + G) * 128:], arena.data_ptr() + (bases[s] + r * nparts * K) * 2, r, N, r * layer_units, L)
    tmaps = tm_host.cuda()
    if layout == "blocks":
        seg = [(-1, 3), (0, 5), (2, T // 3), (1, 1), (3, T // 4), (-1, 2)]
        rows = []
        for sl, n in seg:
            rows += [sl] * n
        rows = (rows + [1] * T)[:T]
    elif layout == "runs":          # runs of 1 to 90 rows, adapters and base-model rows in turn
        g = torch.Generator().manual_seed(T)
        rows = []
        while len(rows) < T:
            rows += [int(torch.randint(-1, len(ranks), (1,), generator=g))] * int(torch.randint(1, 91, (1,), generator=g))
        rows = rows[:T]
    else:
        rows = [(i % (len(ranks) + 1)) - 1 for i in range(T)]
    tl = ref.build_lora_tiles(rows, 32)
    tiles = torch.cat([torch.tensor(tl, device="cuda", dtype=torch.int32).view(-1, 4), torch.full((9, 4), -1, device="cuda", dtype=torch.int32)])
    n0 = parts[0] if nparts > 1 else N
    n1 = parts[0] + parts[1] if nparts > 2 else N
    layer = 1
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / math.sqrt(K)
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    for call in range(2):
        x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
        lf = nat.LoraFused(tiles, tiles.shape[0], len(tl), tmaps, 2 * G, 0, G, slot_rank, slot_base, nparts, n0, n1, layer, max(ranks), arena, layer * layer_units, layer * layer_units + nparts * K)
        got = nat.gemm_lora_fused(x, w, lf, bias=b)
        assert got is not None
        torch.cuda.synchronize()
        nat.workspace().check_status()
        want = x.float() @ w.float().t() + b.float()
        bounds = [0, n0, n1, N] if nparts == 3 else ([0, n0, N] if nparts == 2 else [0, N])
        for t, sl in enumerate(rows):
            if sl < 0:
                continue
            r = ranks[sl]
            A = arena[bases[sl] + r * layer * layer_units:][: nparts * r * K].view(nparts * r, K).float()
            B = arena[bases[sl] + r * (layer * layer_units + nparts * K):][: N * r].view(N, r).float()
            v = (A @ x[t].float()).to(torch.bfloat16).float()            # the kernel rounds the shrink result to bf16
            for pp in range(nparts):
                lo, hi = bounds[pp], bounds[pp + 1]
                want[t, lo:hi] += B[lo:hi] @ v[pp * r:(pp + 1) * r]
        assert _rel_err(got, want) < 6e-3, call
        untouched = [i for i, s_ in enumerate(rows) if s_ < 0]
        base = nat.gemm(x, w, bias=b, mode=1)
        assert _rel_err(got[untouched], base[untouched]) < 1e-6


@pytest.mark.parametrize("T,E,k,H,I,e0,e_local", [(7, 8, 2, 512, 256, 0, 8), (256, 8, 2, 1024, 768, 0, 8), (300, 8, 2, 512, 256, 2, 2),
                                                  (1500, 16, 4, 256, 128, 0, 16), (64, 4, 1, 256, 384, 1, 1)])
def test_moe_ffn_on_the_device(nat, T, E, k, H, I, e0, e_local):
    """Routing kernel, gather, grouped tcgen05 GEMMs and combine against the dense fp32 mixture of experts: softmax over all
    experts, top-k, renormalised weights; under expert parallelism (e_local < E) only the local experts' share."""
    torch.manual_seed(T + E)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    wr = (torch.randn(E, H, device="cuda") * 0.3).to(torch.bfloat16)
    w13 = (torch.randn(e_local, 2 * I, H, device="cuda") / math.sqrt(H)).to(torch.bfloat16)
    w2 = (torch.randn(e_local, H, I, device="cuda") / math.sqrt(I)).to(torch.bfloat16)
    r = nat.moe_route(x, wr, k, e0, e_local)
    torch.cuda.synchronize()
    logits = x.float() @ wr.float().t()
    probs = torch.softmax(logits, -1)
    topv, topi = probs.topk(k, -1)
    # the kernel's choice may differ from torch's on near ties: compare the kept probability mass, and ids where the gap is clear
    gap = (probs.sort(-1, descending=True).values[:, k - 1] - probs.sort(-1, descending=True).values[:, k]) if k < E else torch.ones(T, device="cuda")
    clear = gap > 1e-3
    assert torch.equal(r.topk_ids[clear].long().sort(-1).values, topi[clear].sort(-1).values)
    wsum = r.topk_w.sum(-1)
    assert torch.allclose(wsum, torch.ones_like(wsum), atol=1e-5)
    seg = r.seg.tolist()
    assert seg[0] == 0 and all(a <= b for a, b in zip(seg, seg[1:]))
    ids = r.topk_ids.long()
    for e in range(e_local):
        assert seg[e + 1] - seg[e] == int((ids == e0 + e).sum())
    pos = r.pos.long()
    local = (ids >= e0) & (ids < e0 + e_local)
    assert (pos[~local] == -1).all() and (pos[local] >= 0).all()
    st = r.sorted_tok.long()
    tok = torch.arange(T, device="cuda")[:, None].expand(T, k)
    assert torch.equal(st[pos[local]], tok[local])
    out = nat.moe_ffn(x, wr, w13, w2, k, e0, "silu")
    torch.cuda.synchronize()
    nat.workspace().check_status()
    # oracle with the kernel's own routing decision (so that near ties do not matter), dense fp32 experts
    want = torch.zeros(T, H, device="cuda")
    for e in range(e_local):
        sel = (ids == e0 + e)
        wt = (r.topk_w * sel).sum(-1)
        rows = wt > 0
        if rows.any():
            gu = x[rows].float() @ w13[e].float().t()
            a = (torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]).to(torch.bfloat16).float()
            y = (a @ w2[e].float().t()).to(torch.bfloat16).float()
            want[rows] += y * wt[rows, None]
    assert _rel_err(out, want) < 1.2e-2


@pytest.mark.parametrize("T,N,K", [(1, 256, 256), (16, 4096, 4096), (48, 1024, 14336), (100, 6144, 4096), (128, 384, 512),
                                   (300, 4096, 4096), (1000, 1024, 1024)])
def test_gemm_fp8_block128(nat, T, N, K):
    """Block-scaled e4m3 GEMM (128x128 weight scales, 1x128 activation scales) on tcgen05 kind::f8f6f4 against the
    PyTorch oracle that rounds both operands the same way and multiplies in fp32."""
    torch.manual_seed(T + N + K)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    x[:, ::97] *= 8.0                                  # a few outlier columns: the per-block scales must absorb them
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / math.sqrt(K)
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    wq, ws = ref.quantize_weight_fp8_block128(w)
    # the activation quantiser alone
    xq, sa = nat.quant_act_fp8(x)
    xq_ref, sa_ref = ref.quant_act_fp8(x)
    torch.cuda.synchronize()
    assert torch.allclose(sa[:, :T], sa_ref, rtol=1e-6, atol=0)
    a, b_ = xq.view(torch.float8_e4m3fn).float(), xq_ref.float()
    assert ((a - b_).abs() <= b_.abs() * 0.13 + 2e-3).all()          # x * (1 / s) against x / s: at most one e4m3 step apart
    assert (a != b_).float().mean().item() < 0.03
    saved = nat.FP8_EXPAND_MIN_TOKENS
    nat.FP8_EXPAND_MIN_TOKENS = 1 << 30            # the fp8 tensor-core kernel at every size
    try:
        out = nat.gemm_fp8(x, wq, ws, bias=b)
    finally:
        nat.FP8_EXPAND_MIN_TOKENS = saved
    torch.cuda.synchronize()
    nat.workspace().check_status()
    want = ref.gemm_fp8(x, wq, ws, bias=b)
    assert _rel_err(out, want) < 6e-3
    # long prefills expand the weights to bf16 and keep the activations in bf16: the oracle is x @ dequant(w)^T
    nat.FP8_EXPAND_MIN_TOKENS = 1
    try:
        out2 = nat.gemm_fp8(x, wq, ws, bias=b)
    finally:
        nat.FP8_EXPAND_MIN_TOKENS = saved
    torch.cuda.synchronize()
    nat.workspace().check_status()
    want2 = x.float() @ ref.dequantize_weight_fp8_block128(wq, ws).float().t()[:K, :N] + b.float() if False else \
        x.float() @ ref.dequantize_weight_fp8_block128(wq, ws)[:N, :K].float().t() + b.float()
    assert _rel_err(out2, want2) < 6e-3
    # and the quantised product is close to the bf16 one
    full = x.float() @ w.float().t() + b.float()
    assert _rel_err(out, full) < 6e-2


def test_fp8_weights_expanded_for_long_steps_carry_lora_in_the_gemm_launch(nat):
    """A long step over block-scaled e4m3 weights: the weights are expanded to bf16 once and the GEMM that carries the adapters runs
    over them; against fp32 PyTorch on the dequantised weights."""
    torch.manual_seed(11)
    T, K, parts, ranks = 640, 1024, [512, 256], [16, 32]
    nparts, N = len(parts), sum(parts)
    layer_units = nparts * K + N
    bases, off = [], 0
    for r in ranks:
        bases.append(off)
        off += (r * layer_units + 63) // 64 * 64
    arena = (torch.randn(off, device="cuda") * 0.05).to(torch.bfloat16)
    slot_base = torch.tensor(bases, device="cuda", dtype=torch.int64)
    slot_rank = torch.tensor(ranks, device="cuda", dtype=torch.int32)
    G = 5
    tm_host = torch.zeros(len(ranks) * 2 * G * 128, dtype=torch.uint8).pin_memory()
    for s_, r in enumerate(ranks):
        nat.lora_encode_tmap(tm_host[(s_ * 2 * G) * 128:], arena.data_ptr() + bases[s_] * 2, K, nparts * r, r * layer_units, 1)
        nat.lora_encode_tmap_b(tm_host[(s_ * 2 * G + G) * 128:], arena.data_ptr() + (bases[s_] + r * nparts * K) * 2, r, N, r * layer_units, 1)
    tmaps = tm_host.cuda()
    rows = [0] * 200 + [-1] * 40 + [1] * 400
    tl = ref.build_lora_tiles(rows, 32)
    tiles = torch.cat([torch.tensor(tl, device="cuda", dtype=torch.int32).view(-1, 4), torch.full((7, 4), -1, device="cuda", dtype=torch.int32)])
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / math.sqrt(K)
    wq, wscale = ref.quantize_weight_fp8_block128(w)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w16 = nat.fp8_expand(wq.view(torch.uint8), wscale)
    assert w16 is not None
    wd = ref.dequantize_weight_fp8_block128(wq, wscale)[:N, :K].float()
    assert _rel_err(w16.float(), wd) < 1e-2
    lf = nat.LoraFused(tiles, tiles.shape[0], len(tl), tmaps, 2 * G, 0, G, slot_rank, slot_base, nparts, parts[0], N, 0, max(ranks), arena, 0, nparts * K)
    got = nat.gemm_lora_fused(x, w16, lf)
    assert got is not None
    torch.cuda.synchronize()
    nat.workspace().check_status()
    want = x.float() @ wd.t()
    bounds = [0, parts[0], N]
    for sl in (0, 1):
        r = ranks[sl]
        idx = torch.tensor([t for t, s_ in enumerate(rows) if s_ == sl], device="cuda")
        A = arena[bases[sl]:][: nparts * r * K].view(nparts * r, K).float()
        B = arena[bases[sl] + r * nparts * K:][: N * r].view(N, r).float()
        v = (x[idx].float() @ A.t()).to(torch.bfloat16).float()
        for pp in range(nparts):
            lo, hi = bounds[pp], bounds[pp + 1]
            want[idx, lo:hi] += v[:, pp * r:(pp + 1) * r] @ B[lo:hi].t()
    assert _rel_err(got, want) < 6e-3
