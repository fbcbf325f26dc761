"""Plain PyTorch statements of every operator.

They are the oracle for the CUDA kernels (tests compare a kernel against the fp32 version of the same
function) and the compute path of the engine on a machine without a GPU.  Signatures mirror
:mod:`lorax_b200.ops.native`.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def gemm(x, w, bias=None, out=None, out_scale: float = 1.0, lora=None, **_):
    y = (x.float() @ w.float().t()) * out_scale
    if bias is not None:
        y = y + bias.float()
    if lora is not None:      # the CUDA kernel adds the delta in its epilogue, before the one rounding to bf16
        d = torch.zeros_like(y)
        lora_expand(lora.v, lora.tok_slot, lora.arena, lora.slot_base, lora.slot_rank, lora.unit_off, d, lora.n0, lora.n1)
        y = y + d
    y = y.to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


FP8_MAX = 448.0


def quantize_weight_fp8_block128(w: torch.Tensor):
    """[N, K] -> (e4m3 [N, K], fp32 scales [ceil(N/128), ceil(K/128)]): w ~= q * scale of its 128 x 128 block."""
    N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    wp = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, 128, kb, 128)
    scale = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12) / FP8_MAX
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(nb * 128, kb * 128)[:N, :K].to(torch.float8_e4m3fn)
    return q.contiguous(), scale.contiguous()


def dequantize_weight_fp8_block128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    s = scale.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    return q.view(torch.float8_e4m3fn).float() * s


def quant_act_fp8(x):
    """Per token and 128-wide K block: (e4m3 [T, K], scales [K/128, T])."""
    T, K = x.shape
    kb = (K + 127) // 128
    xp = torch.zeros(T, kb * 128, dtype=torch.float32, device=x.device)
    xp[:, :K] = x.float()
    b = xp.view(T, kb, 128)
    scale = b.abs().amax(dim=2).clamp_min(1e-12) / FP8_MAX
    q = (b / scale[:, :, None]).clamp(-FP8_MAX, FP8_MAX).view(T, kb * 128)[:, :K].to(torch.float8_e4m3fn)
    return q.contiguous(), scale.t().contiguous()


def gemm_wq(x, w, bias=None, out=None):
    """Oracle of the weight-only quantised GEMM: the packed matrix expanded to the activation dtype, then a plain product."""
    from ..utils.quant_formats import dequantize
    y = x.float() @ dequantize(w, torch.float32).to(x.dtype).float().t()
    if bias is not None:
        y = y + bias.float()
    y = y.to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def gemm_fp8(x, wq, w_scale, bias=None, out=None):
    """Oracle of the block-scaled fp8 GEMM: both operands rounded to e4m3 with their scales, product in fp32."""
    xq, sa = quant_act_fp8(x)
    T, K = x.shape
    xd = xq.float() * sa.t().repeat_interleave(128, 1)[:, :K]
    y = xd @ dequantize_weight_fp8_block128(wq, w_scale).t()
    if bias is not None:
        y = y + bias.float()
    y = y.to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def norm_residual(x, residual, weight, eps, bias=None, out=None, weight_offset: float = 0.0, x_scale: float = 1.0,
                  layernorm: bool = False):
    h = x.float() * x_scale
    if residual is not None:
        h = h + residual.float()
        residual.copy_(h.to(residual.dtype))
        h = residual.float()
    if layernorm:
        mean = h.mean(-1, keepdim=True)
        var = (h * h).mean(-1, keepdim=True) - mean * mean
        y = (h - mean) * torch.rsqrt(var.clamp_min(0) + eps)
    else:
        y = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps)
    y = y * (weight.float() + weight_offset)
    if bias is not None:
        y = y + bias.float()
    y = y.to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def apply_rope(x, cos, sin, rot):
    """x: [T, heads, d]; cos/sin: [T, rot/2].  Rotate-half convention on the first `rot` dims."""
    half = rot // 2
    x1, x2, rest = x[..., :half].float(), x[..., half:rot].float(), x[..., rot:]
    c, s = cos[:, None, :], sin[:, None, :]
    o1 = x1 * c - x2 * s
    o2 = x2 * c + x1 * s
    return torch.cat([o1.to(x.dtype), o2.to(x.dtype), rest], dim=-1)


def _to_e4m3_bytes(x, scale):
    """x / scale as e4m3 bytes, saturating at +-448 like the kernel."""
    return (x.float() / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


def rope_kvwrite(qkv, positions, cos_sin, kv_cache, slots, nh, nkv, d, rot, apply_rope_flag: bool = True, kv_scale=None):
    """In place on qkv [T, (nh+2nkv)*d]; kv_cache [blocks, nkv, 2, page, d] (bf16 / fp32, or e4m3 holding value / scale)."""
    T = qkv.shape[0]
    page = kv_cache.shape[3]
    q = qkv[:, : nh * d].view(T, nh, d)
    k = qkv[:, nh * d: (nh + nkv) * d].view(T, nkv, d)
    v = qkv[:, (nh + nkv) * d: (nh + 2 * nkv) * d].view(T, nkv, d)
    if apply_rope_flag:
        cs = cos_sin[positions.long()]
        cos, sin = cs[:, : rot // 2], cs[:, rot // 2: rot]
        q.copy_(apply_rope(q, cos, sin, rot))
        k.copy_(apply_rope(k, cos, sin, rot))
    if slots is not None:
        ok = slots >= 0
        s = slots[ok].long()
        blk, off = s // page, s % page
        if kv_cache.dtype == torch.float8_e4m3fn:
            ks, vs = kv_scale or (1.0, 1.0)
            raw = kv_cache.view(torch.uint8)
            raw[blk, :, 0, off, :] = _to_e4m3_bytes(k[ok], ks)
            raw[blk, :, 1, off, :] = _to_e4m3_bytes(v[ok], vs)
        else:
            kv_cache[blk, :, 0, off, :] = k[ok]
            kv_cache[blk, :, 1, off, :] = v[ok]


def _act(x, act):
    if act in ("silu", "swish"):
        return F.silu(x)
    if act == "gelu":
        return F.gelu(x)
    if act in ("gelu_new", "gelu_pytorch_tanh", "gelu_fast", "gelu_tanh"):
        return F.gelu(x, approximate="tanh")
    if act == "relu":
        return F.relu(x)
    raise ValueError(act)


def act_mul(x, inter, act="silu", gated=True, out=None):
    g = _act(x[:, :inter].float(), act)
    if gated:
        g = g * x[:, inter: 2 * inter].float()
    g = g.to(x.dtype)
    if out is not None:
        out.copy_(g)
        return out
    return g


def embed(ids, table, v0=0, v1=None, mult=1.0, out=None):
    if v1 is None:
        v1 = v0 + table.shape[0]
    idl = ids.long()
    ok = (idl >= v0) & (idl < v1)
    y = table[(idl - v0).clamp(0, table.shape[0] - 1)]
    if mult != 1.0:
        y = (y.float() * mult).to(table.dtype)
    y = torch.where(ok[:, None], y, torch.zeros_like(y))
    if out is not None:
        out.copy_(y)
        return out
    return y


def argmax_logprob(logits, ids=None, logprobs=None, softcap: float = 0.0):
    x = logits.float()
    if softcap > 0:
        x = softcap * torch.tanh(x / softcap)
    i = x.argmax(-1)
    lp = torch.log_softmax(x, -1).gather(1, i[:, None])[:, 0]
    if ids is not None:
        ids.copy_(i.to(ids.dtype))
        logprobs.copy_(lp)
        return ids, logprobs
    return i.to(torch.int32), lp


def advance_decode(input_ids, next_ids, positions, ctx_lens, slots, block_tables, page):
    live = ctx_lens > 0
    input_ids[live] = next_ids[live].to(input_ids.dtype)
    positions[live] += 1
    ctx_lens[live] = positions[live] + 1
    pos = positions.long()
    blk = block_tables.gather(1, (pos // page).clamp(0, block_tables.shape[1] - 1)[:, None])[:, 0]
    new_slots = blk * page + (pos % page).to(blk.dtype)
    slots.copy_(torch.where(live, new_slots.to(slots.dtype), torch.full_like(slots, -1)))


def prefill_metadata(cu_q, cache_lens, seq_slot, block_tables, page, T):
    """-> (positions [T], slots [T], tok_slot [T]) int32 of a ragged prefill whose sequence b owns tokens [cu_q[b], cu_q[b+1])."""
    t = torch.arange(T, device=cu_q.device)
    b = torch.searchsorted(cu_q[1:].long().contiguous(), t, right=True).clamp(max=cache_lens.shape[0] - 1)
    pos = cache_lens.long()[b] + (t - cu_q.long()[b])
    blk = (pos // page).clamp(max=block_tables.shape[1] - 1)
    slots = block_tables.long()[b, blk] * page + pos % page
    return pos.to(torch.int32), slots.to(torch.int32), seq_slot[b].to(torch.int32)


def _gather_kv(kv_cache, block_table, n_keys, kvh, kv_scale=None):
    """-> K [n_keys, d], V [n_keys, d] for one sequence and kv head."""
    page = kv_cache.shape[3]
    nblk = (n_keys + page - 1) // page
    blocks = block_table[:nblk].long()
    if kv_cache.dtype == torch.float8_e4m3fn:
        ks, vs = kv_scale or (1.0, 1.0)
        raw = kv_cache.view(torch.uint8)
        k = raw[blocks, kvh, 0].reshape(-1, kv_cache.shape[-1])[:n_keys].view(torch.float8_e4m3fn).float() * ks
        v = raw[blocks, kvh, 1].reshape(-1, kv_cache.shape[-1])[:n_keys].view(torch.float8_e4m3fn).float() * vs
        return k, v
    k = kv_cache[blocks, kvh, 0].reshape(-1, kv_cache.shape[-1])[:n_keys]
    v = kv_cache[blocks, kvh, 1].reshape(-1, kv_cache.shape[-1])[:n_keys]
    return k, v


def _attend(q, k, v, q_pos, scale, window, softcap, slope=None):
    """q: [nq, d] at absolute positions q_pos [nq]; k, v: [nk, d] at positions 0..nk-1.  `slope` (scalar or [nq]) adds the
    ALiBi bias -slope * (query position - key position)."""
    s = (q.float() @ k.float().t()) * scale
    if softcap and softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    kp = torch.arange(k.shape[0], device=q.device)[None, :]
    if slope is not None:
        sl = slope if torch.is_tensor(slope) and slope.dim() else torch.as_tensor(slope, device=q.device).reshape(1)
        s = s - sl.float().reshape(-1, 1) * (q_pos[:, None] - kp).float()
    mask = kp <= q_pos[:, None]
    if window and window > 0:
        mask &= kp > (q_pos[:, None] - window)
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    p = torch.nan_to_num(p, nan=0.0)
    return p @ v.float()


def attn_decode(q, kv_cache, block_tables, ctx_lens, nh, nkv, d, scale, window=0, softcap=0.0, nsplit=1, out=None, alibi=None,
                kv_scale=None):
    T = q.shape[0]
    res = torch.zeros(T, nh * d, dtype=q.dtype, device=q.device)
    g = nh // nkv
    for t in range(T):
        n = int(ctx_lens[t])
        if n <= 0:
            continue
        for kvh in range(nkv):
            k, v = _gather_kv(kv_cache, block_tables[t], n, kvh, kv_scale)
            qh = q[t, kvh * g * d: (kvh + 1) * g * d].view(g, d)
            o = _attend(qh, k, v, torch.full((g,), n - 1, device=q.device), scale, window, softcap,
                        None if alibi is None else alibi[kvh * g: (kvh + 1) * g])
            res[t, kvh * g * d: (kvh + 1) * g * d] = o.reshape(-1).to(q.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def attn_prefill(q, kv_cache, block_tables, cu_q, cache_lens, tile_seq, tile_q0, nh, nkv, d, scale, window=0, softcap=0.0,
                 out=None, alibi=None, kv_scale=None):
    T = q.shape[0]
    res = torch.zeros(T, nh * d, dtype=q.dtype, device=q.device)
    g = nh // nkv
    B = cache_lens.shape[0]
    for b in range(B):
        s, e = int(cu_q[b]), int(cu_q[b + 1])
        if e <= s:
            continue
        c = int(cache_lens[b])
        n = c + (e - s)
        pos = torch.arange(c, n, device=q.device)
        for kvh in range(nkv):
            k, v = _gather_kv(kv_cache, block_tables[b], n, kvh, kv_scale)
            for gi in range(g):
                h = kvh * g + gi
                o = _attend(q[s:e, h * d: (h + 1) * d], k, v, pos, scale, window, softcap, None if alibi is None else alibi[h])
                res[s:e, h * d: (h + 1) * d] = o.to(q.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def prefill_tiles(q_lens, tile: int = 64):
    """Host-side tile map for attn_prefill: (tile_seq, tile_q0) int32 lists."""
    seq, q0 = [], []
    for b, n in enumerate(q_lens):
        for s in range(0, n, tile):
            seq.append(b)
            q0.append(s)
    return seq, q0


def lora_shrink(x, tok_slot, arena, slot_base, slot_rank, unit_off, nparts, max_rank, v=None):
    T, K = x.shape
    if v is None:
        v = torch.zeros(T, nparts * max_rank, dtype=torch.float32, device=x.device)
    for t in range(T):
        s = int(tok_slot[t])
        if s < 0 or int(slot_base[s]) < 0:
            continue
        r = int(slot_rank[s])
        off = int(slot_base[s]) + r * unit_off
        A = arena[off: off + nparts * r * K].view(nparts * r, K)
        v[t, : nparts * r] = x[t].float() @ A.float().t()
    return v


def lora_expand(v, tok_slot, arena, slot_base, slot_rank, unit_off, y, n0, n1):
    T, N = y.shape
    bounds = [0, n0, n1, N]
    for t in range(T):
        s = int(tok_slot[t])
        if s < 0 or int(slot_base[s]) < 0:
            continue
        r = int(slot_rank[s])
        off = int(slot_base[s]) + r * unit_off
        B = arena[off: off + N * r].view(N, r).float()
        delta = torch.zeros(N, dtype=torch.float32, device=y.device)
        for part in range(3):
            a, b = bounds[part], bounds[part + 1]
            if b > a:
                delta[a:b] = B[a:b] @ v[t, part * r: (part + 1) * r].float()
        y[t] = (y[t].float() + delta).to(y.dtype)


def lora_shrink_tiles(x, tiles, num_tiles, max_tile_rows, arena, slot_base, slot_rank, unit_off, nparts, max_rank, v=None):
    """Tile-table form (tiles: int32 [n, 4] = slot, row0, nrows, -).  The CPU oracle reads A_cat straight from the
    arena; the CUDA kernel reads the same bytes through the per-slot tensor maps."""
    T, K = x.shape
    if v is None:
        v = torch.zeros(T, nparts * max_rank, dtype=torch.float32, device=x.device)
    for i in range(num_tiles):
        s, row0, n, _ = (int(q) for q in tiles[i])
        n = min(n, T - row0)                 # a table may be older than the batch: rows past T are gone
        if s < 0 or n <= 0 or int(slot_base[s]) < 0:
            continue
        r = int(slot_rank[s])
        off = int(slot_base[s]) + r * unit_off
        A = arena[off: off + nparts * r * K].view(nparts * r, K).float()
        v[row0:row0 + n, : nparts * r] = x[row0:row0 + n].float() @ A.t()
    return v


def lora_expand_tiles(v, tiles, num_tiles, max_tile_rows, arena, slot_base, slot_rank, unit_off, y, n0, n1):
    T, N = y.shape
    bounds = [0, n0, n1, N]
    for i in range(num_tiles):
        s, row0, n, _ = (int(q) for q in tiles[i])
        n = min(n, T - row0)
        if s < 0 or n <= 0 or int(slot_base[s]) < 0:
            continue
        r = int(slot_rank[s])
        off = int(slot_base[s]) + r * unit_off
        B = arena[off: off + N * r].view(N, r).float()
        delta = torch.zeros(n, N, dtype=torch.float32, device=y.device)
        for part in range(3):
            a, b = bounds[part], bounds[part + 1]
            if b > a:
                delta[:, a:b] = v[row0:row0 + n, part * r:(part + 1) * r].float() @ B[a:b].t()
        y[row0:row0 + n] = (y[row0:row0 + n].float() + delta).to(y.dtype)


def build_lora_tiles(slots_per_row, max_rows: int):
    """Host helper: rows with equal adapter slot that are adjacent form a segment; segments are cut into tiles of at
    most `max_rows` rows.  -> list of (slot, row0, nrows, 0); rows without adapter (slot < 0) get no tile."""
    tiles = []
    i, n = 0, len(slots_per_row)
    while i < n:
        s = slots_per_row[i]
        j = i
        while j < n and slots_per_row[j] == s:
            j += 1
        if s >= 0:
            for a in range(i, j, max_rows):
                tiles.append((s, a, min(max_rows, j - a), 0))
        i = j
    return tiles


def rope_cache(rot: int, max_pos: int, theta: float, scaling: Optional[dict] = None, device="cpu") -> torch.Tensor:
    """[max_pos, rot] fp32 table: cos in the first half, sin in the second.

    Scaling variants follow `server/lorax_server/utils/layers.py:484-816` of the reference: linear,
    dynamic NTK, YaRN, Su/LongRoPE and llama3.
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    mscale = 1.0
    t = torch.arange(max_pos, dtype=torch.float32)
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type", "default"))
        factor = float(scaling.get("factor", 1.0))
        if kind == "linear":
            t = t / factor
        elif kind == "dynamic":
            orig = int(scaling.get("original_max_position_embeddings", max_pos))
            if max_pos > orig:
                base = theta * ((factor * max_pos / orig) - (factor - 1)) ** (rot / (rot - 2))
                inv_freq = 1.0 / (base ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
        elif kind == "llama3":
            low = float(scaling.get("low_freq_factor", 1.0))
            high = float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv_freq
            smooth = ((orig / wavelen) - low) / (high - low)
            scaled = torch.where(wavelen > orig / low, inv_freq / factor, inv_freq)
            mid = (wavelen <= orig / low) & (wavelen >= orig / high)
            inv_freq = torch.where(mid, (1 - smooth) * inv_freq / factor + smooth * inv_freq, scaled)
        elif kind == "yarn":
            orig = float(scaling.get("original_max_position_embeddings", 4096))
            beta_fast, beta_slow = float(scaling.get("beta_fast", 32)), float(scaling.get("beta_slow", 1))

            def corr_dim(nrot):
                return (rot * math.log(orig / (nrot * 2 * math.pi))) / (2 * math.log(theta))

            lo = max(math.floor(corr_dim(beta_fast)), 0)
            hi = min(math.ceil(corr_dim(beta_slow)), rot - 1)
            ramp = ((torch.arange(rot // 2, dtype=torch.float32) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
            inv_mask = 1 - ramp
            inv_freq = (inv_freq / factor) * (1 - inv_mask) + inv_freq * inv_mask
            mscale = float(scaling.get("attention_factor") or (0.1 * math.log(factor) + 1.0 if factor > 1 else 1.0))
        elif kind in ("su", "longrope"):
            orig = int(scaling.get("original_max_position_embeddings", max_pos))
            ext = torch.tensor(scaling["long_factor"] if max_pos > orig else scaling["short_factor"], dtype=torch.float32)
            inv_freq = inv_freq / ext
            sc = max_pos / orig
            mscale = 1.0 if sc <= 1 else math.sqrt(1 + math.log(sc) / math.log(orig))
    freqs = torch.outer(t, inv_freq)
    return torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1).to(device)
