"""Weight-only quantisation formats and the one resident layout the kernels read.

The reference serves GPTQ (exllama / exllamav2 / Triton), AWQ, EETQ (int8), bitsandbytes (int8, nf4, fp4) and HQQ (4 / 3 / 2 bit)
through one extension per format (`server/lorax_server/layers/linear.py:93-181`).  Here every format is converted at load time
into `GroupQuantWeight`:

    codes   uint8 [N, K * bits / 8]   bits in {2, 4, 8}; for 4 bits the eight codes of each 32-bit word are interleaved
                                      (nibble i holds k = 8 * word + NIBBLE_K[i]) so the kernel's mask-and-or expansion yields
                                      pairs of neighbouring k
    sz      float16 [N, K / group, 2] (scale, zero): w = (code - zero) * scale
    table   float32 [16] or None      code-book formats (nf4 / fp4): w = table[code] * scale

and `lorax_b200/csrc/kernels/quant_wo.cu` multiplies straight from it.  This module holds

* readers of the checkpoint layouts (AutoGPTQ `qweight / qzeros / scales / g_idx`, AutoAWQ `qweight / qzeros / scales`) and
  packers that write them (used by the offline quantiser and by the tests),
* the on-load quantisers: round-to-nearest affine groups (int4 / int8 per channel = EETQ and bitsandbytes int8), nf4 / fp4
  code books with block-wise absmax (bitsandbytes), HQQ's half-quadratic zero-point refinement,
* GPTQ itself (Hessian-compensated rounding, `utils/gptq/quantize.py` in the reference).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

NIBBLE_K = (0, 2, 4, 6, 1, 3, 5, 7)          # nibble i of a word -> k offset
AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)         # AutoAWQ packs column order[i] into nibble i

NF4_TABLE = (-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635, -0.18477343022823334,
             -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
             0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0)
# fp4 (1 sign, 2 exponent, 1 mantissa bit) normalised to [-1, 1], in code order
FP4_TABLE = (0.0, 0.0052083333, 0.6666666667, 1.0, 0.3333333333, 0.5, 0.1666666667, 0.25,
             -0.0, -0.0052083333, -0.6666666667, -1.0, -0.3333333333, -0.5, -0.1666666667, -0.25)


@dataclass
class GroupQuantWeight:
    """A projection matrix [N, K] (out, in) in the resident packed layout."""
    codes: torch.Tensor
    sz: torch.Tensor
    bits: int
    group: int
    shape: Tuple[int, int]
    table: Optional[torch.Tensor] = None
    method: str = "int4"
    int_zero: bool = False          # every zero point is an integer (GPTQ, AWQ, round-to-nearest): the 4-bit kernel's exact path
    # act-order GPTQ: stored column i is input feature perm[i] (int32 [K]), which makes every group a contiguous run again; the
    # caller multiplies x[:, perm] by this matrix (exllama's x_map: exllama_kernels/cuda_func/q4_matmul.cu in the reference)
    perm: Optional[torch.Tensor] = None

    @property
    def device(self):
        return self.codes.device

    def to(self, device) -> "GroupQuantWeight":
        return GroupQuantWeight(self.codes.to(device), self.sz.to(device), self.bits, self.group, self.shape,
                                None if self.table is None else self.table.to(device), self.method, self.int_zero,
                                None if self.perm is None else self.perm.to(device))

    def nbytes(self) -> int:
        return self.codes.numel() + self.sz.numel() * 2 + (0 if self.perm is None else self.perm.numel() * 4)

    # ---- slicing used by tensor-parallel sharding (`w[a:b]` = rows, `w[:, a:b]` = columns, like a tensor)
    def __getitem__(self, key):
        if isinstance(key, slice):
            a, b, _ = key.indices(self.shape[0])
            return self.rows(a, b)
        if isinstance(key, tuple) and len(key) == 2 and key[0] == slice(None) and isinstance(key[1], slice):
            a, b, _ = key[1].indices(self.shape[1])
            return self.cols(a, b)
        raise TypeError(f"a packed weight supports row and column slices only, not {key!r}")

    def rows(self, start: int, stop: int) -> "GroupQuantWeight":
        return GroupQuantWeight(self.codes[start:stop].contiguous(), self.sz[start:stop].contiguous(), self.bits, self.group,
                                (stop - start, self.shape[1]), self.table, self.method, self.int_zero, self.perm)

    def cols(self, start: int, stop: int) -> "GroupQuantWeight":
        if start == 0 and stop == self.shape[1]:
            return self
        if self.perm is not None:
            raise ValueError("an act-order layer cannot be sharded by input columns while packed: its groups mix columns of all shards")
        if start % self.group or stop % self.group:
            raise ValueError(f"a column shard must start and end on a group boundary ({self.group}); got [{start}, {stop})")
        b = self.bits
        return GroupQuantWeight(self.codes[:, start * b // 8: stop * b // 8].contiguous(),
                                self.sz[:, start // self.group: stop // self.group].contiguous(), self.bits, self.group,
                                (self.shape[0], stop - start), self.table, self.method, self.int_zero)


def cat_rows(parts) -> GroupQuantWeight:
    p0 = parts[0]
    assert all(p.bits == p0.bits and p.group == p0.group and p.shape[1] == p0.shape[1] for p in parts)
    assert same_perm(parts), "projections with different act-order permutations cannot share one packed matrix"
    return GroupQuantWeight(torch.cat([p.codes for p in parts], 0), torch.cat([p.sz for p in parts], 0), p0.bits, p0.group,
                            (sum(p.shape[0] for p in parts), p0.shape[1]), p0.table, p0.method, all(p.int_zero for p in parts), p0.perm)


def same_perm(parts) -> bool:
    """Whether packed matrices read their input in the same column order (q / k / v, or gate / up, of an act-order GPTQ
    checkpoint do: the order comes from the Hessian of their common input)."""
    p0 = parts[0].perm
    if p0 is None:
        return all(p.perm is None for p in parts)
    return all(p.perm is not None and torch.equal(p.perm.cpu(), p0.cpu()) for p in parts)


# ------------------------------------------------------------------------------------------------ resident layout

def pack_codes(q: torch.Tensor, bits: int) -> torch.Tensor:
    """Integer codes [N, K] -> uint8 [N, K * bits / 8] in the resident order."""
    N, K = q.shape
    q = q.to(torch.int32)
    if bits == 8:
        return q.to(torch.uint8).contiguous()
    if bits == 4:
        if K % 8:
            raise ValueError("4-bit rows must be a multiple of 8 long")
        w = q.view(N, K // 8, 8)
        nib = torch.empty_like(w)
        for i, k in enumerate(NIBBLE_K):
            nib[..., i] = w[..., k]
        return (nib[..., 0::2] | (nib[..., 1::2] << 4)).to(torch.uint8).view(N, K // 2).contiguous()
    if bits == 2:
        w = q.view(N, K // 4, 4)
        return (w[..., 0] | (w[..., 1] << 2) | (w[..., 2] << 4) | (w[..., 3] << 6)).to(torch.uint8).contiguous()
    raise ValueError(f"bits={bits}")


def unpack_codes(codes: torch.Tensor, bits: int, K: int) -> torch.Tensor:
    """Inverse of `pack_codes`: int32 [N, K]."""
    N = codes.shape[0]
    c = codes.to(torch.int32)
    if bits == 8:
        return c
    if bits == 4:
        nib = torch.stack([c & 15, c >> 4], -1).view(N, K // 8, 8)
        out = torch.empty_like(nib)
        for i, k in enumerate(NIBBLE_K):
            out[..., k] = nib[..., i]
        return out.view(N, K)
    if bits == 2:
        return torch.stack([c & 3, (c >> 2) & 3, (c >> 4) & 3, (c >> 6) & 3], -1).view(N, K)
    raise ValueError(f"bits={bits}")


def make_weight(q: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, bits: int, group: int, table=None,
                method: str = "int4") -> GroupQuantWeight:
    """codes [N, K] ints, scale / zero [N, K / group] floats."""
    N, K = q.shape
    sz = torch.stack([scale.float(), zero.float()], -1).to(torch.float16).contiguous()
    tab = None if table is None else torch.tensor(table, dtype=torch.float32, device=q.device)
    int_zero = table is None and bool(torch.equal(sz[..., 1].float(), sz[..., 1].float().round()))
    return GroupQuantWeight(pack_codes(q, bits), sz, bits, group, (N, K), tab, method, int_zero)


def dequantize(w: GroupQuantWeight, dtype=torch.float32) -> torch.Tensor:
    """The matrix the kernels multiply by, [N, K]."""
    N, K = w.shape
    q = unpack_codes(w.codes, w.bits, K)
    s = w.sz[..., 0].float().repeat_interleave(w.group, 1)
    if w.table is not None:
        d = w.table.float()[q.long()] * s
    else:
        d = (q.float() - w.sz[..., 1].float().repeat_interleave(w.group, 1)) * s
    if w.perm is not None:                             # stored column i is input feature perm[i]
        d = torch.empty_like(d).index_copy_(1, w.perm.long(), d)
    return d.to(dtype)


# ------------------------------------------------------------------------------------------------ on-load quantisers

def quantize_rtn(w: torch.Tensor, bits: int = 4, group: int = 128, symmetric: bool = False, method: Optional[str] = None) -> GroupQuantWeight:
    """Round-to-nearest affine groups along K.  `group <= 0` means one group per row (per-channel scales: the EETQ and
    bitsandbytes-int8 layout).  Asymmetric: the group's min and max map to codes 0 and 2^bits - 1, so a matrix that already lies
    on such a grid (a dequantised GPTQ / AWQ checkpoint with contiguous groups) is reproduced exactly."""
    N, K = w.shape
    g = K if group <= 0 else group
    if K % g:
        raise ValueError(f"K={K} is not a multiple of the group size {g}")
    maxq = (1 << bits) - 1
    x = w.float().view(N, K // g, g)
    if symmetric:
        amax = x.abs().amax(-1).clamp_min(1e-8)
        scale = amax / ((maxq - 1) / 2)
        zero = torch.full_like(scale, (maxq + 1) / 2)
    else:
        lo, hi = x.amin(-1), x.amax(-1)
        scale = ((hi - lo) / maxq).clamp_min(1e-8)
        zero = torch.round(-lo / scale)
    scale = scale.to(torch.float16).float()             # the scale the kernel will see
    q = torch.clamp(torch.round(x / scale[..., None] + zero[..., None]), 0, maxq).to(torch.int32).view(N, K)
    return make_weight(q, scale, zero, bits, g, method=method or f"int{bits}")


def quantize_codebook(w: torch.Tensor, table=NF4_TABLE, block: int = 64, method: str = "nf4") -> GroupQuantWeight:
    """bitsandbytes' 4-bit formats: every block of `block` weights is divided by its absmax and each value takes the nearest
    entry of a 16-entry table (layers/bnb.py: Linear4bit with quant_type nf4 / fp4)."""
    N, K = w.shape
    if K % block:
        raise ValueError(f"K={K} is not a multiple of the block size {block}")
    x = w.float().view(N, K // block, block)
    absmax = x.abs().amax(-1).clamp_min(1e-8).to(torch.float16).float()
    tab = torch.tensor(table, dtype=torch.float32, device=w.device)
    q = (x / absmax[..., None]).unsqueeze(-1).sub(tab).abs().argmin(-1).to(torch.int32).view(N, K)
    return make_weight(q, absmax, torch.zeros_like(absmax), 4, block, table=table, method=method)


def quantize_hqq(w: torch.Tensor, bits: int = 4, group: int = 64, iters: int = 20, lp_norm: float = 0.7, beta: float = 10.0,
                 kappa: float = 1.01) -> GroupQuantWeight:
    """Half-quadratic quantisation (layers/hqq.py: HQQLinear with nbits 4 / 3 / 2, group 64): start from the min-max grid and
    refine the (fractional) zero point by alternating a generalised soft-threshold on the error with a closed-form zero
    update.  3-bit codes are stored in 4-bit containers."""
    N, K = w.shape
    if K % group:
        raise ValueError(f"K={K} is not a multiple of the group size {group}")
    maxq = (1 << bits) - 1
    x = w.float().view(N, K // group, group)
    lo, hi = x.amin(-1, keepdim=True), x.amax(-1, keepdim=True)
    inv_scale = (maxq / (hi - lo).clamp_min(1e-8))
    zero = -lo * inv_scale
    best_err, best_zero = None, zero
    for _ in range(iters):
        q = torch.clamp(torch.round(x * inv_scale + zero), 0, maxq)
        r = (q - zero) / inv_scale
        e = x - r
        # shrinkage operator of the l_p norm (p < 1)
        e = torch.sign(e) * torch.relu(e.abs() - (1.0 / beta) * e.abs().clamp_min(1e-8).pow(lp_norm - 1))
        zero = (q - (x - e) * inv_scale).mean(-1, keepdim=True)
        beta *= kappa
        err = (x - r).abs().mean().item()
        if best_err is not None and err >= best_err:
            break
        best_err, best_zero = err, zero
    zero = best_zero
    q = torch.clamp(torch.round(x * inv_scale + zero), 0, maxq).to(torch.int32).view(N, K)
    store = 4 if bits == 3 else bits
    return make_weight(q, (1.0 / inv_scale)[..., 0], zero[..., 0], store, group, method=f"hqq-{bits}bit")


QUANT_METHODS = ("int4", "int8", "gptq", "awq", "eetq", "bitsandbytes", "bitsandbytes-nf4", "bitsandbytes-fp4", "hqq-4bit", "hqq-3bit",
                 "hqq-2bit")


def quantize_weight(w: torch.Tensor, method: str, group: int = 128) -> GroupQuantWeight:
    """Quantise a dense matrix for serving under one of the reference's `--quantize` names (cli.py:15-28).  `gptq` and `awq`
    name checkpoint formats; applied to a dense matrix they mean 4-bit groups of 128 with round-to-nearest."""
    K = w.shape[1]

    def fit(g):                                        # the largest power-of-two fraction of g that divides K
        while g > 32 and K % g:
            g //= 2
        return g
    if method in ("int4", "gptq", "awq"):
        return quantize_rtn(w, 4, fit(group), method=method)
    if method in ("int8", "eetq", "bitsandbytes"):
        return quantize_rtn(w, 8, 0, symmetric=True, method=method)
    if method == "bitsandbytes-nf4":
        return quantize_codebook(w, NF4_TABLE, fit(64), "nf4")
    if method == "bitsandbytes-fp4":
        return quantize_codebook(w, FP4_TABLE, fit(64), "fp4")
    if method.startswith("hqq-"):
        return quantize_hqq(w, int(method[4]), fit(64))
    raise ValueError(f"unknown quantisation method {method!r}; known: {', '.join(QUANT_METHODS)}")


# ------------------------------------------------------------------------------------------------ checkpoint layouts

def _unpack_int32(t: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    """Expand every int32 along `dim` into 32 / bits codes (code j at bit j * bits)."""
    per = 32 // bits
    shifts = torch.arange(per, dtype=torch.int32, device=t.device) * bits
    mask = (1 << bits) - 1
    if dim == 0:                                       # [R, C] -> [R * per, C]
        return ((t.unsqueeze(1) >> shifts.view(1, per, 1)) & mask).reshape(t.shape[0] * per, t.shape[1])
    return ((t.unsqueeze(2) >> shifts.view(1, 1, per)) & mask).reshape(t.shape[0], t.shape[1] * per)


def _pack_int32(q: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    per = 32 // bits
    q = q.to(torch.int64)
    shifts = torch.arange(per, dtype=torch.int64, device=q.device) * bits
    if dim == 0:
        v = (q.view(q.shape[0] // per, per, q.shape[1]) << shifts.view(1, per, 1)).sum(1)
    else:
        v = (q.view(q.shape[0], q.shape[1] // per, per) << shifts.view(1, 1, per)).sum(2)
    v = torch.where(v >= 2 ** 31, v - 2 ** 32, v)      # two's complement int32
    return v.to(torch.int32)


def _unpack_bitstream(t: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    """Codes of a width that does not divide 32 (3-bit GPTQ): along `dim` every `bits` int32 hold 32 codes as one little-endian
    bit stream, code j at bit j * bits (a code may straddle two words)."""
    if dim == 1:
        return _unpack_bitstream(t.t().contiguous(), bits, 0).t().contiguous()
    R, C = t.shape
    assert R % bits == 0, "rows must come in groups of `bits` words"
    w = (t.to(torch.int64) & 0xFFFFFFFF).view(R // bits, bits, C)                     # unsigned words
    j = torch.arange(32, device=t.device)
    off = j * bits
    word, shift = off // 32, off % 32
    lo = w[:, word, :] >> shift.view(1, 32, 1)
    nxt = torch.where(word + 1 < bits, word + 1, word)
    hi = torch.where((shift + bits > 32).view(1, 32, 1), w[:, nxt, :] << (32 - shift).view(1, 32, 1), torch.zeros_like(lo))
    return (((lo | hi) & ((1 << bits) - 1)).to(torch.int32)).reshape(R // bits * 32, C)


def _pack_bitstream(q: torch.Tensor, bits: int, dim: int) -> torch.Tensor:
    """Inverse of `_unpack_bitstream` (what AutoGPTQ's `pack` writes for 3 bits)."""
    if dim == 1:
        return _pack_bitstream(q.t().contiguous(), bits, 0).t().contiguous()
    R, C = q.shape
    assert R % 32 == 0
    v = q.to(torch.int64).view(R // 32, 32, C)
    out = torch.zeros(R // 32, bits, C, dtype=torch.int64, device=q.device)
    for j in range(32):
        off = j * bits
        word, shift = off // 32, off % 32
        out[:, word] |= (v[:, j] << shift) & 0xFFFFFFFF
        if shift + bits > 32:
            out[:, word + 1] |= v[:, j] >> (32 - shift)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32).reshape(R // 32 * bits, C)


def gptq_unpack(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, bits: int, zero_offset: int = 1):
    """AutoGPTQ tensors (`qweight` int32 [K * bits / 32, N] packed along K, `qzeros` int32 [G, N * bits / 32] packed along N
    holding zero - 1, `scales` [G, N]) -> codes [N, K], scales [N, G], zeros [N, G].  `zero_offset=0` reads the v2 format,
    which stores the zero point itself."""
    if bits not in (2, 3, 4, 8):
        raise NotImplementedError(f"GPTQ with {bits} bits")
    if bits == 3:                                      # 32 codes in three words, straddling word boundaries
        q = _unpack_bitstream(qweight, 3, 0).t().contiguous()
        z = (_unpack_bitstream(qzeros, 3, 1) + zero_offset) & 7
        return q, scales.float().t().contiguous(), z[:, : scales.shape[1]].float().t().contiguous()
    q = _unpack_int32(qweight, bits, 0).t().contiguous()
    z = (_unpack_int32(qzeros, bits, 1) + zero_offset) & ((1 << bits) - 1)
    return q, scales.float().t().contiguous(), z[:, : scales.shape[1]].float().t().contiguous()


def gptq_pack(q: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, bits: int, group: int, zero_offset: int = 1):
    """Inverse of `gptq_unpack`: codes [N, K], scale / zero [N, G] -> dict of AutoGPTQ tensors (with the trivial `g_idx`)."""
    N, K = q.shape
    if bits == 3:
        zz = ((zero.t().to(torch.int64) - zero_offset) & 7).contiguous()
        pad = (-zz.shape[1]) % 32
        if pad:
            zz = torch.nn.functional.pad(zz, (0, pad))
        return {"qweight": _pack_bitstream(q.t().contiguous(), 3, 0), "qzeros": _pack_bitstream(zz, 3, 1),
                "scales": scale.t().contiguous().to(torch.float16), "g_idx": (torch.arange(K, dtype=torch.int32) // group)}
    return {"qweight": _pack_int32(q.t().contiguous(), bits, 0),
            "qzeros": _pack_int32(((zero.t().to(torch.int64) - zero_offset) & ((1 << bits) - 1)).contiguous(), bits, 1),
            "scales": scale.t().contiguous().to(torch.float16),
            "g_idx": (torch.arange(K, dtype=torch.int32) // group)}


def awq_unpack(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor):
    """AutoAWQ GEMM tensors (`qweight` int32 [K, N / 8], `qzeros` int32 [G, N / 8], both with nibble i holding column
    8 * c + AWQ_ORDER[i]; `scales` [G, N]) -> codes [N, K], scales [N, G], zeros [N, G]."""
    def cols(t):
        nib = _unpack_int32(t, 4, 1).view(t.shape[0], t.shape[1], 8)
        out = torch.empty_like(nib)
        for i, c in enumerate(AWQ_ORDER):
            out[..., c] = nib[..., i]
        return out.view(t.shape[0], t.shape[1] * 8)
    return cols(qweight).t().contiguous(), scales.float().t().contiguous(), cols(qzeros).float().t().contiguous()


def awq_pack(q: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor):
    def cols(t):                                       # [R, N] -> int32 [R, N / 8]
        w = t.to(torch.int64).view(t.shape[0], t.shape[1] // 8, 8)
        nib = torch.empty_like(w)
        for i, c in enumerate(AWQ_ORDER):
            nib[..., i] = w[..., c]
        return _pack_int32(nib.view(t.shape[0], t.shape[1]), 4, 1)
    return {"qweight": cols(q.t().contiguous()), "qzeros": cols(zero.t().contiguous()), "scales": scale.t().contiguous().to(torch.float16)}


def from_checkpoint(tensors: dict, quant_method: str, bits: int, group: int, zero_offset: int = 1, dtype=torch.float32,
                    want_dense: bool = True):
    """One linear layer of a GPTQ / AWQ checkpoint -> (GroupQuantWeight or None, dense [N, K] in `dtype`).

    The resident layout keeps one (scale, zero) per run of `group` inputs.  An act-order GPTQ layer (`g_idx` not monotone)
    is stored with its columns sorted by group, which makes the runs contiguous again, and carries the order in `perm`; only a
    layer whose groups are not all of `group` columns has the dense form alone."""
    if quant_method == "awq":
        q, s, z = awq_unpack(tensors["qweight"], tensors["qzeros"], tensors["scales"])
        g_idx = None
    else:
        q, s, z = gptq_unpack(tensors["qweight"], tensors["qzeros"], tensors["scales"], bits, zero_offset)
        g_idx = tensors.get("g_idx")
    if bits == 3:
        bits = 4                                       # 3-bit codes and zero points are exact in the 4-bit resident layout
    N, K = q.shape
    G = s.shape[1]
    grp = K // G if group <= 0 else group
    trivial = g_idx is None or bool(torch.equal(g_idx.to(torch.int64).cpu(), torch.arange(K) // grp))
    if trivial:
        packed = make_weight(q, s, z, bits, grp, method=quant_method)
        return packed, (dequantize(packed, dtype) if want_dense else None)
    gi = g_idx.to(torch.int64).cpu()
    perm = torch.argsort(gi, stable=True)
    if bool(torch.equal(gi[perm], torch.arange(K) // grp)):
        packed = make_weight(q[:, perm].contiguous(), s, z, bits, grp, method=quant_method)
        packed.perm = perm.to(torch.int32)
        return packed, (dequantize(packed, dtype) if want_dense else None)
    dense = (q.float() - z[:, gi]) * s[:, gi]
    return None, dense.to(dtype)


# ------------------------------------------------------------------------------------------------ GPTQ

def gptq_quantize(w: torch.Tensor, hessian: torch.Tensor, bits: int = 4, group: int = 128, damp: float = 0.01, block: int = 128):
    """GPTQ (Frantar et al.; `utils/gptq/quantize.py` in the reference): quantise the columns of W [N, K] one after the other
    and push each column's rounding error onto the columns not yet quantised through the inverse Hessian of the layer's
    inputs, H = sum x x^T [K, K].  Returns codes [N, K], scale [N, G], zero [N, G] on a min-max grid per group of `group`
    inputs (grids are fixed when the group is reached, after the updates from earlier columns)."""
    W = w.float().clone()
    N, K = W.shape
    H = hessian.float().clone()
    dead = torch.diag(H) == 0
    H[dead, dead] = 1
    W[:, dead] = 0
    H += torch.eye(K, device=H.device) * damp * torch.diag(H).mean()
    Hinv = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True)
    maxq = (1 << bits) - 1
    g = K if group <= 0 else group
    Q = torch.zeros(N, K, dtype=torch.int32, device=W.device)
    scale = torch.zeros(N, K // g, device=W.device)
    zero = torch.zeros(N, K // g, device=W.device)
    for i1 in range(0, K, block):
        i2 = min(i1 + block, K)
        W1 = W[:, i1:i2].clone()
        Err = torch.zeros_like(W1)
        Hinv1 = Hinv[i1:i2, i1:i2]
        for i in range(i2 - i1):
            k = i1 + i
            if k % g == 0:
                seg = W[:, k:k + g] if k + g > i2 else torch.cat([W1[:, i:], W[:, i2:k + g]], 1)[:, :g]
                lo, hi = seg.amin(1), seg.amax(1)
                sc = ((hi - lo) / maxq).clamp_min(1e-8).to(torch.float16).float()
                scale[:, k // g] = sc
                zero[:, k // g] = torch.round(-lo / sc)
            sc, zp = scale[:, k // g], zero[:, k // g]
            col = W1[:, i]
            qc = torch.clamp(torch.round(col / sc + zp), 0, maxq)
            Q[:, k] = qc.to(torch.int32)
            err = (col - (qc - zp) * sc) / Hinv1[i, i]
            W1[:, i:] -= err[:, None] * Hinv1[i, i:][None, :]
            Err[:, i] = err
        W[:, i1:i2] = W1
        W[:, i2:] -= Err @ Hinv[i1:i2, i2:]
    return Q, scale, zero
