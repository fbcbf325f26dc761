"""ctypes bindings for ``_lx_kernels.so`` (the sm_100a CUDA kernels).

The library exports a plain C ABI; tensors are passed as raw device pointers together with the current
CUDA stream, so a call is a direct kernel launch with no framework dispatch in between and is safe to
capture into a CUDA graph.  Loading fails loudly on a GPU machine when the library is missing: there is
no silent eager fallback.
"""

from __future__ import annotations

import ctypes
import dataclasses
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from pathlib import Path
from typing import NamedTuple, Optional

import torch

_PKG = Path(__file__).resolve().parent.parent
_LIB_PATH = _PKG / "_lx_kernels.so"
_lib: Optional[ctypes.CDLL] = None

# number of kernel launches issued through this module (bench.py reports it as `gpu_launches`)
launch_count = 0


class NativeError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        if os.environ.get("LORAX_B200_NO_BUILD") != "1":
            from lorax_b200.csrc import build as _build
            _build.build_kernels()
        if not _LIB_PATH.exists():
            raise NativeError(f"{_LIB_PATH} is missing; run `python -m lorax_b200.csrc.build`")
    lib = ctypes.CDLL(str(_LIB_PATH))
    P, I, L, F = c_void_p, c_int, c_longlong, c_float
    sigs = {
        "lx_gemm_ws_bytes": ([], L),
        "lx_gemm_max_tiles": ([], I),
        "lx_gemm_plan": ([I, I, I, I, L, I, I, P], I),
        "lx_gemm_bf16": ([P, P, P, P, I, I, I, L, L, L, F, P, L, P, P, I, I, I, P], I),
        "lx_norm_residual": ([P, P, P, P, P, I, I, L, L, L, F, F, F, I, P], I),
        "lx_rope_kvwrite": ([P, P, P, P, P, I, I, I, I, I, I, L, I, P], I),
        "lx_act_mul": ([P, P, I, I, L, L, I, I, P], I),
        "lx_embed": ([P, P, P, I, I, I, I, F, P], I),
        "lx_argmax_logprob": ([P, L, I, I, P, P, F, P], I),
        "lx_advance_decode": ([P, P, P, P, P, P, I, I, I, P], I),
        "lx_prefill_metadata": ([P, P, P, P, I, I, I, I, P, P, P, P], I),
        "lx_attn_page_size": ([], I),
        "lx_attn_decode": ([P, L, P, P, I, P, P, L, P, P, I, I, I, I, I, F, F, I, P], I),
        "lx_attn_prefill": ([P, L, P, P, I, P, P, P, P, I, P, L, I, I, I, I, F, F, P], I),
        "lx_attn_decode_alibi": ([P, L, P, P, I, P, P, L, P, P, I, I, I, I, I, F, F, I, P, P], I),
        "lx_attn_prefill_alibi": ([P, L, P, P, I, P, P, P, P, I, P, L, I, I, I, I, F, F, P, P], I),
        "lx_rope_kvwrite_kv8": ([P, P, P, P, P, I, I, I, I, I, I, L, I, I, F, F, P], I),
        "lx_attn_decode_kv8": ([P, L, P, P, I, P, P, L, P, P, I, I, I, I, I, F, F, I, P, F, F, P], I),
        "lx_attn_prefill_kv8": ([P, L, P, P, I, P, P, P, P, I, P, L, I, I, I, I, F, F, P, F, F, P], I),
        "lx_lora_shrink": ([P, L, P, P, P, P, I, L, I, P, I, I, I, I, P, P], I),
        "lx_lora_expand": ([P, I, P, P, P, P, I, L, P, L, I, I, I, I, P, P], I),
        "lx_tensormap_bytes": ([], I),
        "lx_lora_encode_tmap": ([P, P, I, I, L, I], I),
        "lx_lora_encode_tmap_b": ([P, P, I, I, L, I], I),
        "lx_lora_shrink_tc": ([P, L, P, I, I, P, I, I, P, I, I, I, P, I, L, I, P, P, I, I, I, I, P, P], I),
        "lx_gemm_bf16_lora": ([P, P, P, P, I, I, I, L, L, L, P, L, P, P, I, P, P], I),
        "lx_lora_fused_desc_bytes": ([], I),
        "lx_quant_act_fp8": ([P, L, P, L, P, I, I, I, P], I),
        "lx_gemm_fp8_block128": ([P, L, P, I, P, L, P, P, L, P, I, I, I, P, L, P, I, P], I),
        "lx_fp8_block128_dequant": ([P, L, P, I, P, L, I, I, P], I),
        "lx_wq_dequant": ([P, P, P, P, L, I, I, I, I, P], I),
        "lx_wq4_gemm": ([P, L, P, P, P, P, L, I, I, I, I, P], I),
        "lx_wq4_gemm_ex": ([P, L, P, P, P, P, L, I, I, I, I, I, P], I),
        "lx_lora_expand_tiled": ([P, I, L, I, P, I, I, P, P, P, I, L, P, L, I, I, I, I, P, P], I),
        "lx_attn_prefill_tc_supported": ([I, I, I, L, L], I),
        "lx_attn_prefill_tc": ([P, L, I, P, I, P, I, P, P, P, P, I, P, L, I, I, I, I, F, F, P, P, P], I),
        "lx_moe_router_logits": ([P, L, P, L, P, I, I, I, P], I),
        "lx_moe_route": ([P, I, I, I, I, I, P, P, P, P, P, P], I),
        "lx_moe_gather": ([P, L, P, P, I, P, L, I, I, P], I),
        "lx_moe_combine": ([P, L, P, P, I, P, L, I, I, P], I),
        "lx_moe_grouped_gemm": ([P, L, P, L, P, L, P, I, I, I, I, I, P, I, P], I),
    }
    for name, (argtypes, restype) in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    _lib = lib
    return lib


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str):
    global launch_count
    launch_count += 1
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")


STATUS_NAMES = {1: "TMA data never landed", 2: "smem stage never released", 3: "accumulator never completed",
                4: "accumulator never drained", 5: "peer flag timeout", 6: "split-K / LoRA image timeout", 7: "index out of range"}


class Workspace:
    """Device scratch shared by the kernels of one process: split-K partials and counters, split-KV partials,
    the status words written by bounded waits, and the LoRA intermediate."""

    LORA_KSPLIT = 8

    def __init__(self, device: torch.device, max_tokens: int = 16384, max_lora_cols: int = 3 * 64,
                 attn_splits: int = 8, num_heads: int = 64, head_dim: int = 128):
        lib = load()
        self.device = device
        self.gemm_ws = torch.empty(lib.lx_gemm_ws_bytes(), dtype=torch.uint8, device=device)
        self.gemm_counters = torch.zeros(lib.lx_gemm_max_tiles(), dtype=torch.int32, device=device)
        self.status = torch.zeros(2, dtype=torch.int32, device=device)
        # LoRA intermediate: [K-split][token][nparts * rank] fp32 partial sums (split 0 alone for the per-token kernels)
        self.lora_v3 = torch.zeros(self.LORA_KSPLIT, max_tokens, max_lora_cols, dtype=torch.float32, device=device)
        self.lora_v = torch.zeros(max_tokens, max_lora_cols, dtype=torch.float32, device=device)     # shrink result
        self.lora_counters = torch.zeros(16384, dtype=torch.int32, device=device)
        # LoRA expand inside the GEMM launch: bf16 operand images of the shrink results (6 KB per table entry and part)
        self.lora_max_entries = 1024
        self.lora_vimg = torch.zeros(self.lora_max_entries * 3 * 48 * 64, dtype=torch.bfloat16, device=device)
        self.lora_sync = torch.zeros(2, dtype=torch.int32, device=device)       # launch-wide counters of the in-kernel shrink
        self.fp8_scratch = None              # bf16 image of one fp8 projection (long prefills), allocated on first use
        self.attn_part_tokens = 256
        self.attn_splits = attn_splits
        self.attn_part_o = torch.empty(self.attn_part_tokens * num_heads * attn_splits * head_dim, dtype=torch.float32, device=device)
        self.attn_part_lse = torch.empty(self.attn_part_tokens * num_heads * attn_splits, dtype=torch.float32, device=device)
        self.num_sms = torch.cuda.get_device_properties(device).multi_processor_count

    def check_status(self):
        """Raise if a bounded device-side wait ran out since the last check (one D2H of 8 bytes)."""
        st = self.status.tolist()
        if st[0] != 0:
            self.status.zero_()
            raise NativeError(f"device status {st[0]} ({STATUS_NAMES.get(st[0], '?')}), detail {st[1]}")


_workspaces = {}


def workspace(device=None) -> Workspace:
    device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    ws = _workspaces.get(device)
    if ws is None:
        ws = _workspaces[device] = Workspace(device)
    return ws


# ------------------------------------------------------------------------------------------------ GEMM
def gemm_plan(T: int, N: int, K: int, num_sms: int = 148, ws_bytes: int = 64 << 20, force_split: int = 0, sk_policy: int = 0) -> dict:
    """Tiling the weights-on-M GEMM path would choose for a shape (no GPU needed)."""
    out = (ctypes.c_int * 5)()
    load().lx_gemm_plan(T, N, K, num_sms, ws_bytes, force_split, sk_policy, out)
    return dict(zip(("bn", "split", "dp_tiles", "sk_ctas", "grid"), out))


class LoraEpilogue(NamedTuple):
    """Result of a stand-alone shrink, as the stand-alone expand kernels take it: v and where each slot's B_cat of the
    projection group sits in the arena."""
    v: torch.Tensor            # [T, ldv] fp32
    tok_slot: torch.Tensor     # [T] int32, -1 = no adapter
    arena: torch.Tensor
    slot_base: torch.Tensor
    slot_rank: torch.Tensor
    unit_off: int
    n0: int
    n1: int


# 1 (default): the GEMM that carries LoRA acquire-fences a slot's B_cat tensor map before every use, as a tensor map that lives
# in global memory and was written by a copy asks for; 0 skips it (measurement: the fences cost about 3 % of a decode step).
LORA_FENCE_MAPS = int(os.environ.get("LORAX_LORA_FENCE_MAPS", "1"))
TC_PREFILL = os.environ.get("LORAX_TC_PREFILL", "1") != "0"       # 0: the mma.sync prefill attention kernel for every shape
# rows from which an fp8 projection is expanded to bf16 in front of the bf16 GEMM instead of running on the fp8 tensor-core kernel
FP8_EXPAND_MIN_TOKENS = int(os.environ.get("LORAX_FP8_EXPAND_MIN_TOKENS", "512"))


class LxLoraFused(ctypes.Structure):
    """Mirror of the C struct of the same name (csrc/kernels/gemm_bf16.cu)."""
    _fields_ = [("tiles", ctypes.c_void_p), ("num_tiles", ctypes.c_int),
                ("slot_tmaps", ctypes.c_void_p), ("maps_per_slot", ctypes.c_int), ("map_a", ctypes.c_int), ("map_b", ctypes.c_int),
                ("slot_rank", ctypes.c_void_p), ("slot_base", ctypes.c_void_p), ("num_slots", ctypes.c_int),
                ("nparts", ctypes.c_int), ("n0", ctypes.c_int), ("n1", ctypes.c_int), ("layer", ctypes.c_int),
                ("max_rank", ctypes.c_int),
                ("vimg", ctypes.c_void_p), ("vimg_bytes", ctypes.c_longlong),
                ("fence_maps", ctypes.c_int),
                ("arena", ctypes.c_void_p), ("off_a", ctypes.c_longlong),
                ("off_b", ctypes.c_longlong), ("arena_elems", ctypes.c_longlong), ("sync", ctypes.c_void_p)]


class LoraFused(NamedTuple):
    """The multi-adapter LoRA of one projection group for the GEMM that carries it in its own launch."""
    tiles: torch.Tensor        # [n, 4] int32 (slot, first row, rows <= 32, -), live entries first
    num_tiles: int
    live: int                  # live entries (0: all of them); sizes the K split of the shrink items
    slot_tmaps: torch.Tensor
    maps_per_slot: int
    map_a: int
    map_b: int
    slot_rank: torch.Tensor
    slot_base: torch.Tensor
    nparts: int
    n0: int
    n1: int
    layer: int
    max_rank: int
    arena: Optional[torch.Tensor] = None      # the slots' blobs; A_cat of the group and layer at slot_base + rank * off_a (elements)
    off_a: int = 0
    off_b: int = 0                            # B_cat likewise


def lora_fused_desc(ws: "Workspace", lf: LoraFused, K: int) -> LxLoraFused:
    d = LxLoraFused()
    d.tiles, d.num_tiles = lf.tiles.data_ptr(), lf.num_tiles
    d.slot_tmaps, d.maps_per_slot, d.map_a, d.map_b = lf.slot_tmaps.data_ptr(), lf.maps_per_slot, lf.map_a, lf.map_b
    d.slot_rank, d.slot_base, d.num_slots = lf.slot_rank.data_ptr(), lf.slot_base.data_ptr(), lf.slot_rank.shape[0]
    d.nparts, d.n0, d.n1, d.layer, d.max_rank = lf.nparts, lf.n0, lf.n1, lf.layer, lf.max_rank
    d.vimg, d.vimg_bytes = ws.lora_vimg.data_ptr(), ws.lora_vimg.numel() * 2
    d.arena, d.off_a = (lf.arena.data_ptr() if lf.arena is not None else None), lf.off_a
    d.off_b, d.arena_elems = lf.off_b, (lf.arena.numel() if lf.arena is not None else 0)
    d.sync = ws.lora_sync.data_ptr()
    d.fence_maps = LORA_FENCE_MAPS
    return d


def gemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
         out_scale: float = 1.0, mode: int = 0, force_split: int = 0) -> torch.Tensor:
    """out[T, N] = x[T, K] @ w[N, K]^T (+ bias).  bf16 in, fp32 accumulate on tcgen05, bf16 out."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
    assert x.stride(1) == 1 and w.stride(1) == 1
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    assert out.stride(1) == 1
    ws = workspace(x.device)
    lib = load()
    rc = lib.lx_gemm_bf16(_ptr(x), _ptr(w), _ptr(out), _ptr(bias), T, N, K, x.stride(0), w.stride(0), out.stride(0),
                          out_scale, _ptr(ws.gemm_ws), ws.gemm_ws.numel(), _ptr(ws.gemm_counters), _ptr(ws.status),
                          ws.num_sms, mode, force_split, _stream())
    _check(rc, "lx_gemm_bf16")
    return out


def gemm_lora_fused(x: torch.Tensor, w: torch.Tensor, lf: LoraFused, bias: Optional[torch.Tensor] = None,
                    out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """out[T, N] = x @ w^T (+ bias) + the LoRA delta of every row's adapter in one launch of
    `gemm_bf16_tcgen05_kernel<.., true>`: its epilogue warps compute the shrink while the first K loop runs, the expand is
    added by UMMAs after the K loop of every base tile.  None when the step cannot be served this way (rank above 64, part
    boundaries off the 128 grid, table larger than the scratch): the caller then uses the separate kernels."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    T, K = x.shape
    N = w.shape[0]
    given = out
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    ws = workspace(x.device)
    lib = load()
    if lib.lx_lora_fused_desc_bytes() != ctypes.sizeof(LxLoraFused):
        raise NativeError("LxLoraFused: C++ and ctypes disagree")
    d = lora_fused_desc(ws, lf, K)
    rc = lib.lx_gemm_bf16_lora(_ptr(x), _ptr(w), _ptr(out), _ptr(bias), T, N, K, x.stride(0), w.stride(0), out.stride(0),
                               _ptr(ws.gemm_ws), ws.gemm_ws.numel(), _ptr(ws.gemm_counters), _ptr(ws.status), ws.num_sms,
                               ctypes.byref(d), _stream())
    if rc == 1:
        return None
    _check(rc, "lx_gemm_bf16_lora")
    return out if given is None else given


# ------------------------------------------------------------------------------------------------ mixture of experts
class MoeRouting(NamedTuple):
    topk_ids: torch.Tensor     # [T, k] int32
    topk_w: torch.Tensor       # [T, k] fp32, renormalised over the kept experts
    seg: torch.Tensor          # [e_local + 1] int32: rows of every local expert in the sorted order
    pos: torch.Tensor          # [T, k] int32: sorted row of (token, choice), -1 when the expert lives on another rank
    sorted_tok: torch.Tensor   # [T * k] int32


def moe_route(x: torch.Tensor, router_w: torch.Tensor, k: int, e0: int, e_local: int) -> MoeRouting:
    """Router logits (fp32), softmax over all experts, top-k, renormalise, and the sorted order of the rows routed to the
    experts [e0, e0 + e_local) this rank owns: two launches, everything stays on the device."""
    T, H = x.shape
    E = router_w.shape[0]
    dev = x.device
    logits = torch.empty(T, E, dtype=torch.float32, device=dev)
    lib = load()
    _check(lib.lx_moe_router_logits(_ptr(x), x.stride(0), _ptr(router_w), router_w.stride(0), _ptr(logits), T, E, H, _stream()), "lx_moe_router_logits")
    r = MoeRouting(torch.empty(T, k, dtype=torch.int32, device=dev), torch.empty(T, k, dtype=torch.float32, device=dev),
                   torch.empty(e_local + 1, dtype=torch.int32, device=dev), torch.empty(T, k, dtype=torch.int32, device=dev),
                   torch.empty(T * k, dtype=torch.int32, device=dev))
    _check(lib.lx_moe_route(_ptr(logits), T, E, k, e0, e_local, _ptr(r.topk_ids), _ptr(r.topk_w), _ptr(r.seg), _ptr(r.pos), _ptr(r.sorted_tok),
                            _stream()), "lx_moe_route")
    return r


def moe_grouped_gemm(xg: torch.Tensor, w: torch.Tensor, seg: torch.Tensor, avg_rows: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[q] = xg[q] @ w[e(q)]^T for every sorted row q (e(q): the expert whose run [seg[e], seg[e+1]) holds q).
    w: [e_local, n_w, K] bf16, n_w a multiple of 128."""
    e_local, n_w, K = w.shape
    rows = xg.shape[0]
    assert w.is_contiguous() and xg.stride(1) == 1 and xg.shape[1] == K
    if out is None:
        out = torch.empty(rows, n_w, dtype=torch.bfloat16, device=xg.device)
    ws = workspace(xg.device)
    rc = load().lx_moe_grouped_gemm(_ptr(xg), xg.stride(0), _ptr(w), K, _ptr(out), out.stride(0), _ptr(seg), e_local, rows, n_w, K, avg_rows,
                                    _ptr(ws.status), ws.num_sms, _stream())
    _check(rc, "lx_moe_grouped_gemm")
    return out


def moe_ffn(x: torch.Tensor, router_w: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, k: int, e0: int, act: str = "silu") -> torch.Tensor:
    """Top-k mixture-of-experts feed-forward of this rank's experts: route, gather, grouped w1|w3 GEMM, act * up, grouped w2
    GEMM, weighted combine.  w13: [e_local, 2I, H], w2: [e_local, H, I].  Returns [T, H] (a partial sum under expert parallelism)."""
    T, H = x.shape
    e_local, two_i, _ = w13.shape
    E = router_w.shape[0]
    r = moe_route(x, router_w, k, e0, e_local)
    rows = T * k
    lib = load()
    xg = torch.empty(rows, H, dtype=torch.bfloat16, device=x.device)
    _check(lib.lx_moe_gather(_ptr(x), x.stride(0), _ptr(r.sorted_tok), _ptr(r.seg), e_local, _ptr(xg), xg.stride(0), rows, H, _stream()), "lx_moe_gather")
    avg = max(1, (rows + E - 1) // E)
    gu = moe_grouped_gemm(xg, w13, r.seg, avg)
    a = act_mul(gu, two_i // 2, act, gated=True)
    y = moe_grouped_gemm(a, w2, r.seg, avg)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    _check(lib.lx_moe_combine(_ptr(y), y.stride(0), _ptr(r.pos), _ptr(r.topk_w), k, _ptr(out), out.stride(0), T, H, _stream()), "lx_moe_combine")
    return out


def quant_act_fp8(x: torch.Tensor):
    """x [T, K] bf16 -> (xq [T, K] uint8 holding e4m3, sa [K/128, T16] fp32): one scale per token and 128-wide K block."""
    T, K = x.shape
    xq = torch.empty(T, K, dtype=torch.uint8, device=x.device)
    sa = torch.empty((K + 127) // 128, (T + 15) // 16 * 16, dtype=torch.float32, device=x.device)
    rc = load().lx_quant_act_fp8(_ptr(x), x.stride(0), _ptr(xq), xq.stride(0), _ptr(sa), sa.stride(0), T, K, _stream())
    _check(rc, "lx_quant_act_fp8")
    return xq, sa


def fp8_expand(wq: torch.Tensor, w_scale: torch.Tensor) -> Optional[torch.Tensor]:
    """Block-scaled e4m3 weights [N, K] -> bf16 [N, K] in the workspace's scratch buffer (valid until the next call; consumers are
    queued on the same stream).  None when the layout does not fit the kernel (K or the row pitch not a multiple of 16)."""
    N, K = wq.shape
    if K % 16 != 0 or wq.stride(0) % 16 != 0:
        return None
    ws = workspace(wq.device)
    need = N * K
    if ws.fp8_scratch is None or ws.fp8_scratch.numel() < need:
        ws.fp8_scratch = torch.empty(need, dtype=torch.bfloat16, device=wq.device)
    w16 = ws.fp8_scratch[:need].view(N, K)
    _check(load().lx_fp8_block128_dequant(_ptr(wq), wq.stride(0), _ptr(w_scale), w_scale.stride(0), _ptr(w16), K, N, K, _stream()),
           "lx_fp8_block128_dequant")
    return w16


def gemm_fp8(x: torch.Tensor, wq: torch.Tensor, w_scale: torch.Tensor, bias: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[T, N] = x[T, K] @ dequant(wq[N, K], w_scale[N/128, K/128])^T (+ bias): activations are quantised to e4m3 per
    token and 128-wide K block on the fly, the product runs on the fp8 tensor cores, bf16 out."""
    assert x.dtype == torch.bfloat16 and wq.dtype in (torch.uint8, torch.float8_e4m3fn) and w_scale.dtype == torch.float32
    T, K = x.shape
    N = wq.shape[0]
    assert wq.shape[1] == K and w_scale.shape == ((N + 127) // 128, (K + 127) // 128) and w_scale.is_contiguous()
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    ws = workspace(x.device)
    if T >= FP8_EXPAND_MIN_TOKENS:
        # long prefills: expand this projection's weights to bf16 (one pass, a few per cent of the GEMM) and run the bf16 GEMM; the
        # fp8 tensor-core kernel below is bound by the per-128 promotion of its partial sums at this size
        w16 = fp8_expand(wq, w_scale)
        if w16 is not None:
            return gemm(x, w16, bias=bias, out=out)
    xq, sa = quant_act_fp8(x)
    rc = load().lx_gemm_fp8_block128(_ptr(xq), xq.stride(0), _ptr(sa), sa.stride(0), _ptr(wq), wq.stride(0), _ptr(w_scale), _ptr(out),
                                     out.stride(0), _ptr(bias), T, N, K, _ptr(ws.gemm_ws), ws.gemm_ws.numel(), _ptr(ws.status),
                                     ws.num_sms, _stream())
    _check(rc, "lx_gemm_fp8_block128")
    return out


def wq_dequant(w, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Packed group-quantised weight (`utils.quant_formats.GroupQuantWeight`) -> bf16 [N, K]."""
    N, K = w.shape
    if out is None:
        out = torch.empty(N, K, dtype=torch.bfloat16, device=w.codes.device)
    rc = load().lx_wq_dequant(_ptr(w.codes), _ptr(w.sz), _ptr(w.table), _ptr(out), out.stride(0), N, K, w.bits, w.group, _stream())
    _check(rc, "lx_wq_dequant")
    if getattr(w, "perm", None) is not None:          # act-order GPTQ: stored column i is input feature perm[i]
        out.copy_(torch.empty_like(out).index_copy_(1, w.perm.long(), out))
    return out


WQ4_DIRECT_MAX_TOKENS = int(os.environ.get("LORAX_WQ4_DIRECT_TOKENS", "32"))


def gemm_wq(x: torch.Tensor, w, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[T, N] = x[T, K] @ dequant(w)^T (+ bias) for a weight-only quantised matrix.  Few tokens and affine 4-bit codes:
    the tensor-core kernel that multiplies straight from the packed codes (HBM traffic = the packed weights).  Otherwise
    the codes are expanded to bf16 once and the tcgen05 GEMM runs on the expansion."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    if getattr(w, "perm", None) is not None:
        # act-order GPTQ: the stored columns are sorted by group, so the activations are gathered into that order first
        # (2 * T * K bytes against N * K / 2 of weights) and both kernels below see an ordinary grouped matrix
        x = x.index_select(1, w.perm)
        w = dataclasses.replace(w, perm=None)
    if (w.bits == 4 and w.table is None and T <= WQ4_DIRECT_MAX_TOKENS and N % 16 == 0 and K % 128 == 0 and w.group % 32 == 0
            and x.stride(0) % 8 == 0):
        rc = load().lx_wq4_gemm_ex(_ptr(x), x.stride(0), _ptr(w.codes), _ptr(w.sz), _ptr(bias), _ptr(out), out.stride(0), T, N, K, w.group,
                                   1 if getattr(w, "int_zero", False) else 0, _stream())
        _check(rc, "lx_wq4_gemm")
        return out
    return gemm(x, wq_dequant(w), bias=bias, out=out)


# ------------------------------------------------------------------------------------------------ elementwise
def norm_residual(x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                  bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, weight_offset: float = 0.0,
                  x_scale: float = 1.0, layernorm: bool = False) -> torch.Tensor:
    """h = x * x_scale (+ residual); residual <- h (in place); returns norm(h) * (weight + offset) (+ bias)."""
    T, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    rc = load().lx_norm_residual(_ptr(x), _ptr(residual), _ptr(weight), _ptr(bias), _ptr(out), T, H, x.stride(0),
                                 residual.stride(0) if residual is not None else 0, out.stride(0), eps, weight_offset,
                                 x_scale, int(layernorm), _stream())
    _check(rc, "lx_norm_residual")
    return out


def rope_kvwrite(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor, kv_cache: torch.Tensor,
                 slots: Optional[torch.Tensor], nh: int, nkv: int, d: int, rot: int, apply_rope: bool = True,
                 kv_scale: Optional[Tuple[float, float]] = None):
    """RoPE in place on q and k, then k and v into the paged cache.  A `torch.float8_e4m3fn` cache takes value / scale as e4m3
    (`kv_scale` = (k scale, v scale), default 1)."""
    T = qkv.shape[0]
    page = kv_cache.shape[3]
    fp8 = kv_cache.dtype == torch.float8_e4m3fn
    ks, vs = kv_scale if (fp8 and kv_scale) else (1.0, 1.0)
    rc = load().lx_rope_kvwrite_kv8(_ptr(qkv), _ptr(positions), _ptr(cos_sin), _ptr(kv_cache), _ptr(slots), T, nh, nkv, d, rot,
                                    page, qkv.stride(0), int(apply_rope), int(fp8), ks, vs, _stream())
    _check(rc, "lx_rope_kvwrite")


_ACTS = {"silu": 0, "swish": 0, "gelu": 1, "gelu_new": 2, "gelu_pytorch_tanh": 2, "gelu_fast": 2, "gelu_tanh": 2, "relu": 3}


def act_mul(x: torch.Tensor, inter: int, act: str = "silu", gated: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    T = x.shape[0]
    if out is None:
        out = torch.empty(T, inter, dtype=x.dtype, device=x.device)
    rc = load().lx_act_mul(_ptr(x), _ptr(out), T, inter, x.stride(0), out.stride(0), _ACTS[act], int(gated), _stream())
    _check(rc, "lx_act_mul")
    return out


def embed(ids: torch.Tensor, table: torch.Tensor, v0: int = 0, v1: Optional[int] = None, mult: float = 1.0,
          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    T = ids.shape[0]
    H = table.shape[1]
    if v1 is None:
        v1 = v0 + table.shape[0]
    if out is None:
        out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    rc = load().lx_embed(_ptr(ids), _ptr(table), _ptr(out), T, H, v0, v1, mult, _stream())
    _check(rc, "lx_embed")
    return out


def argmax_logprob(logits: torch.Tensor, ids: Optional[torch.Tensor] = None, logprobs: Optional[torch.Tensor] = None,
                   softcap: float = 0.0):
    T, V = logits.shape
    if ids is None:
        ids = torch.empty(T, dtype=torch.int32, device=logits.device)
    if logprobs is None:
        logprobs = torch.empty(T, dtype=torch.float32, device=logits.device)
    rc = load().lx_argmax_logprob(_ptr(logits), logits.stride(0), T, V, _ptr(ids), _ptr(logprobs), softcap, _stream())
    _check(rc, "lx_argmax_logprob")
    return ids, logprobs


def advance_decode(input_ids, next_ids, positions, ctx_lens, slots, block_tables, page: int):
    B = input_ids.shape[0]
    rc = load().lx_advance_decode(_ptr(input_ids), _ptr(next_ids), _ptr(positions), _ptr(ctx_lens), _ptr(slots),
                                  _ptr(block_tables), block_tables.shape[1], page, B, _stream())
    _check(rc, "lx_advance_decode")


def prefill_metadata(cu_q: torch.Tensor, cache_lens: torch.Tensor, seq_slot: torch.Tensor, block_tables: torch.Tensor, page: int, T: int):
    """Per-token (positions, slots, adapter slot) of a ragged prefill from its per-sequence description, on the device."""
    dev = cu_q.device
    out = torch.empty(3, T, dtype=torch.int32, device=dev)
    rc = load().lx_prefill_metadata(_ptr(cu_q), _ptr(cache_lens), _ptr(seq_slot), _ptr(block_tables), block_tables.shape[1], cache_lens.shape[0],
                                    page, T, _ptr(out[0]), _ptr(out[1]), _ptr(out[2]), _stream())
    _check(rc, "lx_prefill_metadata")
    return out[0], out[1], out[2]


# ------------------------------------------------------------------------------------------------ attention
def attn_decode(q: torch.Tensor, kv_cache: torch.Tensor, block_tables: torch.Tensor, ctx_lens: torch.Tensor, nh: int, nkv: int,
                d: int, scale: float, window: int = 0, softcap: float = 0.0, nsplit: int = 1,
                out: Optional[torch.Tensor] = None, alibi: Optional[torch.Tensor] = None,
                kv_scale: Optional[Tuple[float, float]] = None) -> torch.Tensor:
    """q: [T, >= nh*d] (row stride arbitrary), one query token per row.  Returns [T, nh*d].  `alibi`: [nh] fp32 slopes.
    An e4m3 cache is read as stored value * scale (`kv_scale` = (k scale, v scale))."""
    T = q.shape[0]
    if out is None:
        out = torch.empty(T, nh * d, dtype=q.dtype, device=q.device)
    ws = workspace(q.device)
    if nsplit > 1:
        nsplit = min(nsplit, ws.attn_splits)
        if T > ws.attn_part_tokens:
            nsplit = 1
    if kv_cache.dtype == torch.float8_e4m3fn:
        ks, vs = kv_scale or (1.0, 1.0)
        rc = load().lx_attn_decode_kv8(_ptr(q), q.stride(0), _ptr(kv_cache), _ptr(block_tables), block_tables.shape[1], _ptr(ctx_lens),
                                       _ptr(out), out.stride(0), _ptr(ws.attn_part_o), _ptr(ws.attn_part_lse), T, nh, nkv, d, window,
                                       scale, softcap, nsplit, _ptr(alibi), ks, vs, _stream())
        _check(rc, "lx_attn_decode_kv8")
        return out
    rc = load().lx_attn_decode_alibi(_ptr(q), q.stride(0), _ptr(kv_cache), _ptr(block_tables), block_tables.shape[1], _ptr(ctx_lens),
                                     _ptr(out), out.stride(0), _ptr(ws.attn_part_o), _ptr(ws.attn_part_lse), T, nh, nkv, d, window,
                                     scale, softcap, nsplit, _ptr(alibi), _stream())
    _check(rc, "lx_attn_decode")
    return out


def attn_prefill(q: torch.Tensor, kv_cache: torch.Tensor, block_tables: torch.Tensor, cu_q: torch.Tensor, cache_lens: torch.Tensor,
                 tile_seq: torch.Tensor, tile_q0: torch.Tensor, nh: int, nkv: int, d: int, scale: float, window: int = 0,
                 softcap: float = 0.0, out: Optional[torch.Tensor] = None, alibi: Optional[torch.Tensor] = None,
                 kv_scale: Optional[Tuple[float, float]] = None) -> torch.Tensor:
    T = q.shape[0]
    if out is None:
        out = torch.empty(T, nh * d, dtype=q.dtype, device=q.device)
    lib = load()
    if kv_cache.dtype == torch.float8_e4m3fn:
        # e4m3 pages are expanded to bf16 in shared memory by the mma.sync kernel (the tcgen05 kernel reads bf16 pages by TMA)
        ks, vs = kv_scale or (1.0, 1.0)
        rc = lib.lx_attn_prefill_kv8(_ptr(q), q.stride(0), _ptr(kv_cache), _ptr(block_tables), block_tables.shape[1], _ptr(cu_q),
                                     _ptr(cache_lens), _ptr(tile_seq), _ptr(tile_q0), tile_seq.shape[0], _ptr(out), out.stride(0), nh,
                                     nkv, d, window, scale, softcap, _ptr(alibi), ks, vs, _stream())
        _check(rc, "lx_attn_prefill_kv8")
        return out
    if TC_PREFILL and q.dtype == torch.bfloat16 and lib.lx_attn_prefill_tc_supported(nh, nkv, d, q.stride(0), out.stride(0)):
        # tcgen05 flash kernel: two query heads of a KV group per CTA, K / V pages by TMA from the paged cache
        rc = lib.lx_attn_prefill_tc(_ptr(q), q.stride(0), T, _ptr(kv_cache), kv_cache.shape[0], _ptr(block_tables), block_tables.shape[1],
                                    _ptr(cu_q), _ptr(cache_lens), _ptr(tile_seq), _ptr(tile_q0), tile_seq.shape[0], _ptr(out), out.stride(0),
                                    nh, nkv, d, window, scale, softcap, _ptr(alibi), _ptr(workspace(q.device).status), _stream())
        _check(rc, "lx_attn_prefill_tc")
        return out
    rc = lib.lx_attn_prefill_alibi(_ptr(q), q.stride(0), _ptr(kv_cache), _ptr(block_tables), block_tables.shape[1], _ptr(cu_q),
                                      _ptr(cache_lens), _ptr(tile_seq), _ptr(tile_q0), tile_seq.shape[0], _ptr(out), out.stride(0), nh,
                                      nkv, d, window, scale, softcap, _ptr(alibi), _stream())
    _check(rc, "lx_attn_prefill")
    return out


# ------------------------------------------------------------------------------------------------ LoRA
def lora_shrink(x: torch.Tensor, tok_slot: torch.Tensor, arena: torch.Tensor, slot_base: torch.Tensor, slot_rank: torch.Tensor,
                unit_off: int, nparts: int, max_rank: int, v: Optional[torch.Tensor] = None) -> torch.Tensor:
    T, K = x.shape
    ws = workspace(x.device)
    if v is None:
        v = ws.lora_v
    rc = load().lx_lora_shrink(_ptr(x), x.stride(0), _ptr(tok_slot), _ptr(arena), _ptr(slot_base), _ptr(slot_rank),
                               slot_rank.shape[0], unit_off, nparts, _ptr(v), v.stride(0), T, K, max_rank, _ptr(ws.status), _stream())
    _check(rc, "lx_lora_shrink")
    return v


def lora_expand(v: torch.Tensor, tok_slot: torch.Tensor, arena: torch.Tensor, slot_base: torch.Tensor, slot_rank: torch.Tensor,
                unit_off: int, y: torch.Tensor, n0: int, n1: int):
    T, N = y.shape
    ws = workspace(y.device)
    rc = load().lx_lora_expand(_ptr(v), v.stride(0), _ptr(tok_slot), _ptr(arena), _ptr(slot_base), _ptr(slot_rank),
                               slot_rank.shape[0], unit_off, _ptr(y), y.stride(0), T, N, n0, n1, _ptr(ws.status), _stream())
    _check(rc, "lx_lora_expand")


def lora_encode_tmap(out_host: torch.Tensor, base_ptr: int, K: int, R: int, layer_stride: int, layers: int):
    """Encode the 3-D tensor map {K, R, layers} of one adapter's A_cat family into 128 bytes of host memory."""
    rc = load().lx_lora_encode_tmap(out_host.data_ptr(), base_ptr, K, R, layer_stride, layers)
    if rc != 0:
        raise NativeError(f"lx_lora_encode_tmap failed with code {rc}")


def lora_encode_tmap_b(out_host: torch.Tensor, base_ptr: int, r: int, N: int, layer_stride: int, layers: int):
    """Encode the 3-D tensor map {r, N, layers} of one adapter's B_cat family (boxes of 16 ranks x 128 features, 32-byte
    swizzle: the operand slices of the GEMM that adds the LoRA delta itself) into 128 bytes of host memory."""
    rc = load().lx_lora_encode_tmap_b(out_host.data_ptr(), base_ptr, r, N, layer_stride, layers)
    if rc != 0:
        raise NativeError(f"lx_lora_encode_tmap_b failed with code {rc}")


def lora_shrink_tiles(x: torch.Tensor, tiles: torch.Tensor, num_tiles: int, max_tile_rows: int, slot_tmaps: torch.Tensor,
                      groups_per_slot: int, group: int, slot_rank: torch.Tensor, nparts: int, layer: int, max_rank: int,
                      v: Optional[torch.Tensor] = None, ksplit: Optional[int] = None, live_tiles: int = 0):
    """Tensor-core shrink over a tile table -> v [rows, cols] fp32.  K is split over CTAs when the table alone
    cannot fill the GPU; the last split CTA of a tile adds the partial sums in a fixed order."""
    T, K = x.shape
    ws = workspace(x.device)
    vf = ws.lora_v if v is None else v
    v3 = ws.lora_v3
    assert vf.stride(0) == v3.stride(1)
    kblocks = (K + 63) // 64
    chunks = (nparts * max_rank + 127) // 128
    # K split: these skinny tiles are latency bound, so K is cut over as many CTAs as the GPU holds at once (two per SM)
    # and no more: a second, partly filled wave doubles the time.  `live_tiles` is the number of entries that are not
    # padding (CTAs of dead entries exit at once).
    if ksplit is None:
        ksplit = max(1, (2 * ws.num_sms) // max(1, (live_tiles or num_tiles) * chunks))
    ksplit = max(1, min(v3.shape[0], kblocks // 8 if kblocks >= 8 else 1, ksplit))
    rc = load().lx_lora_shrink_tc(_ptr(x), x.stride(0), _ptr(tiles), num_tiles, max_tile_rows, _ptr(slot_tmaps), groups_per_slot, group,
                                  _ptr(slot_rank), slot_rank.shape[0], nparts, layer, _ptr(v3), v3.stride(1), v3.stride(0), ksplit,
                                  _ptr(vf), _ptr(ws.lora_counters), ws.lora_counters.numel(), T, K, max_rank, _ptr(ws.status), _stream())
    _check(rc, "lx_lora_shrink_tc")
    return vf


def lora_expand_tiles(v, tiles: torch.Tensor, num_tiles: int, max_tile_rows: int, arena: torch.Tensor, slot_base: torch.Tensor,
                      slot_rank: torch.Tensor, unit_off: int, y: torch.Tensor, n0: int, n1: int):
    v3, ksplit = v.unsqueeze(0), 1
    T, N = y.shape
    ws = workspace(y.device)
    rc = load().lx_lora_expand_tiled(_ptr(v3), v3.stride(1), v3.stride(0), ksplit, _ptr(tiles), num_tiles, max_tile_rows, _ptr(arena),
                                     _ptr(slot_base), _ptr(slot_rank), slot_rank.shape[0], unit_off, _ptr(y), y.stride(0), T, N, n0, n1,
                                     _ptr(ws.status), _stream())
    _check(rc, "lx_lora_expand_tiled")

# ------------------------------------------------------------------------------------------------ per-op timing
_TIMED_OPS = ("gemm", "gemm_fp8", "norm_residual", "rope_kvwrite", "act_mul", "embed", "argmax_logprob", "advance_decode", "attn_decode",
              "attn_prefill", "lora_shrink", "lora_expand", "lora_shrink_tiles", "lora_expand_tiles")
_timing_records = None
_timing_originals = {}


def enable_timing():
    """Bracket every operator call with CUDA events (eager mode only; do not use while capturing a graph).
    `timing_report()` returns the accumulated device time per (operator, shape)."""
    global _timing_records
    if _timing_records is not None:
        return
    _timing_records = []
    g = globals()

    def wrap(name, fn):
        def timed(*a, **kw):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = fn(*a, **kw)
            e.record()
            shapes = tuple(tuple(x.shape) for x in a[:2] if isinstance(x, torch.Tensor))
            _timing_records.append((name, shapes, s, e))
            return out
        return timed

    for name in _TIMED_OPS:
        _timing_originals[name] = g[name]
        g[name] = wrap(name, g[name])


def disable_timing():
    global _timing_records
    g = globals()
    for name, fn in _timing_originals.items():
        g[name] = fn
    _timing_originals.clear()
    _timing_records = None


def timing_report(reset: bool = True):
    """-> list of dicts sorted by total time: op, shapes, calls, total_ms, mean_us."""
    global _timing_records
    if _timing_records is None:
        return []
    torch.cuda.synchronize()
    agg = {}
    for name, shapes, s, e in _timing_records:
        k = (name, shapes)
        t = s.elapsed_time(e)
        c = agg.setdefault(k, [0, 0.0])
        c[0] += 1
        c[1] += t
    if reset:
        _timing_records = []
    rows = [dict(op=k[0], shapes=str(k[1]), calls=v[0], total_ms=round(v[1], 4), mean_us=round(1e3 * v[1] / v[0], 2)) for k, v in agg.items()]
    rows.sort(key=lambda r: -r["total_ms"])
    return rows
