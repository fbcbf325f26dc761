"""Python side of the native layer executor (`csrc/kernels/layer_exec.cu`).

`NativeExecutor.build(model)` describes the model to the C++ side once (weights, adapter layout, scratch buffers);
`run_layers` then walks the decoder layers with two native calls per layer, one for the attention half and one for the
MLP half, with the tensor-parallel all-reduce in between left to the caller's process group.  It serves the eager
steps (prefill, and prefill riding along with decode rows), where launching every kernel from Python costs more host
time than the GPU needs for the step at tensor parallel 4 and 8.

Supported: dense pre-norm decoders with sequential residuals (llama, mistral, qwen2, gemma, phi3, cohere without
parallel residual, ...), bf16 weights.  Anything else (MoE, parallel residual, gemma2's extra norms, fp8 weights,
learned position embeddings) keeps the Python path in `DecoderModel.forward`.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_void_p
from typing import List, Optional

import torch

from ..ops import native

P, I, L, F = c_void_p, c_int, c_longlong, c_float


class LxLoraSite(Structure):
    _fields_ = [("off_a", L), ("off_b", L), ("nparts", I), ("n0", I), ("n1", I), ("tmap_group", I), ("enabled", I), ("pad_", I)]


class LxLayerDesc(Structure):
    _fields_ = [("input_norm_w", P), ("input_norm_b", P), ("post_norm_w", P), ("post_norm_b", P), ("qkv_w", P), ("qkv_b", P),
                ("o_w", P), ("o_b", P), ("gate_up_w", P), ("gate_up_b", P), ("down_w", P), ("down_b", P),
                ("ld_qkv", L), ("ld_o", L), ("ld_gate_up", L), ("ld_down", L), ("kv_cache", P), ("lora", LxLoraSite * 4),
                ("layer_index", I), ("window", I), ("k_scale", F), ("v_scale", F)]


class LxModelDesc(Structure):
    _fields_ = [("H", I), ("nh", I), ("nkv", I), ("d", I), ("inter", I), ("rot", I), ("page", I), ("apply_rope", I), ("act", I),
                ("gated", I), ("layernorm", I), ("pad0_", I),
                ("n_qkv", I), ("n_o_in", I), ("n_gate_up", I), ("n_down_in", I),
                ("eps", F), ("norm_offset", F), ("attn_scale", F), ("softcap", F),
                ("cos_sin", P),
                ("gemm_ws", P), ("gemm_ws_bytes", L), ("gemm_counters", P), ("status", P), ("num_sms", I), ("pad1_", I),
                ("lora_v3", P), ("v3_plane_stride", L), ("v3_planes", I), ("ldv", I), ("lora_v", P), ("lora_counters", P),
                ("n_lora_counters", I), ("pad2_", I),
                ("attn_part_o", P), ("attn_part_lse", P), ("attn_splits", I), ("attn_part_tokens", I),
                ("arena", P), ("slot_base", P), ("slot_rank", P), ("slot_tmaps", P),
                ("num_slots", I), ("max_rank", I), ("groups_per_slot", I), ("fused_lora", I),
                ("lora_vimg", P), ("lora_vimg_bytes", L), ("arena_elems", L), ("lora_sync", P), ("lora_fence_maps", I),
                ("tc_prefill", I), ("kv_blocks", I), ("kv_fp8", I), ("pad3_", I)]


class LxStepDesc(Structure):
    _fields_ = [("T", I), ("n_decode", I), ("positions", P), ("slots", P),
                ("dec_block_tables", P), ("ctx_lens", P), ("dec_max_blocks", I), ("nsplit", I),
                ("block_tables", P), ("cu_q", P), ("cache_lens", P), ("tile_seq", P), ("tile_q0", P),
                ("max_blocks", I), ("n_attn_tiles", I),
                ("tok_slot", P), ("lora_tiles", P), ("num_tiles", I), ("max_tile_rows", I), ("live_tiles", I), ("pad5_", I),
                ("normed", P), ("qkv", P), ("attn", P), ("gate_up", P), ("act", P)]


class LxAllReduce(ctypes.Structure):
    _fields_ = [("peer_ptrs", P), ("in_off", L), ("out_off", L), ("cnt_off", L), ("state", P), ("status", P), ("rank", I), ("world", I)]


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def supported(model) -> bool:
    c = model.config
    if model.device.type != "cuda" or model.dtype != torch.bfloat16 or model.quantized is not None:
        return False
    if c.is_moe or c.parallel_residual or model.pos_embed is not None or c.model_type == "gemma2":
        return False
    if model.alibi_slopes is not None or c.clip_qkv or model.embed_norm is not None:
        return False
    for lw in model.layers:
        if lw.post_norm is None or lw.gate_up_w is None or lw.down_w is None or lw.post_ffn_norm is not None:
            return False
        for w in (lw.qkv_w, lw.o_w, lw.gate_up_w, lw.down_w):
            if not isinstance(w, torch.Tensor) or w.dtype != torch.bfloat16 or w.stride(1) != 1:
                return False
    return True


class NativeExecutor:
    SITES = ("qkv", "o", "gate_up", "down")

    def __init__(self, model, kv_layers: List[torch.Tensor]):
        lib = native.load()
        for name, st in (("lx_layer_desc_bytes", LxLayerDesc), ("lx_model_desc_bytes", LxModelDesc), ("lx_step_desc_bytes", LxStepDesc)):
            fn = getattr(lib, name)
            fn.restype = I
            if fn() != ctypes.sizeof(st):
                raise RuntimeError(f"{name}: C++ says {fn()} bytes, ctypes says {ctypes.sizeof(st)}")
        if lib.lx_allreduce_desc_bytes() != ctypes.sizeof(LxAllReduce):
            raise RuntimeError("lx_allreduce_desc_bytes: C++ and ctypes disagree")
        lib.lx_run_layers.argtypes = [POINTER(LxModelDesc), POINTER(LxLayerDesc), I, POINTER(LxStepDesc), P, F, POINTER(LxAllReduce), P,
                                      POINTER(ctypes.c_void_p), P]
        lib.lx_run_layers.restype = I
        for name in ("lx_layer_attention", "lx_layer_mlp"):
            fn = getattr(lib, name)
            fn.argtypes = [POINTER(LxModelDesc), POINTER(LxLayerDesc), POINTER(LxStepDesc), P, P, F, P, P]
            fn.restype = I
        self.lib = lib
        self.model = model
        self.adapters = model.adapters
        self.kv_ptrs = [t.data_ptr() for t in kv_layers]
        c = model.config
        ws = native.workspace(model.device)
        m = LxModelDesc()
        m.H, m.nh, m.nkv, m.d, m.inter, m.rot = model.hidden, model.nh, model.nkv, model.d, model.inter, c.rotary_dim
        m.page = kv_layers[0].shape[3]
        m.tc_prefill, m.kv_blocks = int(native.TC_PREFILL), kv_layers[0].shape[0]
        m.kv_fp8 = int(kv_layers[0].dtype == torch.float8_e4m3fn)
        m.apply_rope = int(not c.learned_positions)
        m.act, m.gated = native._ACTS[c.hidden_act], int(model.gated)
        m.layernorm = int(c.norm_type.startswith("layernorm"))
        lw0 = model.layers[0]
        m.n_qkv, m.n_o_in, m.n_gate_up, m.n_down_in = lw0.qkv_w.shape[0], lw0.o_w.shape[1], lw0.gate_up_w.shape[0], lw0.down_w.shape[1]
        m.eps, m.norm_offset, m.attn_scale = c.rms_norm_eps, c.norm_weight_offset, c.attn_scale
        m.softcap = c.attn_logit_softcapping or 0.0
        m.cos_sin = model.cos_sin.data_ptr()
        m.gemm_ws, m.gemm_ws_bytes, m.gemm_counters, m.status, m.num_sms = (ws.gemm_ws.data_ptr(), ws.gemm_ws.numel(),
                                                                            ws.gemm_counters.data_ptr(), ws.status.data_ptr(), ws.num_sms)
        m.lora_v3, m.v3_plane_stride, m.v3_planes, m.ldv = ws.lora_v3.data_ptr(), ws.lora_v3.stride(0), ws.lora_v3.shape[0], ws.lora_v3.stride(1)
        assert ws.lora_v.stride(0) == ws.lora_v3.stride(1)
        m.lora_v, m.lora_counters, m.n_lora_counters = ws.lora_v.data_ptr(), ws.lora_counters.data_ptr(), ws.lora_counters.numel()
        m.attn_part_o, m.attn_part_lse = ws.attn_part_o.data_ptr(), ws.attn_part_lse.data_ptr()
        m.attn_splits, m.attn_part_tokens = ws.attn_splits, ws.attn_part_tokens
        self.max_tokens = ws.lora_v.shape[0]
        ad = self.adapters
        lora = ad is not None and ad.max_rank > 0 and ad.is_cuda
        if lora:
            from ..adapters.manager import TMAP_GROUPS
            m.arena, m.slot_base, m.slot_rank, m.slot_tmaps = (ad.arena.data_ptr(), ad.slot_base.data_ptr(), ad.slot_rank.data_ptr(),
                                                               ad.slot_tmaps.data_ptr())
            m.num_slots, m.max_rank, m.groups_per_slot = ad.slot_rank.shape[0], ad.max_rank, ad.groups_per_slot
            m.fused_lora = int(model.fused_lora_max_tokens)        # rows up to which LoRA rides inside the GEMM launch
            m.lora_vimg, m.lora_vimg_bytes = ws.lora_vimg.data_ptr(), ws.lora_vimg.numel() * 2
            m.arena_elems = ad.arena.numel()
            m.lora_sync = ws.lora_sync.data_ptr()
            m.lora_fence_maps = native.LORA_FENCE_MAPS
        self.m = m
        self.layers = (LxLayerDesc * len(model.layers))()
        for li, lw in enumerate(model.layers):
            d = self.layers[li]
            d.input_norm_w, d.input_norm_b, d.post_norm_w, d.post_norm_b = _p(lw.input_norm), _p(lw.input_norm_b), _p(lw.post_norm), _p(lw.post_norm_b)
            d.qkv_w, d.qkv_b, d.o_w, d.o_b = _p(lw.qkv_w), _p(lw.qkv_b), _p(lw.o_w), _p(lw.o_b)
            d.gate_up_w, d.gate_up_b, d.down_w, d.down_b = _p(lw.gate_up_w), _p(lw.gate_up_b), _p(lw.down_w), _p(lw.down_b)
            d.ld_qkv, d.ld_o, d.ld_gate_up, d.ld_down = lw.qkv_w.stride(0), lw.o_w.stride(0), lw.gate_up_w.stride(0), lw.down_w.stride(0)
            d.kv_cache = self.kv_ptrs[li]
            d.k_scale, d.v_scale = (model.kv_scales[li] if getattr(model, "kv_scales", None) else (1.0, 1.0))
            d.layer_index = li
            d.window = c.sliding_window or 0
            for si, g in enumerate(self.SITES):
                site = d.lora[si]
                gi = ad.layout.groups.get(g) if lora else None
                if gi is None:
                    site.enabled = 0
                    continue
                site.enabled = 1
                site.off_a, site.off_b = ad.layout.unit_off(g, li, "A"), ad.layout.unit_off(g, li, "B")
                site.nparts = len(gi.parts)
                site.n0, site.n1 = gi.bounds
                site.tmap_group = TMAP_GROUPS.index(g)
        self._keep = []      # tensors of the step in flight (the descriptors hold raw pointers)

    def matches(self, model, kv_layers) -> bool:
        return (self.adapters is model.adapters and len(kv_layers) == len(self.kv_ptrs)
                and all(t.data_ptr() == p for t, p in zip(kv_layers, self.kv_ptrs)))

    def run_layers(self, inp, h: torch.Tensor) -> tuple:
        """Runs every decoder layer on the embedded input `h` [T, H].  Returns (pending, residual): the last block's
        output and the residual stream, to be joined by the final norm as in the Python path."""
        model, lib = self.model, self.lib
        c = model.config
        T = h.shape[0]
        if T > self.max_tokens:
            raise ValueError(f"{T} tokens exceed the LoRA scratch of {self.max_tokens} rows")
        dev, bf = h.device, torch.bfloat16
        m = self.m
        normed = torch.empty(T, m.H, dtype=bf, device=dev)
        qkv = torch.empty(T, m.n_qkv, dtype=bf, device=dev)
        attn = torch.empty(T, m.n_o_in, dtype=bf, device=dev)
        gate_up = torch.empty(T, m.n_gate_up, dtype=bf, device=dev)
        act = torch.empty(T, m.inter, dtype=bf, device=dev)
        out_a = torch.empty(T, m.H, dtype=bf, device=dev)
        out_b = torch.empty(T, m.H, dtype=bf, device=dev)
        s = LxStepDesc()
        s.T = T
        s.positions, s.slots = _p(inp.positions), _p(inp.slots)
        if inp.n_decode:
            s.n_decode = inp.n_decode
            s.dec_block_tables, s.dec_max_blocks, s.ctx_lens = _p(inp.dec_block_tables), inp.dec_block_tables.shape[1], _p(inp.ctx_lens)
        elif not inp.is_prefill:
            s.n_decode = T
            s.dec_block_tables, s.dec_max_blocks, s.ctx_lens = _p(inp.block_tables), inp.block_tables.shape[1], _p(inp.ctx_lens)
        if inp.is_prefill:
            s.block_tables, s.max_blocks = _p(inp.block_tables), inp.block_tables.shape[1]
            s.cu_q, s.cache_lens, s.tile_seq, s.tile_q0 = _p(inp.cu_q), _p(inp.cache_lens), _p(inp.tile_seq), _p(inp.tile_q0)
            s.n_attn_tiles = inp.tile_seq.shape[0]
        s.nsplit = inp.attn_nsplit
        if inp.tok_slot is not None and m.max_rank > 0:
            s.tok_slot = _p(inp.tok_slot)
            if inp.lora_tiles is not None:
                s.lora_tiles, s.num_tiles, s.max_tile_rows = _p(inp.lora_tiles.table), inp.lora_tiles.num_tiles, inp.lora_tiles.max_rows
                s.live_tiles = inp.lora_tiles.live
        s.normed, s.qkv, s.attn, s.gate_up, s.act = normed.data_ptr(), qkv.data_ptr(), attn.data_ptr(), gate_up.data_ptr(), act.data_ptr()
        if self.adapters is not None:
            m.max_rank = self.adapters.max_rank if self.adapters.is_cuda else 0      # changes as adapters come and go
        stream = torch.cuda.current_stream().cuda_stream
        tp = model.tp
        rm = float(c.residual_multiplier)
        residual = h
        pending = None
        # under tensor parallelism the O / down projections write their partial sums straight into the symmetric input
        # area of the all-reduce kernel when it fits; the reduced result comes back as a view that the next half consumes
        fused = tp.fused if tp.world_size > 1 else None
        dst = fused.all_reduce_input(T, m.H) if fused is not None else None
        buf_a = dst if dst is not None else out_a
        buf_b = dst if dst is not None else out_b
        nL = len(model.layers)
        if tp.world_size == 1 or dst is not None:
            # the whole layer loop in one native call (under tensor parallelism with the all-reduce kernel launched from there too)
            ar = None
            if tp.world_size > 1:
                ar = LxAllReduce(peer_ptrs=ctypes.cast(fused.ar_ptrs, P), in_off=0, out_off=fused.ar_area, cnt_off=2 * fused.ar_area,
                                 state=fused.ar_state.data_ptr(), status=fused.ws.status.data_ptr(), rank=tp.rank, world=tp.world_size)
            out_ptr = ctypes.c_void_p()
            rc = lib.lx_run_layers(ctypes.byref(m), self.layers, nL, ctypes.byref(s), residual.data_ptr(), rm,
                                   ctypes.byref(ar) if ar is not None else None, out_a.data_ptr(), ctypes.byref(out_ptr), stream)
            native._check(rc, "lx_run_layers")
            pending = fused.ar_out[: T * m.H].view(T, m.H) if ar is not None else out_a
            assert out_ptr.value == pending.data_ptr()
            fused_lora = T <= m.fused_lora and s.lora_tiles and s.max_tile_rows <= 32 and m.max_rank <= 64     # shrink and expand ride in the GEMM then
            lora_launches = (0 if fused_lora else 8) if s.tok_slot else 0        # per layer: shrink and expand at four projections
            attn_kernels = (1 if s.n_decode else 0) + (1 if T > s.n_decode else 0)
            native.launch_count += nL * (10 + attn_kernels + lora_launches + (2 if ar is not None else 0)) - 1      # `_check` counted one
            if ar is not None:
                fused.ar_calls += 2 * nL
            self._keep = [normed, qkv, attn, gate_up, act, out_a, inp, ar]
            return pending, residual
        for li in range(nL):
            l = ctypes.byref(self.layers[li])
            rc = lib.lx_layer_attention(ctypes.byref(m), l, ctypes.byref(s), _p(pending), residual.data_ptr(), rm, buf_a.data_ptr(), stream)
            native._check(rc, "lx_layer_attention")
            a_res = tp.all_reduce(buf_a) if tp.world_size > 1 else buf_a
            rc = lib.lx_layer_mlp(ctypes.byref(m), l, ctypes.byref(s), a_res.data_ptr(), residual.data_ptr(), rm, buf_b.data_ptr(), stream)
            native._check(rc, "lx_layer_mlp")
            pending = tp.all_reduce(buf_b) if tp.world_size > 1 else buf_b
        fused_lora = T <= m.fused_lora and s.lora_tiles and s.max_tile_rows <= 32 and m.max_rank <= 64
        lora_launches = (0 if fused_lora else 8) if s.tok_slot else 0
        attn_kernels = (1 if s.n_decode else 0) + (1 if T > s.n_decode else 0)
        native.launch_count += len(model.layers) * (8 + attn_kernels + lora_launches)
        self._keep = [normed, qkv, attn, gate_up, act, out_a, inp]
        return pending, residual
