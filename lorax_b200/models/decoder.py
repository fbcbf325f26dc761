"""One config-driven decoder for the whole causal-LM zoo.

The reference keeps one hand-written module per architecture (`server/lorax_server/models/custom_modeling/
flash_{llama,mistral,mixtral,qwen2,gemma,gemma2,phi3,gpt2,...}_modeling.py`); they differ in a handful of
switches (norm type, bias, activation, rotary fraction, soft-capping, parallel residual, MoE), which
:class:`lorax_b200.config.ModelConfig` carries.  The layer sequence matches the reference Mistral decoder
(`flash_mistral_modeling.py:230-645`): fused QKV (+LoRA) -> RoPE + KV write -> attention -> O (+LoRA) ->
residual-fused norm -> fused gate_up (+LoRA) -> act*mul -> down (+LoRA), vocab-parallel lm_head.

The forward is ragged (padding-free) over a paged KV cache and is written once against the operator
interface of :mod:`lorax_b200.ops`; on a B200 those are the sm_100a kernels, on CPU the PyTorch oracle.
"""

from __future__ import annotations

import os
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..config import ModelConfig
from ..ops import get_ops, reference
from ..parallel.tp import TensorParallel
from ..utils.quant_formats import GroupQuantWeight
from ..utils.weights import AbstractWeights

# projection groups that share one base GEMM; LoRA blobs follow the same grouping
GROUPS = ("qkv", "o", "gate_up", "down")


def alibi_slopes(n_heads: int, bias_max: float = 8.0, interleave: bool = False) -> torch.Tensor:
    """ALiBi slopes [n_heads] fp32.  Powers of two: slope_i = 2^(-bias_max * i / n), i = 1..n.  Otherwise BLOOM appends the odd
    powers of the next finer base to those of the largest power of two below n (modeling_bloom.py: build_alibi_tensor), and MPT
    (`interleave`) takes the slopes of the next power of two above n, odd positions first."""
    import math
    if interleave:
        m = 2 ** math.ceil(math.log2(n_heads))
        s = torch.pow(2.0, -torch.arange(1, m + 1, dtype=torch.float32) * (bias_max / m))
        return (torch.cat([s[1::2], s[::2]])[:n_heads] if m != n_heads else s).contiguous()
    m = 2 ** math.floor(math.log2(n_heads))
    s = torch.pow(2.0, -torch.arange(1, m + 1, dtype=torch.float32) * (bias_max / m))
    if m < n_heads:
        extra = torch.pow(2.0, -torch.arange(1, 2 * (n_heads - m), 2, dtype=torch.float32) * (bias_max / (2 * m)))
        s = torch.cat([s, extra])
    return s.contiguous()


@dataclass
class Fp8Weight:
    """A projection matrix in block-scaled fp8: e4m3 values [N, K] and one fp32 scale per 128 x 128 block."""
    q: torch.Tensor
    scale: torch.Tensor

    @property
    def shape(self):
        return self.q.shape


@dataclass
class LayerWeights:
    input_norm: torch.Tensor
    qkv_w: torch.Tensor
    o_w: torch.Tensor
    post_norm: Optional[torch.Tensor]
    gate_up_w: Optional[torch.Tensor]
    down_w: Optional[torch.Tensor]
    input_norm_b: Optional[torch.Tensor] = None
    post_norm_b: Optional[torch.Tensor] = None
    qkv_b: Optional[torch.Tensor] = None
    o_b: Optional[torch.Tensor] = None
    gate_up_b: Optional[torch.Tensor] = None
    down_b: Optional[torch.Tensor] = None
    pre_ffn_norm: Optional[torch.Tensor] = None       # gemma2
    post_ffn_norm: Optional[torch.Tensor] = None      # gemma2
    router_w: Optional[torch.Tensor] = None           # MoE gate [E, H]
    experts_w13: Optional[torch.Tensor] = None        # [E_local, 2I, H], or a list of E_local packed matrices
    experts_w2: Optional[torch.Tensor] = None         # [E_local, H, I], likewise


@dataclass
class StepInputs:
    """Everything one forward needs, already on the model's device (int32 index tensors)."""
    input_ids: torch.Tensor
    positions: torch.Tensor
    slots: Optional[torch.Tensor]
    is_prefill: bool
    block_tables: torch.Tensor                       # prefill: [B, max_blocks]; decode: [T, max_blocks]
    ctx_lens: Optional[torch.Tensor] = None          # decode: [T]
    cu_q: Optional[torch.Tensor] = None              # prefill: [B+1]
    cache_lens: Optional[torch.Tensor] = None        # prefill: [B]
    tile_seq: Optional[torch.Tensor] = None
    tile_q0: Optional[torch.Tensor] = None
    lm_head_indices: Optional[torch.Tensor] = None   # rows that need logits (None = all)
    tok_slot: Optional[torch.Tensor] = None          # [T] adapter slot per token (-1 = base); None = no LoRA this step
    head_tok_slot: Optional[torch.Tensor] = None     # adapter slot per lm_head row
    lora_tiles: Optional[object] = None              # adapters.manager.LoraTiles: rows grouped by adapter (tensor-core shrink)
    attn_nsplit: int = 1
    num_tokens: Optional[int] = None                 # live rows when the tensors are padded (graphs)
    local_logits: bool = False                       # TP: return this rank's vocabulary shard instead of gathering
    # Mixed step: rows [0, n_decode) are decode rows (one token each, described by ctx_lens / dec_block_tables), the
    # rows after them are prefill tokens (described by cu_q / cache_lens / block_tables / tile_*).  One pass over
    # the weights then serves both, which is what a prefill costs least when a decode batch is running anyway.
    n_decode: int = 0
    dec_block_tables: Optional[torch.Tensor] = None
    # vision-language prompts: rows of the embedded sequence that are replaced by projected image features
    embed_rows: Optional[torch.Tensor] = None
    embed_values: Optional[torch.Tensor] = None


class DecoderModel:
    def __init__(self, config: ModelConfig, device, dtype: torch.dtype, tp: Optional[TensorParallel] = None,
                 max_positions: Optional[int] = None):
        self.config = config
        self.device = torch.device(device)
        self.dtype = dtype
        self.tp = tp or TensorParallel.single()
        ws = self.tp.world_size
        c = config
        if c.num_attention_heads % ws != 0:
            raise ValueError(f"{c.num_attention_heads} heads cannot be split over {ws} shards")
        self.nh = c.num_attention_heads // ws
        # KV heads are split when possible and replicated otherwise (reference: flash_causal_lm.py:1139-1149)
        self.nkv = max(c.num_key_value_heads // ws, 1)
        self.kv_replicas = max(ws // c.num_key_value_heads, 1)
        self.d = c.head_dim
        self.inter = c.intermediate_size // ws if not c.is_moe else c.intermediate_size
        self.hidden = c.hidden_size
        self.vocab = c.vocab_size
        self.vocab_local = (c.vocab_size + ws - 1) // ws
        self.vocab_start = self.tp.rank * self.vocab_local
        self.ops = get_ops(self.device, dtype)
        self.layers: List[LayerWeights] = []
        self.embed: Optional[torch.Tensor] = None
        self.pos_embed: Optional[torch.Tensor] = None
        self.embed_norm: Optional[torch.Tensor] = None          # BLOOM normalises the embeddings
        self.embed_norm_b: Optional[torch.Tensor] = None
        self.alibi_slopes: Optional[torch.Tensor] = None        # [local heads] fp32 (BLOOM, MPT)
        self.final_norm: Optional[torch.Tensor] = None
        self.final_norm_b: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        self.lm_head_b: Optional[torch.Tensor] = None
        self.max_positions = max_positions or min(c.max_position_embeddings, 32768)
        scaling = c.rope_scaling
        if scaling and scaling.get("rope_type", scaling.get("type")) == "dynamic" and "original_max_position_embeddings" not in scaling:
            # dynamic NTK stretches the base once the table is longer than the length the model was trained at
            scaling = dict(scaling, original_max_position_embeddings=c.max_position_embeddings)
        self.cos_sin = reference.rope_cache(c.rotary_dim, self.max_positions, c.rope_theta, scaling, device=self.device)
        self.adapters = None     # AdapterManager, attached by the runtime
        self.quantized: Optional[str] = None
        self.keep_hidden = False                 # keep the head's input rows of the last eager forward pass in `last_hidden`
        self.last_hidden: Optional[torch.Tensor] = None
        self._native = None
        self.use_native_layers = self.device.type == "cuda" and os.environ.get("LORAX_NATIVE_LAYERS", "1") != "0"
        # LoRA inside the GEMM launch for steps of up to this many rows (0: always separate shrink / expand kernels).  Measured on
        # B200 over the four projections of a Mistral-7B layer with 100 rank-16 adapters: 0.30 ms against 0.38 ms for the three
        # launches at 256 rows, 0.57 against 0.63 at 1024, 1.74 against 2.00 at 4096; steps of 8192 prompt tokens plus their decode rows
        # (Llama-3-8B, fp8 weights expanded per projection) gained 4 % end to end.  A step with more table entries than the kernel
        # holds (512) falls back to the separate kernels by itself.
        self.fused_lora_max_tokens = int(os.environ.get("LORAX_FUSED_LORA_MAX_TOKENS", "16384")) if os.environ.get("LORAX_FUSED_LORA", "1") != "0" else 0
        self.fused_lora = self.fused_lora_max_tokens > 0
        self.kv_scales = None        # per layer (k scale, v scale) of an e4m3 KV cache, set when the cache is built
        self.gated = c.model_type not in ("gpt2", "gpt_bigcode", "gpt_neox", "falcon", "RefinedWeb", "RefinedWebModel", "phi", "bloom",
                                          "mpt", "opt")
        if c.alibi:
            full = alibi_slopes(c.num_attention_heads, c.alibi_bias_max, interleave=c.model_type == "mpt")
            self.alibi_slopes = full[self.tp.rank * self.nh:(self.tp.rank + 1) * self.nh].to(self.device).contiguous()

    # ------------------------------------------------------------------ shapes
    @property
    def q_size(self):
        return self.nh * self.d

    @property
    def kv_size(self):
        return self.nkv * self.d

    @property
    def qkv_size(self):
        return self.q_size + 2 * self.kv_size

    def group_shapes(self) -> Dict[str, dict]:
        """Per projection group: K (input features on this rank), N (outputs on this rank), output part sizes,
        and which side is sharded (column groups shard N, row groups shard K)."""
        g = {
            "qkv": dict(K=self.hidden, parts=[self.q_size, self.kv_size, self.kv_size], shard="col",
                        names=["q_proj", "k_proj", "v_proj"]),
            "o": dict(K=self.q_size, parts=[self.hidden], shard="row", names=["o_proj"]),
        }
        if not self.config.is_moe:
            if self.gated:
                g["gate_up"] = dict(K=self.hidden, parts=[self.inter, self.inter], shard="col", names=["gate_proj", "up_proj"])
            else:
                g["gate_up"] = dict(K=self.hidden, parts=[self.inter], shard="col", names=["up_proj"])
            g["down"] = dict(K=self.inter, parts=[self.hidden], shard="row", names=["down_proj"])
        for v in g.values():
            v["N"] = sum(v["parts"])
        return g

    # ------------------------------------------------------------------ init
    @classmethod
    def random_init(cls, config: ModelConfig, device, dtype, seed: int = 0, tp: Optional[TensorParallel] = None,
                    std: float = 0.02, max_positions: Optional[int] = None) -> "DecoderModel":
        """Random weights of the right shapes.  Every rank draws the FULL tensors from the same seed and keeps its
        shard, so TP=k and TP=1 hold the same model (needed for the rank-consistency tests)."""
        m = cls(config, device, dtype, tp, max_positions)
        c, ws, rk = config, m.tp.world_size, m.tp.rank
        gen = torch.Generator(device="cpu").manual_seed(seed)

        def rnd(*shape, s=std):
            return torch.randn(*shape, generator=gen, dtype=torch.float32) * s

        def put(t):
            return t.to(dtype).to(m.device).contiguous()

        def rows(t, n_total):      # shard dim 0 into ws blocks
            b = n_total // ws
            return t[rk * b:(rk + 1) * b]

        H, d = c.hidden_size, c.head_dim
        emb = rnd(c.vocab_size, H)
        m.embed = put(emb if ws == 1 else _pad_rows(emb, m.vocab_local * ws)[m.vocab_start:m.vocab_start + m.vocab_local])
        if c.learned_positions:
            m.pos_embed = put(rnd(c.max_position_embeddings + c.position_offset, H))
        if c.embed_norm:
            m.embed_norm, m.embed_norm_b = put(torch.ones(H) + rnd(H, s=0.01)), put(rnd(H, s=0.01))
        ln = c.norm_type.startswith("layernorm")
        has_ln_bias = c.norm_type == "layernorm"
        for _ in range(c.num_hidden_layers):
            q = rnd(c.num_attention_heads * d, H)
            k = rnd(c.num_key_value_heads * d, H)
            v = rnd(c.num_key_value_heads * d, H)
            o = rnd(H, c.num_attention_heads * d)
            kv_rank = (rk // m.kv_replicas) if c.num_key_value_heads < ws else rk
            ksh = k.view(c.num_key_value_heads, d, H)[kv_rank * m.nkv:(kv_rank + 1) * m.nkv].reshape(-1, H)
            vsh = v.view(c.num_key_value_heads, d, H)[kv_rank * m.nkv:(kv_rank + 1) * m.nkv].reshape(-1, H)
            qkv = torch.cat([rows(q, q.shape[0]), ksh, vsh], 0)
            ob = o.shape[1] // ws
            lw = LayerWeights(
                input_norm=put(torch.ones(H) - c.norm_weight_offset + rnd(H, s=0.01)),
                qkv_w=put(qkv), o_w=put(o[:, rk * ob:(rk + 1) * ob]),
                post_norm=put(torch.ones(H) - c.norm_weight_offset + rnd(H, s=0.01)) if not c.parallel_residual or c.model_type in ("gpt_neox",) else None,
                gate_up_w=None, down_w=None)
            if ln and has_ln_bias:
                lw.input_norm_b = put(rnd(H, s=0.01))
                if lw.post_norm is not None:
                    lw.post_norm_b = put(rnd(H, s=0.01))
            if c.attention_bias:
                qb, kb, vb = rnd(q.shape[0]), rnd(k.shape[0]), rnd(v.shape[0])
                kbs = kb.view(c.num_key_value_heads, d)[kv_rank * m.nkv:(kv_rank + 1) * m.nkv].reshape(-1)
                vbs = vb.view(c.num_key_value_heads, d)[kv_rank * m.nkv:(kv_rank + 1) * m.nkv].reshape(-1)
                lw.qkv_b = put(torch.cat([rows(qb, qb.shape[0]), kbs, vbs]))
                if c.model_type not in ("qwen2", "qwen"):
                    lw.o_b = put(rnd(H)) if rk == 0 else put(torch.zeros(H))
            I = c.intermediate_size
            if c.is_moe:
                E = c.num_local_experts
                lw.router_w = put(rnd(E, H))
                w1, w3, w2 = rnd(E, I, H), rnd(E, I, H), rnd(E, H, I)
                el = max(E // ws, 1)                 # expert parallel: rank r owns experts [r*el, (r+1)*el)
                esl = slice(rk * el, (rk + 1) * el) if el < E else slice(0, E)
                lw.experts_w13 = put(torch.cat([w1, w3], 1)[esl])
                lw.experts_w2 = put(w2[esl])
            else:
                ib = I // ws
                up = rnd(I, H)
                down = rnd(H, I)
                if m.gated:
                    gate = rnd(I, H)
                    lw.gate_up_w = put(torch.cat([gate[rk * ib:(rk + 1) * ib], up[rk * ib:(rk + 1) * ib]], 0))
                else:
                    lw.gate_up_w = put(up[rk * ib:(rk + 1) * ib])
                lw.down_w = put(down[:, rk * ib:(rk + 1) * ib])
                if c.mlp_bias:
                    ub = rnd(I)
                    lw.gate_up_b = put(ub[rk * ib:(rk + 1) * ib])
                    lw.down_b = put(rnd(H)) if rk == 0 else put(torch.zeros(H))
            if c.model_type == "gemma2":
                lw.pre_ffn_norm = put(torch.ones(H) - c.norm_weight_offset + rnd(H, s=0.01))
                lw.post_ffn_norm = put(torch.ones(H) - c.norm_weight_offset + rnd(H, s=0.01))
            m.layers.append(lw)
        m.final_norm = put(torch.ones(H) - c.norm_weight_offset + rnd(H, s=0.01))
        if ln and has_ln_bias:
            m.final_norm_b = put(rnd(H, s=0.01))
        if c.tie_word_embeddings:
            m.lm_head = m.embed
        else:
            head = rnd(c.vocab_size, H)
            m.lm_head = put(head if ws == 1 else _pad_rows(head, m.vocab_local * ws)[m.vocab_start:m.vocab_start + m.vocab_local])
        return m

    @classmethod
    def random_init_on_device(cls, config: ModelConfig, device, dtype, seed: int = 0, tp: Optional[TensorParallel] = None,
                              std: float = 0.02, max_positions: Optional[int] = None) -> "DecoderModel":
        """Random weights generated directly on the device, one shard per rank (benchmarks with 7B-70B shapes:
        drawing the full tensors on the host as `random_init` does would take minutes).  Ranks use different
        seeds, so this is a statistically equivalent model per TP degree, not the same model."""
        m = cls(config, device, dtype, tp, max_positions)
        c, ws = config, m.tp.world_size
        gen = torch.Generator(device=m.device).manual_seed(seed * 1000 + m.tp.rank)

        def rnd(*shape, s=std):
            return (torch.randn(*shape, generator=gen, device=m.device, dtype=torch.float32) * s).to(dtype)

        def ones(n):
            return (torch.ones(n, device=m.device) - c.norm_weight_offset).to(dtype)

        H = c.hidden_size
        m.embed = rnd(m.vocab_local if ws > 1 else c.vocab_size, H)
        if c.learned_positions:
            m.pos_embed = rnd(c.max_position_embeddings, H)
        for _ in range(c.num_hidden_layers):
            lw = LayerWeights(input_norm=ones(H), qkv_w=rnd(m.qkv_size, H), o_w=rnd(H, m.q_size), post_norm=ones(H),
                              gate_up_w=None, down_w=None)
            if c.attention_bias:
                lw.qkv_b = rnd(m.qkv_size)
            if c.is_moe:
                E, I = c.num_local_experts, c.intermediate_size
                e_local = max(E // ws, 1)
                lw.router_w = rnd(E, H)
                lw.experts_w13 = rnd(e_local, 2 * I, H)
                lw.experts_w2 = rnd(e_local, H, I)
            else:
                lw.gate_up_w = rnd((2 if m.gated else 1) * m.inter, H)
                lw.down_w = rnd(H, m.inter)
            m.layers.append(lw)
        m.final_norm = ones(H)
        m.lm_head = m.embed if c.tie_word_embeddings else rnd(m.vocab_local if ws > 1 else c.vocab_size, H)
        return m

    @classmethod
    def from_weights(cls, config: ModelConfig, weights: AbstractWeights, device, dtype, tp: Optional[TensorParallel] = None,
                     max_positions: Optional[int] = None) -> "DecoderModel":
        from .loading import load_decoder_weights
        m = cls(config, device, dtype, tp, max_positions)
        load_decoder_weights(m, weights)
        return m

    # ------------------------------------------------------------------ forward
    def _norm(self, x, residual, w, b=None, x_scale: float = 1.0):
        c = self.config
        return self.ops.norm_residual(x, residual, w, c.rms_norm_eps, bias=b, weight_offset=c.norm_weight_offset,
                                      x_scale=x_scale, layernorm=c.norm_type.startswith("layernorm"))

    def quantize_fp8(self):
        """Replace the dense projection matrices of every layer by block-scaled fp8 (e4m3, 128 x 128 scales) for the
        fp8 tensor-core GEMM; embeddings, norms, the lm_head, MoE experts and every LoRA adapter stay as they are.
        The reference's `--quantize fp8` does the same on load with per-tensor scales (layers/fp8.py:14-45)."""
        for lw in self.layers:
            for name in ("qkv_w", "o_w", "gate_up_w", "down_w"):
                w = getattr(lw, name)
                if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[1] % 16 == 0:
                    q, s = reference.quantize_weight_fp8_block128(w)
                    setattr(lw, name, Fp8Weight(q.view(torch.uint8) if q.is_cuda else q, s))
        self.quantized = "fp8"
        self._native = None

    def quantize(self, method: str, group: int = 128):
        """Weight-only quantisation of the dense projection matrices on load (`--quantize` of the reference's shard CLI,
        cli.py:15-28): 4-bit groups (`gptq`, `awq`, `int4`), int8 per channel (`eetq`, `bitsandbytes`, `int8`), the nf4 / fp4
        code books (`bitsandbytes-nf4`, `bitsandbytes-fp4`) and HQQ at 4 / 3 / 2 bits.  Matrices the checkpoint already
        holds in packed form are left as loaded."""
        if method == "fp8":
            return self.quantize_fp8()
        from ..utils.quant_formats import quantize_weight
        for lw in self.layers:
            for name in ("qkv_w", "o_w", "gate_up_w", "down_w"):
                w = getattr(lw, name)
                if isinstance(w, torch.Tensor) and w.dim() == 2 and w.shape[1] % 128 == 0 and w.shape[0] % 16 == 0:
                    setattr(lw, name, quantize_weight(w, method, group))
            for name in ("experts_w13", "experts_w2"):       # mixture of experts: one packed matrix per local expert
                w = getattr(lw, name)
                if isinstance(w, torch.Tensor) and w.dim() == 3 and w.shape[2] % 128 == 0 and w.shape[1] % 16 == 0:
                    setattr(lw, name, [quantize_weight(w[e], method, group) for e in range(w.shape[0])])
        self.quantized = method
        self._native = None

    def _gemm(self, x, w, b, out=None):
        if isinstance(w, GroupQuantWeight):
            xb = x if x.dtype == torch.bfloat16 or not x.is_cuda else x.to(torch.bfloat16)
            y = self.ops.gemm_wq(xb, w, bias=b, out=out if out is not None and out.dtype == xb.dtype else None)
            if out is not None and y is not out:
                out.copy_(y)
                return out
            return y if y.dtype == x.dtype else y.to(x.dtype)
        if out is not None and isinstance(w, torch.Tensor):
            return self.ops.gemm(x, w, bias=b, out=out)
        if isinstance(w, Fp8Weight):
            y = self.ops.gemm_fp8(x if x.dtype == torch.bfloat16 or not x.is_cuda else x.to(torch.bfloat16), w.q, w.scale, bias=b)
            return y if y.dtype == x.dtype else y.to(x.dtype)
        return self.ops.gemm(x, w, bias=b)

    def _linear(self, x, w, b, group: str, layer: int, inp: StepInputs, tok_slot=None, out=None):
        """Base GEMM plus the multi-adapter LoRA delta for the projection group.  On a GPU with the rows grouped by adapter
        that is ONE launch (shrink items, base tiles, expand UMMAs); otherwise a shrink launch, the GEMM and an expand launch."""
        ts = tok_slot if tok_slot is not None else inp.tok_slot
        epi = None
        if (self.fused_lora and x.shape[0] <= self.fused_lora_max_tokens and self.adapters is not None and ts is not None
                and inp.lora_tiles is not None and x.is_cuda and x.dtype == torch.bfloat16):
            bf16_w = isinstance(w, torch.Tensor) and w.dtype == torch.bfloat16
            # long steps run fp8 projections as bf16 GEMMs over expanded weights anyway: the adapters ride in that launch too
            fp8_long = isinstance(w, Fp8Weight) and x.shape[0] >= getattr(self.ops, "FP8_EXPAND_MIN_TOKENS", 1 << 30)
            lf = self.adapters.fused(group, layer, inp.lora_tiles) if (bf16_w or fp8_long) else None
            if lf is not None:
                wb = w if bf16_w else self.ops.fp8_expand(w.q, w.scale)
                if wb is not None:
                    y = self.ops.gemm_lora_fused(x, wb, lf, bias=b, out=out)      # shrink, base GEMM and expand: one launch
                    if y is not None:
                        return y
        if self.adapters is not None and ts is not None:
            epi = self.adapters.shrink(self.ops, x, ts, group, layer, tiles=inp.lora_tiles)
        if epi is None:
            return self._gemm(x, w, b, out=out)
        y = self._gemm(x, w, b, out=out)
        self.adapters.expand(self.ops, epi, y, tiles=inp.lora_tiles)
        return y

    def _row_parallel(self, x, w, b, group: str, layer: int, inp: StepInputs):
        """Row-parallel projection + all-reduce.  With the NVLink kernels enabled and a decode-sized batch this is one
        fused GEMM -> reduce-scatter -> all-gather kernel; the rank's partial LoRA delta is reduced with it."""
        fused = self.tp.fused if self.tp.world_size > 1 else None
        if (fused is not None and x.is_cuda and x.shape[0] <= min(fused.MAX_TOKENS, fused.max_fused_tokens) and b is None
                and not self.config.parallel_residual and isinstance(w, torch.Tensor)):
            addend = None
            if self.adapters is not None and (inp.tok_slot is not None or inp.lora_tiles is not None) and self.adapters.max_rank > 0:
                addend = torch.zeros(x.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
                self.adapters.apply(self.ops, x, addend, inp.tok_slot, group, layer, tiles=inp.lora_tiles)
            return fused.gemm_allreduce(x, w, None, addend)
        dst = None
        if fused is not None and x.is_cuda and isinstance(w, torch.Tensor):
            dst = fused.all_reduce_input(x.shape[0], w.shape[0])      # the GEMM writes where the all-reduce kernel reads
        out = self._linear(x, w, b, group, layer, inp, out=dst)
        if self.tp.world_size > 1:
            out = self.tp.all_reduce(out)
        return out

    def _native_executor(self, inp: StepInputs, kv_cache: List[torch.Tensor]):
        """The C++ layer executor for eager steps (prefill, mixed prefill + decode) of the architectures it covers;
        None keeps the per-kernel Python path (decode steps are CUDA graphs, where host time does not matter)."""
        if not inp.is_prefill or not self.use_native_layers or torch.cuda.is_current_stream_capturing():
            return None
        from . import native_exec
        ex = self._native
        if ex is not None and ex.matches(self, kv_cache):
            return ex
        if not native_exec.supported(self):
            return None
        self._native = native_exec.NativeExecutor(self, kv_cache)
        return self._native

    def forward(self, inp: StepInputs, kv_cache: List[torch.Tensor]) -> torch.Tensor:
        """-> logits [n_out, vocab] (full vocabulary on every rank)."""
        c, ops = self.config, self.ops
        fused = self.tp.fused if self.tp.world_size > 1 else None
        if fused is not None and fused.embed_ptrs is not None and inp.input_ids.is_cuda:
            h = fused.embed(inp.input_ids, c.embedding_multiplier)       # peer reads, no collective
        else:
            h = ops.embed(inp.input_ids, self.embed, v0=self.vocab_start, v1=self.vocab_start + self.embed.shape[0],
                          mult=c.embedding_multiplier)
            if self.tp.world_size > 1:
                h = self.tp.all_reduce(h)
        if inp.embed_rows is not None:
            h = h.index_copy(0, inp.embed_rows + inp.n_decode, inp.embed_values.to(h.dtype))
        if self.pos_embed is not None:
            h = h + self.pos_embed[inp.positions.long() + c.position_offset]
        if self.embed_norm is not None:
            h = self._norm(h, None, self.embed_norm, self.embed_norm_b)
        residual = h
        pending = None      # output of the previous block that still has to be added to the residual stream
        rm = c.residual_multiplier
        native_exec = self._native_executor(inp, kv_cache)
        if native_exec is not None:
            pending, residual = native_exec.run_layers(inp, h.contiguous())
        for li, lw in enumerate(self.layers if native_exec is None else ()):
            if pending is None:
                normed = self._norm(residual, None, lw.input_norm, lw.input_norm_b)
            else:
                normed = self._norm(pending, residual, lw.input_norm, lw.input_norm_b, x_scale=rm)
            attn_out = self._attention(normed, lw, li, inp, kv_cache[li])
            if c.parallel_residual:
                mlp_in = normed if lw.post_norm is None else self._norm(residual, None, lw.post_norm, lw.post_norm_b)
                mlp_out = self._mlp(mlp_in, lw, li, inp)
                pending = attn_out + mlp_out
                continue
            if lw.post_ffn_norm is not None:      # gemma2: norm the block output before it joins the residual
                attn_out = self._norm(attn_out, None, lw.post_norm)
                normed2 = self._norm(attn_out, residual, lw.pre_ffn_norm)
                mlp_out = self._mlp(normed2, lw, li, inp)
                pending = self._norm(mlp_out, None, lw.post_ffn_norm)
                continue
            normed2 = self._norm(attn_out, residual, lw.post_norm, lw.post_norm_b, x_scale=rm)
            pending = self._moe(normed2, lw, li, inp) if c.is_moe else self._mlp(normed2, lw, li, inp)
        hidden = self._norm(pending, residual, self.final_norm, self.final_norm_b, x_scale=rm)
        if inp.lm_head_indices is not None:
            hidden = hidden.index_select(0, inp.lm_head_indices.long()) if hidden.device.type == "cpu" else hidden[inp.lm_head_indices.long()]
        if self.keep_hidden:
            self.last_hidden = hidden          # rows match the returned logits (Medusa heads read them)
        if hidden.shape[0] == 0:               # a step of prompt chunks only: keys and values are written, no row is scored
            return torch.empty(0, self.vocab, dtype=hidden.dtype, device=hidden.device)
        return self.lm_head_forward(hidden, inp)

    def lm_head_forward(self, hidden: torch.Tensor, inp: StepInputs) -> torch.Tensor:
        c = self.config
        scale = c.logit_scale / c.logits_scaling if c.logits_scaling != 1.0 else c.logit_scale
        logits = self.ops.gemm(hidden, self.lm_head, bias=self.lm_head_b, out_scale=scale)
        ts = inp.head_tok_slot
        if ts is not None and self.adapters is not None and self.adapters.layout.has_lm_head:
            self.adapters.apply(self.ops, hidden, logits, ts, "lm_head", 0)
        if self.tp.world_size > 1:
            if inp.local_logits:
                return logits
            logits = self.tp.all_gather_cols(logits)[:, : self.vocab]
        elif logits.shape[1] != self.vocab:
            logits = logits[:, : self.vocab]
        return logits

    def _attention(self, x, lw: LayerWeights, li: int, inp: StepInputs, kv: torch.Tensor):
        c, ops = self.config, self.ops
        qkv = self._linear(x, lw.qkv_w, lw.qkv_b, "qkv", li, inp)
        if c.clip_qkv:
            qkv.clamp_(-c.clip_qkv, c.clip_qkv)
        kvs = {"kv_scale": self.kv_scales[li]} if (self.kv_scales and kv.dtype == torch.float8_e4m3fn) else {}
        ops.rope_kvwrite(qkv, inp.positions, self.cos_sin, kv, inp.slots, self.nh, self.nkv, self.d, c.rotary_dim,
                         not (c.learned_positions or c.alibi), **kvs)
        ali = {"alibi": self.alibi_slopes} if self.alibi_slopes is not None else {}
        ali.update(kvs)
        window = c.sliding_window or 0
        if c.model_type == "gemma2" and li % 2 == 1:
            window = 0
        softcap = c.attn_logit_softcapping or 0.0
        if inp.n_decode:
            nd = inp.n_decode
            attn = torch.empty(qkv.shape[0], self.nh * self.d, dtype=qkv.dtype, device=qkv.device)
            a = ops.attn_decode(qkv[:nd], kv, inp.dec_block_tables, inp.ctx_lens, self.nh, self.nkv, self.d, c.attn_scale, window,
                                softcap, inp.attn_nsplit, out=attn[:nd], **ali)
            b = ops.attn_prefill(qkv[nd:], kv, inp.block_tables, inp.cu_q, inp.cache_lens, inp.tile_seq, inp.tile_q0,
                                 self.nh, self.nkv, self.d, c.attn_scale, window, softcap, out=attn[nd:], **ali)
            if a.data_ptr() != attn.data_ptr():      # ops that ignore `out`
                attn[:nd] = a
                attn[nd:] = b
        elif inp.is_prefill:
            attn = ops.attn_prefill(qkv, kv, inp.block_tables, inp.cu_q, inp.cache_lens, inp.tile_seq, inp.tile_q0,
                                    self.nh, self.nkv, self.d, c.attn_scale, window, softcap, **ali)
        else:
            attn = ops.attn_decode(qkv, kv, inp.block_tables, inp.ctx_lens, self.nh, self.nkv, self.d, c.attn_scale, window,
                                   softcap, inp.attn_nsplit, **ali)
        return self._row_parallel(attn, lw.o_w, lw.o_b, "o", li, inp)

    def _mlp(self, x, lw: LayerWeights, li: int, inp: StepInputs):
        c, ops = self.config, self.ops
        gu = self._linear(x, lw.gate_up_w, lw.gate_up_b, "gate_up", li, inp)
        act = ops.act_mul(gu, self.inter, c.hidden_act, gated=self.gated)
        return self._row_parallel(act, lw.down_w, lw.down_b, "down", li, inp)

    def _moe(self, x, lw: LayerWeights, li: int, inp: StepInputs):
        """Top-k mixture of experts (reference math: flash_mixtral_modeling.py:449-459, 668-716): softmax over all
        experts, keep top-k, renormalise.  Experts are expert-parallel: rank r owns experts [r*E/ws, (r+1)*E/ws)."""
        from .moe import moe_forward
        return moe_forward(self, x, lw, li, inp)


def _pad_rows(t: torch.Tensor, n: int) -> torch.Tensor:
    if t.shape[0] >= n:
        return t
    return torch.cat([t, torch.zeros(n - t.shape[0], *t.shape[1:], dtype=t.dtype)], 0)
