"""Encoder-decoder (T5 family) model and its batch state.

The reference serves T5 / Flan-T5 through `Seq2SeqLM` (`server/lorax_server/models/seq2seq_lm.py`, model code
`models/custom_modeling/t5_modeling.py`): a padded batch, the encoder run once at Prefill, the decoder stepped with a growing
`past_key_values`.  This module keeps the same division of work with ragged state instead of padding:

* `encode(list of token lists)` runs the encoder over each input and returns, per request, the cross-attention keys and values of
  every decoder layer (computed once: they do not change during decoding);
* `decode_step(states)` advances every request by one position: self-attention over the request's own cached keys / values,
  cross-attention over its encoder projections, feed-forward, final norm, shared or separate lm_head.

T5 specifics: RMS layer norm without bias, no 1/sqrt(d) in the attention scores, a learned relative-position bias (32 buckets,
shared by all layers of a stack; bidirectional in the encoder, causal in the decoder), ReLU or gated-GELU feed-forward,
logits scaled by d_model^-0.5 when the lm_head is tied to the embedding.

The math runs as PyTorch matmuls in the model dtype: the requests of a step differ in encoder length and decoder position, and
these models (hundreds of millions of parameters) are not what the tcgen05 kernels of the decoder-only path were sized for.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..utils.weights import AbstractWeights

SEQ2SEQ_TYPES = ("t5", "mt5", "umt5")


@dataclass
class Seq2SeqConfig:
    model_type: str = "t5"
    vocab_size: int = 32128
    d_model: int = 512
    d_kv: int = 64
    d_ff: int = 2048
    num_layers: int = 6
    num_decoder_layers: Optional[int] = None
    num_heads: int = 8
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128
    layer_norm_epsilon: float = 1e-6
    feed_forward_proj: str = "relu"               # "relu" | "gated-gelu"
    tie_word_embeddings: bool = True
    decoder_start_token_id: int = 0
    eos_token_id: int = 1
    pad_token_id: int = 0

    def __post_init__(self):
        if self.num_decoder_layers is None:
            self.num_decoder_layers = self.num_layers

    @classmethod
    def from_dict(cls, d: dict) -> "Seq2SeqConfig":
        known = {f for f in cls.__dataclass_fields__}
        kw = {k: v for k, v in d.items() if k in known and v is not None}
        if d.get("model_type") == "umt5":
            raise NotImplementedError("umt5 keeps one relative-position table per layer")
        return cls(**kw)

    # what the shard runtime reads from a model config
    @property
    def num_hidden_layers(self):
        return self.num_decoder_layers

    sliding_window = None


def relative_position_bucket(rel: torch.Tensor, bidirectional: bool, num_buckets: int, max_distance: int) -> torch.Tensor:
    """T5's log-spaced bucketing of (key position - query position)."""
    ret = torch.zeros_like(rel)
    if bidirectional:
        num_buckets //= 2
        ret = ret + (rel > 0).long() * num_buckets
        rel = rel.abs()
    else:
        rel = -torch.min(rel, torch.zeros_like(rel))
    max_exact = num_buckets // 2
    small = rel < max_exact
    large = max_exact + (torch.log(rel.float().clamp_min(1) / max_exact) / math.log(max_distance / max_exact) * (num_buckets - max_exact)).long()
    large = torch.min(large, torch.full_like(large, num_buckets - 1))
    return ret + torch.where(small, rel, large)


@dataclass
class _Attn:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    o: torch.Tensor


@dataclass
class _Layer:
    self_attn: _Attn
    self_norm: torch.Tensor
    ff_norm: torch.Tensor
    wi: List[torch.Tensor]
    wo: torch.Tensor
    cross_attn: Optional[_Attn] = None
    cross_norm: Optional[torch.Tensor] = None


@dataclass
class Seq2SeqState:
    """One request while it decodes."""
    cross_k: List[torch.Tensor]                    # per decoder layer [heads, S, d_kv]
    cross_v: List[torch.Tensor]
    self_k: List[Optional[torch.Tensor]] = field(default_factory=list)    # per layer [heads, t, d_kv], grows by one per step
    self_v: List[Optional[torch.Tensor]] = field(default_factory=list)
    last_token: int = 0
    position: int = 0                              # decoder position of `last_token`


class Seq2SeqModel:
    def __init__(self, config: Seq2SeqConfig, device, dtype):
        self.config = config
        self.device = torch.device(device)
        self.dtype = dtype
        self.shared: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        self.enc: List[_Layer] = []
        self.dec: List[_Layer] = []
        self.enc_bias: Optional[torch.Tensor] = None      # [buckets, heads]
        self.dec_bias: Optional[torch.Tensor] = None
        self.enc_final: Optional[torch.Tensor] = None
        self.dec_final: Optional[torch.Tensor] = None
        self.adapters = None
        from ..parallel.tp import TensorParallel
        self.tp = TensorParallel.single()

    # ------------------------------------------------------------------ loading
    @classmethod
    def from_weights(cls, config: Seq2SeqConfig, w: AbstractWeights, device, dtype) -> "Seq2SeqModel":
        m = cls(config, device, dtype)

        def get(name):
            return w.get_tensor(name).to(dtype).to(m.device).contiguous()

        def attn(prefix):
            return _Attn(get(prefix + ".q.weight"), get(prefix + ".k.weight"), get(prefix + ".v.weight"), get(prefix + ".o.weight"))

        def ff(prefix):
            if w.has_tensor(prefix + ".wi_0.weight"):
                return [get(prefix + ".wi_0.weight"), get(prefix + ".wi_1.weight")], get(prefix + ".wo.weight")
            return [get(prefix + ".wi.weight")], get(prefix + ".wo.weight")
        m.shared = get("shared.weight") if w.has_tensor("shared.weight") else get("encoder.embed_tokens.weight")
        m.lm_head = m.shared if (config.tie_word_embeddings or not w.has_tensor("lm_head.weight")) else get("lm_head.weight")
        for i in range(config.num_layers):
            p = f"encoder.block.{i}.layer."
            wi, wo = ff(p + "1.DenseReluDense")
            m.enc.append(_Layer(attn(p + "0.SelfAttention"), get(p + "0.layer_norm.weight"), get(p + "1.layer_norm.weight"), wi, wo))
        for i in range(config.num_decoder_layers):
            p = f"decoder.block.{i}.layer."
            wi, wo = ff(p + "2.DenseReluDense")
            m.dec.append(_Layer(attn(p + "0.SelfAttention"), get(p + "0.layer_norm.weight"), get(p + "2.layer_norm.weight"), wi, wo,
                                attn(p + "1.EncDecAttention"), get(p + "1.layer_norm.weight")))
        m.enc_bias = get("encoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight")
        m.dec_bias = get("decoder.block.0.layer.0.SelfAttention.relative_attention_bias.weight")
        m.enc_final = get("encoder.final_layer_norm.weight")
        m.dec_final = get("decoder.final_layer_norm.weight")
        return m

    # ------------------------------------------------------------------ pieces
    def _norm(self, x, w):
        v = x.float().pow(2).mean(-1, keepdim=True)
        return (x.float() * torch.rsqrt(v + self.config.layer_norm_epsilon)).to(x.dtype) * w

    def _heads(self, x, w):
        c = self.config
        return (x @ w.t()).view(x.shape[0], c.num_heads, c.d_kv).transpose(0, 1)          # [heads, T, d_kv]

    def _ff(self, x, layer: _Layer):
        if len(layer.wi) == 2:
            h = F.gelu(x @ layer.wi[0].t(), approximate="tanh") * (x @ layer.wi[1].t())
        else:
            h = F.relu(x @ layer.wi[0].t())
        return h @ layer.wo.t()

    def _bias(self, table, q_pos: torch.Tensor, k_pos: torch.Tensor, bidirectional: bool) -> torch.Tensor:
        c = self.config
        rel = k_pos[None, :] - q_pos[:, None]
        b = relative_position_bucket(rel, bidirectional, c.relative_attention_num_buckets, c.relative_attention_max_distance)
        return table[b].permute(2, 0, 1).float()                                          # [heads, Tq, Tk]

    @staticmethod
    def _attend(q, k, v, bias=None):
        s = q.float() @ k.float().transpose(1, 2)                                          # no 1/sqrt(d) in T5
        if bias is not None:
            s = s + bias
        return (torch.softmax(s, -1) @ v.float()).to(q.dtype)                              # [heads, Tq, d_kv]

    def _merge(self, x, w):
        return x.transpose(0, 1).reshape(x.shape[1], -1) @ w.t()

    # ------------------------------------------------------------------ encoder
    def encode(self, ids: List[int]) -> Seq2SeqState:
        """Encoder over one input; returns the request's decoding state with the cross-attention projections filled in."""
        c = self.config
        x = self.shared[torch.tensor(ids, dtype=torch.long, device=self.device)]
        pos = torch.arange(len(ids), device=self.device)
        bias = self._bias(self.enc_bias, pos, pos, True)
        for l in self.enc:
            n = self._norm(x, l.self_norm)
            a = self._attend(self._heads(n, l.self_attn.q), self._heads(n, l.self_attn.k), self._heads(n, l.self_attn.v), bias)
            x = x + self._merge(a, l.self_attn.o)
            x = x + self._ff(self._norm(x, l.ff_norm), l)
        x = self._norm(x, self.enc_final)
        st = Seq2SeqState(cross_k=[self._heads(x, l.cross_attn.k) for l in self.dec], cross_v=[self._heads(x, l.cross_attn.v) for l in self.dec],
                          self_k=[None] * len(self.dec), self_v=[None] * len(self.dec), last_token=c.decoder_start_token_id, position=0)
        return st

    # ------------------------------------------------------------------ decoder
    def decode_step(self, states: List[Seq2SeqState]) -> torch.Tensor:
        """One decoder position for every request: consumes `last_token` at `position`, appends to the self-attention cache and
        returns logits [len(states), vocab] (fp32).  The caller stores the chosen token in `last_token` and bumps `position`."""
        c = self.config
        toks = torch.tensor([s.last_token for s in states], dtype=torch.long, device=self.device)
        x = self.shared[toks]                                                              # [R, d_model]
        for li, l in enumerate(self.dec):
            n = self._norm(x, l.self_norm)
            q, k, v = self._heads(n, l.self_attn.q), self._heads(n, l.self_attn.k), self._heads(n, l.self_attn.v)      # [heads, R, d]
            outs = []
            for r, s in enumerate(states):
                s.self_k[li] = k[:, r:r + 1] if s.self_k[li] is None else torch.cat([s.self_k[li], k[:, r:r + 1]], 1)
                s.self_v[li] = v[:, r:r + 1] if s.self_v[li] is None else torch.cat([s.self_v[li], v[:, r:r + 1]], 1)
                kp = torch.arange(s.position + 1, device=self.device)
                bias = self._bias(self.dec_bias, kp[-1:], kp, False)
                outs.append(self._attend(q[:, r:r + 1], s.self_k[li], s.self_v[li], bias))
            x = x + self._merge(torch.cat(outs, 1), l.self_attn.o)
            n = self._norm(x, l.cross_norm)
            q = self._heads(n, l.cross_attn.q)
            outs = [self._attend(q[:, r:r + 1], s.cross_k[li], s.cross_v[li]) for r, s in enumerate(states)]
            x = x + self._merge(torch.cat(outs, 1), l.cross_attn.o)
            x = x + self._ff(self._norm(x, l.ff_norm), l)
        x = self._norm(x, self.dec_final)
        if self.lm_head is self.shared:
            x = x * (c.d_model ** -0.5)
        return (x @ self.lm_head.t()).float()

    def generate(self, ids: List[int], max_new_tokens: int = 20) -> List[int]:
        """Greedy decoding of one input (tests, quick checks)."""
        st = self.encode(ids)
        out = []
        for _ in range(max_new_tokens):
            tok = int(self.decode_step([st])[0].argmax())
            out.append(tok)
            st.last_token, st.position = tok, st.position + 1
            if tok == self.config.eos_token_id:
                break
        return out
