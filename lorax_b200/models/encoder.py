"""Bidirectional encoders for the embedding and token-classification endpoints: BERT, RoBERTa / XLM-R, DistilBERT.

The reference serves these through `FlashBert`, `FlashXlmRoberta` and `FlashDistilBert`
(`server/lorax_server/models/flash_bert.py:186-218`, `flash_roberta.py`, `flash_distilbert.py:150-180`): `embed` returns
the hidden state of each sequence's first token, `classify` runs the token-classification head and returns, per
token, the arg-max label with its softmax probability.

Everything dense runs on the same operator layer as the decoder (tcgen05 GEMM with bias, fused residual + LayerNorm,
GELU); one forward pass takes a ragged batch (no padding: `cu_seqlens` marks the sequences).  The attention itself is
bidirectional over a few hundred tokens and is computed per sequence with PyTorch's scaled-dot-product attention --
these endpoints are not on the generation hot path.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..ops import get_ops
from ..utils.weights import AbstractWeights

ENCODER_TYPES = ("bert", "roberta", "xlm-roberta", "distilbert", "camembert")


@dataclass
class EncoderConfig:
    model_type: str = "bert"
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12
    hidden_act: str = "gelu"
    pad_token_id: int = 0
    id2label: Dict[int, str] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: dict) -> "EncoderConfig":
        mt = d.get("model_type", "bert")
        if mt == "distilbert":      # DistilBERT spells its sizes differently
            return cls(model_type=mt, vocab_size=d["vocab_size"], hidden_size=d["dim"], num_hidden_layers=d["n_layers"],
                       num_attention_heads=d["n_heads"], intermediate_size=d["hidden_dim"],
                       max_position_embeddings=d.get("max_position_embeddings", 512), type_vocab_size=0, layer_norm_eps=1e-12,
                       hidden_act=d.get("activation", "gelu"), pad_token_id=d.get("pad_token_id", 0),
                       id2label={int(k): v for k, v in (d.get("id2label") or {}).items()})
        return cls(model_type=mt, vocab_size=d["vocab_size"], hidden_size=d["hidden_size"], num_hidden_layers=d["num_hidden_layers"],
                   num_attention_heads=d["num_attention_heads"], intermediate_size=d["intermediate_size"],
                   max_position_embeddings=d.get("max_position_embeddings", 512), type_vocab_size=d.get("type_vocab_size", 2),
                   layer_norm_eps=d.get("layer_norm_eps", 1e-12), hidden_act=d.get("hidden_act", "gelu"),
                   pad_token_id=d.get("pad_token_id", 0), id2label={int(k): v for k, v in (d.get("id2label") or {}).items()})


@dataclass
class EncoderLayer:
    qkv_w: torch.Tensor
    qkv_b: torch.Tensor
    o_w: torch.Tensor
    o_b: torch.Tensor
    attn_ln_w: torch.Tensor
    attn_ln_b: torch.Tensor
    ffn1_w: torch.Tensor
    ffn1_b: torch.Tensor
    ffn2_w: torch.Tensor
    ffn2_b: torch.Tensor
    out_ln_w: torch.Tensor
    out_ln_b: torch.Tensor


def _names(mt: str, i: int) -> Dict[str, str]:
    if mt == "distilbert":
        p = f"transformer.layer.{i}."
        return dict(q=p + "attention.q_lin", k=p + "attention.k_lin", v=p + "attention.v_lin", o=p + "attention.out_lin",
                    attn_ln=p + "sa_layer_norm", ffn1=p + "ffn.lin1", ffn2=p + "ffn.lin2", out_ln=p + "output_layer_norm")
    p = f"encoder.layer.{i}."
    return dict(q=p + "attention.self.query", k=p + "attention.self.key", v=p + "attention.self.value", o=p + "attention.output.dense",
                attn_ln=p + "attention.output.LayerNorm", ffn1=p + "intermediate.dense", ffn2=p + "output.dense",
                out_ln=p + "output.LayerNorm")


class EncoderModel:
    """Post-LayerNorm transformer encoder with an optional token-classification head."""

    def __init__(self, config: EncoderConfig, device, dtype: torch.dtype):
        self.config = config
        self.device = torch.device(device)
        self.dtype = dtype
        self.ops = get_ops(self.device, dtype)
        self.nh = config.num_attention_heads
        self.d = config.hidden_size // config.num_attention_heads
        self.layers: List[EncoderLayer] = []
        self.word_emb = self.pos_emb = self.type_emb = None
        self.emb_ln_w = self.emb_ln_b = None
        self.cls_w = self.cls_b = None
        # RoBERTa numbers positions from pad_token_id + 1 (HF `create_position_ids_from_input_ids`)
        self.pos_offset = config.pad_token_id + 1 if config.model_type in ("roberta", "xlm-roberta", "camembert") else 0

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_weights(cls, config: EncoderConfig, weights: AbstractWeights, device, dtype: torch.dtype) -> "EncoderModel":
        m = cls(config, device, dtype)
        mt = config.model_type
        prefixes = ["", mt.replace("-", "_") + ".", "bert.", "roberta.", "distilbert."]

        def get(name: str) -> torch.Tensor:
            for p in prefixes:
                if weights.has_tensor(p + name):
                    return weights.get_tensor(p + name).to(device=m.device, dtype=dtype)
            raise KeyError(f"encoder weight {name} not found")

        def opt(name: str) -> Optional[torch.Tensor]:
            try:
                return get(name)
            except KeyError:
                return None

        m.word_emb = get("embeddings.word_embeddings.weight")
        m.pos_emb = get("embeddings.position_embeddings.weight")
        m.type_emb = opt("embeddings.token_type_embeddings.weight")
        m.emb_ln_w, m.emb_ln_b = get("embeddings.LayerNorm.weight"), get("embeddings.LayerNorm.bias")
        for i in range(config.num_hidden_layers):
            n = _names(mt, i)
            m.layers.append(EncoderLayer(
                qkv_w=torch.cat([get(n[x] + ".weight") for x in "qkv"], 0).contiguous(),
                qkv_b=torch.cat([get(n[x] + ".bias") for x in "qkv"], 0).contiguous(),
                o_w=get(n["o"] + ".weight"), o_b=get(n["o"] + ".bias"),
                attn_ln_w=get(n["attn_ln"] + ".weight"), attn_ln_b=get(n["attn_ln"] + ".bias"),
                ffn1_w=get(n["ffn1"] + ".weight"), ffn1_b=get(n["ffn1"] + ".bias"),
                ffn2_w=get(n["ffn2"] + ".weight"), ffn2_b=get(n["ffn2"] + ".bias"),
                out_ln_w=get(n["out_ln"] + ".weight"), out_ln_b=get(n["out_ln"] + ".bias")))
        if weights.has_tensor("classifier.weight"):
            m.cls_w = weights.get_tensor("classifier.weight").to(device=m.device, dtype=dtype)
            m.cls_b = weights.get_tensor("classifier.bias").to(device=m.device, dtype=dtype)
        return m

    @classmethod
    def random_init(cls, config: EncoderConfig, device, dtype: torch.dtype, seed: int = 0, num_labels: int = 0) -> "EncoderModel":
        from ..utils.weights import InMemoryWeights
        return cls.from_weights(config, InMemoryWeights(random_encoder_state_dict(config, seed, num_labels)), device, dtype)

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids: torch.Tensor, cu_seqlens: Sequence[int], token_type_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """input_ids [T] (sequences back to back, `cu_seqlens` = their boundaries on the host) -> hidden states [T, H]."""
        c, ops = self.config, self.ops
        T = input_ids.shape[0]
        pos = torch.cat([torch.arange(b - a, device=self.device) for a, b in zip(cu_seqlens[:-1], cu_seqlens[1:])]) + self.pos_offset
        h = self.word_emb[input_ids.long()] + self.pos_emb[pos]
        if self.type_emb is not None:
            tt = token_type_ids.long() if token_type_ids is not None else torch.zeros(T, dtype=torch.long, device=self.device)
            h = h + self.type_emb[tt]
        h = ops.norm_residual(h.contiguous(), None, self.emb_ln_w, c.layer_norm_eps, bias=self.emb_ln_b, layernorm=True)
        H = c.hidden_size
        act = "gelu" if c.hidden_act in ("gelu", "gelu_new") else c.hidden_act
        for lw in self.layers:
            qkv = ops.gemm(h, lw.qkv_w, bias=lw.qkv_b)
            attn = torch.empty(T, H, dtype=h.dtype, device=h.device)
            for a, b in zip(cu_seqlens[:-1], cu_seqlens[1:]):
                q, k, v = (qkv[a:b, i * H:(i + 1) * H].view(b - a, self.nh, self.d).transpose(0, 1) for i in range(3))
                attn[a:b] = F.scaled_dot_product_attention(q, k, v).transpose(0, 1).reshape(b - a, H)
            o = ops.gemm(attn, lw.o_w, bias=lw.o_b)
            # post-LN: h <- LN(h + o); norm_residual adds into `h` (the residual stream) and returns the normed value
            h = ops.norm_residual(o, h, lw.attn_ln_w, c.layer_norm_eps, bias=lw.attn_ln_b, layernorm=True)
            f = ops.act_mul(ops.gemm(h, lw.ffn1_w, bias=lw.ffn1_b), c.intermediate_size, act, gated=False)
            f = ops.gemm(f, lw.ffn2_w, bias=lw.ffn2_b)
            h = ops.norm_residual(f, h, lw.out_ln_w, c.layer_norm_eps, bias=lw.out_ln_b, layernorm=True)
        return h

    def embed(self, seqs: Sequence[Sequence[int]]) -> List[List[float]]:
        """One vector per sequence: the final hidden state of its first token."""
        ids, cu = self._pack(seqs)
        h = self.forward(ids, cu)
        first = torch.tensor(cu[:-1], device=self.device)
        return h[first].float().cpu().tolist()

    def classify(self, seqs: Sequence[Sequence[int]]) -> Tuple[List[List[str]], List[List[float]]]:
        """Per token: the arg-max label of the classification head and its softmax probability."""
        if self.cls_w is None:
            raise ValueError("this checkpoint has no `classifier` head")
        ids, cu = self._pack(seqs)
        logits = self.ops.gemm(self.forward(ids, cu), self.cls_w, bias=self.cls_b).float()
        prob, pred = torch.softmax(logits, dim=-1).max(dim=-1)
        prob, pred = prob.cpu().tolist(), pred.cpu().tolist()
        labels = self.config.id2label
        out_l, out_p = [], []
        for a, b in zip(cu[:-1], cu[1:]):
            out_l.append([labels.get(i, f"LABEL_{i}") for i in pred[a:b]])
            out_p.append(prob[a:b])
        return out_l, out_p

    def _pack(self, seqs: Sequence[Sequence[int]]):
        cu = [0]
        flat: List[int] = []
        limit = self.config.max_position_embeddings - self.pos_offset
        for s in seqs:
            s = list(s)[:limit]
            if not s:
                raise ValueError("empty input")
            flat += s
            cu.append(len(flat))
        return torch.tensor(flat, dtype=torch.int32, device=self.device), cu


def random_encoder_state_dict(config: EncoderConfig, seed: int = 0, num_labels: int = 0) -> Dict[str, torch.Tensor]:
    """Random weights under the HuggingFace names of the architecture (tests, synthetic benchmarks)."""
    g = torch.Generator().manual_seed(seed)
    H, I = config.hidden_size, config.intermediate_size
    mt = config.model_type

    def rn(*shape, std=0.05):
        return torch.randn(*shape, generator=g) * std

    sd = {"embeddings.word_embeddings.weight": rn(config.vocab_size, H), "embeddings.position_embeddings.weight": rn(config.max_position_embeddings, H),
          "embeddings.LayerNorm.weight": 1 + rn(H), "embeddings.LayerNorm.bias": rn(H)}
    if config.type_vocab_size:
        sd["embeddings.token_type_embeddings.weight"] = rn(config.type_vocab_size, H)
    for i in range(config.num_hidden_layers):
        n = _names(mt, i)
        for key, (o, k) in dict(q=(H, H), k=(H, H), v=(H, H), o=(H, H), ffn1=(I, H), ffn2=(H, I)).items():
            sd[n[key] + ".weight"] = rn(o, k)
            sd[n[key] + ".bias"] = rn(o)
        for key in ("attn_ln", "out_ln"):
            sd[n[key] + ".weight"] = 1 + rn(H)
            sd[n[key] + ".bias"] = rn(H)
    if num_labels:
        sd["classifier.weight"] = rn(num_labels, H, std=0.2)
        sd["classifier.bias"] = rn(num_labels)
    return sd
