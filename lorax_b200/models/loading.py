"""Checkpoint <-> DecoderModel.  Tensor names per architecture (HuggingFace layouts), fused-projection
assembly and tensor-parallel slicing.

Reference counterparts: the per-architecture loaders in `server/lorax_server/models/custom_modeling/*`
(e.g. `flash_mistral_modeling.py:186-190,405-431,577-596`) on top of `utils/weights.py`.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..utils.quant_formats import GroupQuantWeight, cat_rows, dequantize, same_perm
from ..utils.weights import AbstractWeights
from .decoder import DecoderModel, LayerWeights

# name templates; {i} = layer index
LLAMA_LIKE = dict(
    embed="model.embed_tokens.weight", final_norm="model.norm.weight", lm_head="lm_head.weight",
    layer="model.layers.{i}.", input_norm="input_layernorm.weight", post_norm="post_attention_layernorm.weight",
    q="self_attn.q_proj", k="self_attn.k_proj", v="self_attn.v_proj", o="self_attn.o_proj",
    gate="mlp.gate_proj", up="mlp.up_proj", down="mlp.down_proj",
)
NAME_MAPS: Dict[str, dict] = {
    "llama": LLAMA_LIKE, "mistral": LLAMA_LIKE, "qwen2": LLAMA_LIKE, "gemma": LLAMA_LIKE, "granite": LLAMA_LIKE,
    "solar": LLAMA_LIKE, "cohere": dict(LLAMA_LIKE, post_norm=None),
    "gemma2": dict(LLAMA_LIKE, pre_ffn_norm="pre_feedforward_layernorm.weight", post_ffn_norm="post_feedforward_layernorm.weight"),
    "phi3": dict(LLAMA_LIKE, qkv="self_attn.qkv_proj", gate_up="mlp.gate_up_proj", q=None, k=None, v=None, gate=None, up=None),
    "mixtral": dict(LLAMA_LIKE, gate=None, up=None, down=None, router="block_sparse_moe.gate.weight",
                    expert="block_sparse_moe.experts.{e}."),
    "gpt2": dict(embed="wte.weight", pos_embed="wpe.weight", final_norm="ln_f.weight", final_norm_b="ln_f.bias", lm_head=None,
                 layer="h.{i}.", input_norm="ln_1.weight", input_norm_b="ln_1.bias", post_norm="ln_2.weight", post_norm_b="ln_2.bias",
                 qkv="attn.c_attn", o="attn.c_proj", up="mlp.c_fc", down="mlp.c_proj", conv1d=True, q=None, k=None, v=None, gate=None,
                 prefixes=["", "transformer."]),
    "gpt_neox": dict(embed="gpt_neox.embed_in.weight", final_norm="gpt_neox.final_layer_norm.weight",
                     final_norm_b="gpt_neox.final_layer_norm.bias", lm_head="embed_out.weight", layer="gpt_neox.layers.{i}.",
                     input_norm="input_layernorm.weight", input_norm_b="input_layernorm.bias",
                     post_norm="post_attention_layernorm.weight", post_norm_b="post_attention_layernorm.bias",
                     qkv="attention.query_key_value", o="attention.dense", up="mlp.dense_h_to_4h", down="mlp.dense_4h_to_h",
                     qkv_interleaved=True, q=None, k=None, v=None, gate=None),
    "phi": dict(embed="model.embed_tokens.weight", final_norm="model.final_layernorm.weight", final_norm_b="model.final_layernorm.bias",
                lm_head="lm_head.weight", lm_head_b="lm_head.bias", layer="model.layers.{i}.", input_norm="input_layernorm.weight",
                input_norm_b="input_layernorm.bias", post_norm=None, q="self_attn.q_proj", k="self_attn.k_proj", v="self_attn.v_proj",
                o="self_attn.dense", up="mlp.fc1", down="mlp.fc2", gate=None),
    "falcon": dict(embed="transformer.word_embeddings.weight", final_norm="transformer.ln_f.weight", final_norm_b="transformer.ln_f.bias",
                   lm_head="lm_head.weight", layer="transformer.h.{i}.", input_norm="input_layernorm.weight",
                   input_norm_b="input_layernorm.bias", post_norm=None, qkv="self_attention.query_key_value", o="self_attention.dense",
                   up="mlp.dense_h_to_4h", down="mlp.dense_4h_to_h", q=None, k=None, v=None, gate=None, qkv_grouped=True),
    "gpt_bigcode": dict(embed="transformer.wte.weight", pos_embed="transformer.wpe.weight", final_norm="transformer.ln_f.weight",
                        final_norm_b="transformer.ln_f.bias", lm_head=None, layer="transformer.h.{i}.", input_norm="ln_1.weight",
                        input_norm_b="ln_1.bias", post_norm="ln_2.weight", post_norm_b="ln_2.bias", qkv="attn.c_attn", o="attn.c_proj",
                        up="mlp.c_fc", down="mlp.c_proj", q=None, k=None, v=None, gate=None),
}
NAME_MAPS["RefinedWeb"] = NAME_MAPS["RefinedWebModel"] = NAME_MAPS["falcon"]
NAME_MAPS.update({
    # first-generation Qwen: fused c_attn (q | k | v) with bias, mlp.w2 is the gate, mlp.w1 the up projection
    "qwen": dict(embed="transformer.wte.weight", final_norm="transformer.ln_f.weight", lm_head="lm_head.weight", layer="transformer.h.{i}.",
                 input_norm="ln_1.weight", post_norm="ln_2.weight", qkv="attn.c_attn", o="attn.c_proj", gate="mlp.w2", up="mlp.w1",
                 down="mlp.c_proj", q=None, k=None, v=None),
    "bloom": dict(embed="word_embeddings.weight", embed_norm="word_embeddings_layernorm.weight", embed_norm_b="word_embeddings_layernorm.bias",
                  final_norm="ln_f.weight", final_norm_b="ln_f.bias", lm_head=None, layer="h.{i}.", input_norm="input_layernorm.weight",
                  input_norm_b="input_layernorm.bias", post_norm="post_attention_layernorm.weight",
                  post_norm_b="post_attention_layernorm.bias", qkv="self_attention.query_key_value", o="self_attention.dense",
                  up="mlp.dense_h_to_4h", down="mlp.dense_4h_to_h", qkv_interleaved=True, q=None, k=None, v=None, gate=None,
                  prefixes=["transformer.", ""]),
    "mpt": dict(embed="wte.weight", pos_embed="wpe.weight", final_norm="norm_f.weight", final_norm_b="norm_f.bias", lm_head=None,
                layer="blocks.{i}.", input_norm="norm_1.weight", input_norm_b="norm_1.bias", post_norm="norm_2.weight",
                post_norm_b="norm_2.bias", qkv="attn.Wqkv", o="attn.out_proj", up="ffn.up_proj", down="ffn.down_proj", q=None, k=None,
                v=None, gate=None, prefixes=["transformer.", ""]),
    "opt": dict(embed="decoder.embed_tokens.weight", pos_embed="decoder.embed_positions.weight", final_norm="decoder.final_layer_norm.weight",
                final_norm_b="decoder.final_layer_norm.bias", lm_head=None, layer="decoder.layers.{i}.",
                input_norm="self_attn_layer_norm.weight", input_norm_b="self_attn_layer_norm.bias", post_norm="final_layer_norm.weight",
                post_norm_b="final_layer_norm.bias", q="self_attn.q_proj", k="self_attn.k_proj", v="self_attn.v_proj",
                o="self_attn.out_proj", up="fc1", down="fc2", gate=None, prefixes=["model.", ""]),
    # DBRX: fused Wqkv (clamped), LayerNorm without bias, experts stacked along rows: w1 / v1 / w2 are [E * I, H]
    "dbrx": dict(embed="transformer.wte.weight", final_norm="transformer.norm_f.weight", lm_head="lm_head.weight",
                 layer="transformer.blocks.{i}.", input_norm="norm_attn_norm.norm_1.weight", post_norm="norm_attn_norm.norm_2.weight",
                 qkv="norm_attn_norm.attn.Wqkv", o="norm_attn_norm.attn.out_proj", router="ffn.router.layer.weight",
                 experts_stacked="ffn.experts.mlp.", q=None, k=None, v=None, gate=None, up=None, down=None),
})


def _get(w: AbstractWeights, name: str, prefixes=("",)) -> Optional[torch.Tensor]:
    for p in prefixes:
        if w.has_tensor(p + name):
            return w.get_tensor(p + name)
    return None


def _need(w: AbstractWeights, name: str, prefixes=("",)) -> torch.Tensor:
    t = _get(w, name, prefixes)
    if t is None:
        raise KeyError(f"weight {name} does not exist")
    return t


def _split_qkv_full(m: DecoderModel, qkv: torch.Tensor, nm: dict):
    """Split a fused checkpoint QKV [*, H] (or bias [*]) into full q, k, v by the architecture's packing."""
    c = m.config
    nh, nkv, d = c.num_attention_heads, c.num_key_value_heads, c.head_dim
    if nm.get("qkv_interleaved"):            # neox: [nh, 3, d]
        x = qkv.view(nh, 3, d, *qkv.shape[1:])
        return (x[:, 0].reshape(nh * d, *qkv.shape[1:]), x[:, 1].reshape(nh * d, *qkv.shape[1:]), x[:, 2].reshape(nh * d, *qkv.shape[1:]))
    if nm.get("qkv_grouped"):   # falcon: [nkv, group + 2, d]; one kv head gives q | k | v, as many as q heads gives [nh, 3, d]
        g = nh // nkv
        x = qkv.view(nkv, g + 2, d, *qkv.shape[1:])
        return (x[:, :g].reshape(nh * d, *qkv.shape[1:]), x[:, g].reshape(nkv * d, *qkv.shape[1:]), x[:, g + 1].reshape(nkv * d, *qkv.shape[1:]))
    return qkv[: nh * d], qkv[nh * d: (nh + nkv) * d], qkv[(nh + nkv) * d: (nh + 2 * nkv) * d]


def _cat0(parts):
    """Row concatenation of dense matrices or of packed ones (fused QKV / gate_up of a GPTQ / AWQ checkpoint)."""
    if all(isinstance(p, GroupQuantWeight) for p in parts) and same_perm(parts):
        return cat_rows(parts)
    dt = next(p.dtype for p in parts if isinstance(p, torch.Tensor))
    return torch.cat([dequantize(p, dt) if isinstance(p, GroupQuantWeight) else p for p in parts], 0)


def _shard_qkv(m: DecoderModel, q, k, v):
    c, ws, rk = m.config, m.tp.world_size, m.tp.rank
    d = c.head_dim
    qb = q.shape[0] // ws
    kv_rank = (rk // m.kv_replicas) if c.num_key_value_heads < ws else rk
    ks = k[kv_rank * m.nkv * d:(kv_rank + 1) * m.nkv * d]
    vs = v[kv_rank * m.nkv * d:(kv_rank + 1) * m.nkv * d]
    return _cat0([q[rk * qb:(rk + 1) * qb], ks, vs])


def load_decoder_weights(m: DecoderModel, w: AbstractWeights):
    c = m.config
    nm = NAME_MAPS.get(c.model_type)
    if nm is None:
        raise NotImplementedError(f"no weight map for model_type={c.model_type}")
    pre = tuple(nm.get("prefixes", [""]))
    ws, rk = m.tp.world_size, m.tp.rank
    dev, dt = m.device, m.dtype
    conv1d = nm.get("conv1d", False)

    def fin(t):
        if isinstance(t, GroupQuantWeight):
            return t.to(dev)
        return t.to(dt).to(dev).contiguous() if t is not None else None

    def dense(t):
        return dequantize(t, dt) if isinstance(t, GroupQuantWeight) else t

    def lin(name, packed=True):            # weight as [out, in]; a packed checkpoint layer stays packed unless asked otherwise
        t = _need(w, name + ".weight", pre)
        if conv1d or not packed:
            t = dense(t)
        return t.t() if conv1d else t

    def bias(name):
        return _get(w, name + ".bias", pre)

    def rows(t, n=None):
        b = t.shape[0] // ws
        return t[rk * b:(rk + 1) * b]

    def cols(t):
        if ws > 1 and isinstance(t, GroupQuantWeight) and t.perm is not None:
            t = dense(t)                    # an act-order layer's groups mix the column shards of all ranks
        b = t.shape[1] // ws
        return t[:, rk * b:(rk + 1) * b]

    emb = _need(w, nm["embed"], pre)
    if ws > 1:
        padded = torch.zeros(m.vocab_local * ws, emb.shape[1], dtype=emb.dtype)
        padded[: emb.shape[0]] = emb
        emb_l = padded[m.vocab_start: m.vocab_start + m.vocab_local]
    else:
        emb_l = emb
    m.embed = fin(emb_l)
    if nm.get("pos_embed") and c.learned_positions:
        m.pos_embed = fin(_need(w, nm["pos_embed"], pre))
    if nm.get("embed_norm"):
        m.embed_norm = fin(_need(w, nm["embed_norm"], pre))
        m.embed_norm_b = fin(_get(w, nm["embed_norm_b"], pre))
    m.final_norm = fin(_need(w, nm["final_norm"], pre))
    if nm.get("final_norm_b"):
        m.final_norm_b = fin(_get(w, nm["final_norm_b"], pre))
    head = _get(w, nm["lm_head"], pre) if nm.get("lm_head") else None
    if head is None or c.tie_word_embeddings:
        m.lm_head = m.embed
    else:
        if ws > 1:
            padded = torch.zeros(m.vocab_local * ws, head.shape[1], dtype=head.dtype)
            padded[: head.shape[0]] = head
            head = padded[m.vocab_start: m.vocab_start + m.vocab_local]
        m.lm_head = fin(head)
    if nm.get("lm_head_b"):
        hb = _get(w, nm["lm_head_b"], pre)
        if hb is not None:
            m.lm_head_b = fin(rows(hb) if ws > 1 else hb)

    m.layers = []
    for i in range(c.num_hidden_layers):
        L = nm["layer"].format(i=i)
        if nm.get("qkv_grouped"):
            # falcon: the 40b layout has one LayerNorm per branch (ln_attn, ln_mlp); blocks without parallel attention
            # carry a post_attention_layernorm instead
            nm = dict(nm)
            if w.has_tensor(pre[0] + L + "ln_attn.weight"):
                nm.update(input_norm="ln_attn.weight", input_norm_b="ln_attn.bias", post_norm="ln_mlp.weight", post_norm_b="ln_mlp.bias")
            elif w.has_tensor(pre[0] + L + "post_attention_layernorm.weight"):
                nm.update(post_norm="post_attention_layernorm.weight", post_norm_b="post_attention_layernorm.bias")
        if nm.get("qkv"):
            q, k, v = _split_qkv_full(m, lin(L + nm["qkv"], packed=not (nm.get("qkv_interleaved") or nm.get("qkv_grouped"))), nm)
            qb_ = bias(L + nm["qkv"])
            qkv_b = _shard_qkv(m, *_split_qkv_full(m, qb_, nm)) if qb_ is not None else None
        else:
            q, k, v = lin(L + nm["q"]), lin(L + nm["k"]), lin(L + nm["v"])
            bq, bk, bv = bias(L + nm["q"]), bias(L + nm["k"]), bias(L + nm["v"])
            qkv_b = _shard_qkv(m, bq, bk, bv) if bq is not None else None
        o_w = lin(L + nm["o"])
        o_b = bias(L + nm["o"])
        lw = LayerWeights(input_norm=fin(_need(w, L + nm["input_norm"], pre)), qkv_w=fin(_shard_qkv(m, q, k, v)),
                          o_w=fin(cols(o_w)), post_norm=fin(_get(w, L + nm["post_norm"], pre)) if nm.get("post_norm") else None,
                          gate_up_w=None, down_w=None, qkv_b=fin(qkv_b))
        if o_b is not None:
            lw.o_b = fin(o_b if rk == 0 else torch.zeros_like(o_b))
        if nm.get("input_norm_b"):
            lw.input_norm_b = fin(_get(w, L + nm["input_norm_b"], pre))
        if nm.get("post_norm_b") and lw.post_norm is not None:
            lw.post_norm_b = fin(_get(w, L + nm["post_norm_b"], pre))
        for extra in ("pre_ffn_norm", "post_ffn_norm"):
            if nm.get(extra):
                setattr(lw, extra, fin(_need(w, L + nm[extra], pre)))
        if c.is_moe:
            lw.router_w = fin(_need(w, L + nm["router"], pre))
            E = c.num_local_experts
            el = max(E // ws, 1)                     # expert parallel: rank r owns experts [r*el, (r+1)*el) in full
            mine = range(rk * el, (rk + 1) * el) if el < E else range(E)
            w13, w2 = [], []
            if nm.get("experts_stacked"):
                P = L + nm["experts_stacked"]
                I = c.intermediate_size
                w1s, v1s, w2s = (dense(_need(w, P + n, pre)).view(E, I, -1) for n in ("w1", "v1", "w2"))
                w13 = [torch.cat([w1s[e], v1s[e]], 0) for e in mine]
                w2 = [w2s[e].t() for e in mine]
            for e in (mine if not nm.get("experts_stacked") else ()):
                P = L + nm["expert"].format(e=e)
                w13.append(_cat0([_need(w, P + "w1.weight", pre), _need(w, P + "w3.weight", pre)]))
                w2.append(_need(w, P + "w2.weight", pre))
            if all(isinstance(t, GroupQuantWeight) for t in w13 + w2):
                # a GPTQ / AWQ checkpoint: every expert stays packed, one matrix each
                lw.experts_w13, lw.experts_w2 = [fin(t) for t in w13], [fin(t) for t in w2]
            else:
                lw.experts_w13 = fin(torch.stack([dense(t) for t in w13]))
                lw.experts_w2 = fin(torch.stack([dense(t) for t in w2]))
        else:
            if nm.get("gate_up"):
                gu = lin(L + nm["gate_up"])
                I = gu.shape[0] // 2
                lw.gate_up_w = fin(_cat0([rows(gu[:I]), rows(gu[I:])]))
            elif nm.get("gate"):
                lw.gate_up_w = fin(_cat0([rows(lin(L + nm["gate"])), rows(lin(L + nm["up"]))]))
                gb, ub = bias(L + nm["gate"]), bias(L + nm["up"])
                if gb is not None and ub is not None:      # llama / granite with mlp_bias
                    lw.gate_up_b = fin(torch.cat([rows(gb), rows(ub)], 0))
            else:
                lw.gate_up_w = fin(rows(lin(L + nm["up"])))
                ub = bias(L + nm["up"])
                if ub is not None:
                    lw.gate_up_b = fin(rows(ub))
            lw.down_w = fin(cols(lin(L + nm["down"])))
            db = bias(L + nm["down"])
            if db is not None:
                lw.down_b = fin(db if rk == 0 else torch.zeros_like(db))
        m.layers.append(lw)
    if any(isinstance(getattr(lw, n, None), (GroupQuantWeight, list)) for lw in m.layers
           for n in ("qkv_w", "o_w", "gate_up_w", "down_w", "experts_w13")):
        m.quantized = (getattr(w, "quant", None) or {}).get("quant_method", "int4")
        m._native = None


def export_hf_state_dict(m: DecoderModel) -> Dict[str, torch.Tensor]:
    """Inverse of the loader for llama-like architectures at TP=1 (tests build HF oracles from it, and the
    static adapter merge writes checkpoints with it)."""
    assert m.tp.world_size == 1
    c = m.config
    nm = NAME_MAPS[c.model_type]
    if nm.get("qkv") or nm.get("conv1d"):
        raise NotImplementedError("export is implemented for separately stored q/k/v projections")
    sd = {nm["embed"]: m.embed, nm["final_norm"]: m.final_norm}
    if not c.tie_word_embeddings:
        sd[nm["lm_head"]] = m.lm_head
    qs, kvs = m.q_size, m.kv_size
    for i, lw in enumerate(m.layers):
        L = nm["layer"].format(i=i)
        sd[L + nm["input_norm"]] = lw.input_norm
        if lw.post_norm is not None and nm.get("post_norm"):
            sd[L + nm["post_norm"]] = lw.post_norm
        sd[L + nm["q"] + ".weight"] = lw.qkv_w[:qs]
        sd[L + nm["k"] + ".weight"] = lw.qkv_w[qs:qs + kvs]
        sd[L + nm["v"] + ".weight"] = lw.qkv_w[qs + kvs:]
        if lw.qkv_b is not None:
            sd[L + nm["q"] + ".bias"] = lw.qkv_b[:qs]
            sd[L + nm["k"] + ".bias"] = lw.qkv_b[qs:qs + kvs]
            sd[L + nm["v"] + ".bias"] = lw.qkv_b[qs + kvs:]
        sd[L + nm["o"] + ".weight"] = lw.o_w
        for extra in ("pre_ffn_norm", "post_ffn_norm"):
            if nm.get(extra) and getattr(lw, extra) is not None:
                sd[L + nm[extra]] = getattr(lw, extra)
        if c.is_moe:
            sd[L + nm["router"]] = lw.router_w
            I = c.intermediate_size
            for e in range(c.num_local_experts):
                P = L + nm["expert"].format(e=e)
                sd[P + "w1.weight"] = lw.experts_w13[e, :I]
                sd[P + "w3.weight"] = lw.experts_w13[e, I:]
                sd[P + "w2.weight"] = lw.experts_w2[e]
        else:
            I = m.inter
            sd[L + nm["gate"] + ".weight"] = lw.gate_up_w[:I]
            sd[L + nm["up"] + ".weight"] = lw.gate_up_w[I:]
            sd[L + nm["down"] + ".weight"] = lw.down_w
    return {k: v.detach().cpu().contiguous().clone() for k, v in sd.items()}
