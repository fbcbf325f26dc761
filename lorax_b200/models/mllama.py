"""Mllama (Llama 3.2 Vision): a tiled vision encoder whose output the text decoder reads through gated cross-attention layers.

The reference serves it as `MllamaCausalLM` (`server/lorax_server/models/mllama.py`, model code
`custom_modeling/mllama.py`): the vision tower runs once per request, its projected output becomes the cross-attention
states, and every fifth or so layer of the 40-layer text model is a cross-attention block instead of a self-attention block.
Same structure here:

1. `pixel_values(image)`: the image is resized into the best canvas of up to `max_num_tiles` tiles (the arrangement that needs
   the least up-scaling, else the least down-scaling), padded bottom / right, normalised and cut into tiles;
2. `vision_features(tiles, aspect_ratio_id, num_tiles)`: patch convolution, gated tile and position embeddings, the local
   encoder (whose chosen intermediate states are kept), the gated global encoder, all concatenated -> projector
   -> `[max_num_tiles * (patches + 1), hidden]` cross-attention states;
3. the text model: Llama self-attention layers with RoPE and a per-request key / value store, and cross-attention layers
   (per-head RMS-normed q and k, tanh gates on the attention and MLP branches) whose keys and values are computed once from
   the states.  A token attends to the tiles of the last `<|image|>` token at or before it; a token in front of every image
   has its cross-attention MLP branch switched off.  A prompt without an image skips the cross-attention layers.

Requests keep their own state (the decoding path of the encoder-decoder runtime): cross-attention keys / values are per
request and never change, so they do not belong in the paged cache.  The model runs as PyTorch ops; adapters are not applied.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..ops import reference as ref
from ..parallel.tp import TensorParallel
from ..utils.weights import AbstractWeights

IMAGE_MEAN = (0.48145466, 0.4578275, 0.40821073)
IMAGE_STD = (0.26862954, 0.26130258, 0.27577711)


@dataclass
class MllamaVisionConfig:
    hidden_size: int = 1280
    hidden_act: str = "gelu"
    num_hidden_layers: int = 32
    num_global_layers: int = 8
    attention_heads: int = 16
    num_channels: int = 3
    intermediate_size: int = 5120
    vision_output_dim: int = 7680
    image_size: int = 448
    patch_size: int = 14
    norm_eps: float = 1e-5
    max_num_tiles: int = 4
    intermediate_layers_indices: List[int] = field(default_factory=lambda: [3, 7, 15, 23, 30])
    supported_aspect_ratios: Optional[List[List[int]]] = None

    @classmethod
    def from_dict(cls, d: dict) -> "MllamaVisionConfig":
        return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__ and v is not None})

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2 + 1

    @property
    def aspect_ratios(self) -> List[Tuple[int, int]]:
        if self.supported_aspect_ratios:
            return [tuple(a) for a in self.supported_aspect_ratios]
        return [(w, h) for w in range(1, self.max_num_tiles + 1) for h in range(1, self.max_num_tiles + 1) if w * h <= self.max_num_tiles]


@dataclass
class MllamaTextConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    hidden_act: str = "silu"
    num_hidden_layers: int = 40
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    intermediate_size: int = 14336
    rope_theta: float = 500000.0
    rope_scaling: Optional[dict] = None
    rms_norm_eps: float = 1e-5
    max_position_embeddings: int = 131072
    cross_attention_layers: List[int] = field(default_factory=lambda: [3, 8, 13, 18, 23, 28, 33, 38])
    eos_token_id: object = 128001
    pad_token_id: Optional[int] = 128004
    tie_word_embeddings: bool = False

    @classmethod
    def from_dict(cls, d: dict) -> "MllamaTextConfig":
        kw = {k: v for k, v in d.items() if k in cls.__dataclass_fields__ and v is not None}
        rp = d.get("rope_parameters")          # newer exports keep theta and the scaling in one dict
        if isinstance(rp, dict):
            kw.setdefault("rope_theta", rp.get("rope_theta", 500000.0))
            if rp.get("rope_type", "default") != "default":
                kw.setdefault("rope_scaling", rp)
        return cls(**kw)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


@dataclass
class MllamaConfig:
    vision: MllamaVisionConfig
    text: MllamaTextConfig
    image_token_index: int = 128256
    model_type: str = "mllama"

    @classmethod
    def from_dict(cls, d: dict) -> "MllamaConfig":
        return cls(MllamaVisionConfig.from_dict(d.get("vision_config", {})), MllamaTextConfig.from_dict(d.get("text_config", {})),
                   image_token_index=d.get("image_token_index", 128256))

    # what the generic runtime reads
    @property
    def eos_token_id(self):
        e = self.text.eos_token_id
        return e[0] if isinstance(e, (list, tuple)) else e

    @property
    def pad_token_id(self):
        return self.text.pad_token_id if self.text.pad_token_id is not None else self.eos_token_id


# ------------------------------------------------------------------------------------------------ image geometry
def optimal_canvas(height: int, width: int, max_tiles: int, tile: int) -> Tuple[int, int]:
    """(canvas height, canvas width): the tile arrangement that needs the least up-scaling; if every arrangement is smaller than
    the image, the one that needs the least down-scaling; ties go to the smaller area."""
    cands = [(a * tile, b * tile) for a in range(1, max_tiles + 1) for b in range(1, max_tiles + 1) if a * b <= max_tiles]
    scales = [min(ch / height, cw / width) for ch, cw in cands]
    up = [s for s in scales if s >= 1]
    pick = min(up) if up else max(s for s in scales if s < 1)
    best = [c for c, s in zip(cands, scales) if s == pick]
    return min(best, key=lambda c: c[0] * c[1])


def fit_to_canvas(height: int, width: int, canvas_h: int, canvas_w: int, tile: int) -> Tuple[int, int]:
    """Size of the image inside the canvas: aspect ratio kept, never smaller than a tile along the limiting side."""
    tw = min(max(width, tile), canvas_w)
    th = min(max(height, tile), canvas_h)
    sh, sw = th / height, tw / width
    if sw < sh:
        return min(math.floor(height * sw) or 1, th), tw
    return th, min(math.floor(width * sh) or 1, tw)


def cross_attention_spans(ids: Sequence[int], image_token: int) -> List[Tuple[int, int]]:
    """For every `<|image|>` token the half-open range of positions whose tokens read that image: up to the next image token,
    the last one to the end of the sequence (-1); image tokens that directly follow each other all reach as far as the last."""
    locs = [i for i, t in enumerate(ids) if t == image_token]
    if not locs:
        return []
    if len(locs) == 1:
        return [(locs[0], -1)]
    spans = [[a, b] for a, b in zip(locs[:-1], locs[1:])] + [[locs[-1], len(ids)]]
    end = spans[-1][1]
    for sp in reversed(spans):
        if sp[0] == sp[1] - 1:
            sp[1] = end
        end = sp[1]
    spans[-1][1] = -1 if spans[-1][1] == len(ids) else spans[-1][1]
    return [(a, b if b != len(ids) else -1) for a, b in spans]


class MllamaState:
    """Decoding state of one request."""

    def __init__(self, ids: Sequence[int]):
        self.pending: Optional[List[int]] = list(ids)      # tokens not yet run through the text model (the prompt at first)
        self.position = 0                                 # bookkeeping of the runtime (tokens emitted)
        self.cached = 0                                   # tokens in the self-attention store
        self.last_token = int(ids[-1]) if len(ids) else 0
        self.k: dict = {}                                 # layer -> [kv heads, tokens, head dim]
        self.v: dict = {}
        self.cross_k: dict = {}                           # layer -> [kv heads, vision tokens, head dim]; empty: no image
        self.cross_v: dict = {}
        self.spans: List[Tuple[int, int]] = []            # per image: positions that read it
        self.tiles: List[int] = []                        # per image: valid tiles


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class MllamaModel:
    def __init__(self, config: MllamaConfig, device="cpu", dtype=torch.float32):
        self.config = config
        self.device, self.dtype = torch.device(device), dtype
        self.tp = TensorParallel.single()
        self.vw: dict = {}
        self.tw: dict = {}
        t = config.text
        self.cos_sin = ref.rope_cache(t.head_dim, min(t.max_position_embeddings, 8192), t.rope_theta, t.rope_scaling, device=self.device)

    # ------------------------------------------------------------------ loading
    @classmethod
    def from_weights(cls, config: MllamaConfig, w: AbstractWeights, device="cpu", dtype=torch.float32) -> "MllamaModel":
        m = cls(config, device, dtype)
        names = list(w.keys())

        def prefix_of(suffix):
            hits = [k for k in names if k.endswith(suffix)]
            if not hits:
                raise KeyError(f"no tensor ending in {suffix}")
            return min(hits, key=len)[: -len(suffix)]

        def get(name):
            return w.get_tensor(name).to(dtype).to(m.device).contiguous()
        vp = prefix_of("patch_embedding.weight")
        v, g = config.vision, m.vw
        g["patch"], g["cls"] = get(vp + "patch_embedding.weight"), get(vp + "class_embedding")
        g["pos_gate"], g["pos"] = get(vp + "gated_positional_embedding.gate"), get(vp + "gated_positional_embedding.embedding")
        g["pos_tile"] = get(vp + "gated_positional_embedding.tile_embedding.weight")
        for k in ("pre", "post"):
            g[k + "_tile"], g[k + "_tile_gate"] = get(vp + f"{k}_tile_positional_embedding.embedding.weight"), get(vp + f"{k}_tile_positional_embedding.gate")
            g["ln_" + k + "_w"], g["ln_" + k + "_b"] = get(vp + f"layernorm_{k}.weight"), get(vp + f"layernorm_{k}.bias")

        def vlayer(p, gated):
            d = {k: get(p + n) for k, n in (
                ("ln1_w", "input_layernorm.weight"), ("ln1_b", "input_layernorm.bias"), ("ln2_w", "post_attention_layernorm.weight"),
                ("ln2_b", "post_attention_layernorm.bias"), ("q", "self_attn.q_proj.weight"), ("k", "self_attn.k_proj.weight"),
                ("v", "self_attn.v_proj.weight"), ("o", "self_attn.o_proj.weight"), ("fc1_w", "mlp.fc1.weight"), ("fc1_b", "mlp.fc1.bias"),
                ("fc2_w", "mlp.fc2.weight"), ("fc2_b", "mlp.fc2.bias"))}
            if gated:
                d["gate_attn"], d["gate_ffn"] = get(p + "gate_attn"), get(p + "gate_ffn")
            return d
        g["local"] = [vlayer(vp + f"transformer.layers.{i}.", False) for i in range(v.num_hidden_layers)]
        g["global"] = [vlayer(vp + f"global_transformer.layers.{i}.", True) for i in range(v.num_global_layers)]
        pj = prefix_of("multi_modal_projector.weight")
        g["proj_w"], g["proj_b"] = get(pj + "multi_modal_projector.weight"), get(pj + "multi_modal_projector.bias")
        # text
        t, tw = config.text, m.tw
        tp_ = prefix_of("embed_tokens.weight")
        tw["embed"], tw["norm"] = get(tp_ + "embed_tokens.weight"), get(tp_ + "norm.weight")
        head = [k for k in names if k.endswith("lm_head.weight")]
        tw["lm_head"] = get(head[0]) if head else tw["embed"][: t.vocab_size]
        tw["layers"] = []
        for i in range(t.num_hidden_layers):
            p = tp_ + f"layers.{i}."
            d = {"in_norm": get(p + "input_layernorm.weight"), "post_norm": get(p + "post_attention_layernorm.weight"),
                 "gate": get(p + "mlp.gate_proj.weight"), "up": get(p + "mlp.up_proj.weight"), "down": get(p + "mlp.down_proj.weight")}
            if i in t.cross_attention_layers:
                a = p + "cross_attn."
                d.update(cross=True, q=get(a + "q_proj.weight"), k=get(a + "k_proj.weight"), v=get(a + "v_proj.weight"), o=get(a + "o_proj.weight"),
                         q_norm=get(a + "q_norm.weight"), k_norm=get(a + "k_norm.weight"), gate_attn=get(p + "cross_attn_attn_gate"),
                         gate_mlp=get(p + "cross_attn_mlp_gate"))
            else:
                a = p + "self_attn."
                d.update(cross=False, q=get(a + "q_proj.weight"), k=get(a + "k_proj.weight"), v=get(a + "v_proj.weight"), o=get(a + "o_proj.weight"))
            tw["layers"].append(d)
        return m

    # ------------------------------------------------------------------ step 1: pixels
    def pixel_values(self, image) -> Tuple[torch.Tensor, int, int]:
        """PIL image -> (tiles [max_num_tiles, 3, S, S] normalised fp32 with unused tiles zero, aspect-ratio id, valid tiles)."""
        import numpy as np
        v = self.config.vision
        S = v.image_size
        image = image.convert("RGB")
        w0, h0 = image.size
        ch, cw = optimal_canvas(h0, w0, v.max_num_tiles, S)
        nh, nw = fit_to_canvas(h0, w0, ch, cw, S)
        arr = torch.from_numpy(np.asarray(image, dtype=np.float32)).permute(2, 0, 1)[None]          # [1, 3, h, w] in 0..255
        arr = F.interpolate(arr, size=(nh, nw), mode="bilinear", antialias=True, align_corners=False)[0]
        arr = arr.round().clamp_(0, 255)                   # the processor resizes 8-bit images
        canvas = torch.zeros(3, ch, cw)
        canvas[:, :nh, :nw] = arr
        canvas = canvas / 255.0
        mean = torch.tensor(IMAGE_MEAN).view(3, 1, 1)
        std = torch.tensor(IMAGE_STD).view(3, 1, 1)
        canvas = (canvas - mean) / std
        th, tw_ = ch // S, cw // S
        tiles = canvas.view(3, th, S, tw_, S).permute(1, 3, 0, 2, 4).reshape(th * tw_, 3, S, S)
        out = torch.zeros(v.max_num_tiles, 3, S, S)
        out[: th * tw_] = tiles
        return out, v.aspect_ratios.index((th, tw_)) + 1, th * tw_

    # ------------------------------------------------------------------ step 2: vision tower
    def _vision_layer(self, x, l, mask, gated: bool):
        v = self.config.vision
        nh, d = v.attention_heads, v.hidden_size // v.attention_heads
        h = F.layer_norm(x, (v.hidden_size,), l["ln1_w"], l["ln1_b"], v.norm_eps)
        q = F.linear(h, l["q"]).view(*h.shape[:2], nh, d).transpose(1, 2)
        k = F.linear(h, l["k"]).view(*h.shape[:2], nh, d).transpose(1, 2)
        val = F.linear(h, l["v"]).view(*h.shape[:2], nh, d).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, val, attn_mask=mask).transpose(1, 2).reshape(*h.shape[:2], -1)
        a = F.linear(a, l["o"])
        x = x + (torch.tanh(l["gate_attn"]) * a if gated else a)
        h = F.layer_norm(x, (v.hidden_size,), l["ln2_w"], l["ln2_b"], v.norm_eps)
        h = F.linear(F.gelu(F.linear(h, l["fc1_w"], l["fc1_b"])), l["fc2_w"], l["fc2_b"])
        return x + (torch.tanh(l["gate_ffn"]) * h if gated else h)

    def vision_features(self, tiles: torch.Tensor, aspect_ratio_id: int, num_tiles: int) -> torch.Tensor:
        """Tiles of one image -> cross-attention states [max_num_tiles * (patches + 1), text hidden]."""
        v, g = self.config.vision, self.vw
        nt, H, P = v.max_num_tiles, v.hidden_size, v.num_patches
        x = F.conv2d(tiles.to(self.dtype).to(self.device), g["patch"], None, stride=v.patch_size).flatten(2).transpose(1, 2)   # [tiles, P-1, H]
        x = x + (g["pre_tile"][aspect_ratio_id].view(nt, 1, H) * torch.tanh(g["pre_tile_gate"]))
        x = torch.cat([g["cls"].view(1, 1, H).expand(nt, 1, H), x], 1)                                                   # [tiles, P, H]
        x = x + (1 - torch.tanh(g["pos_gate"])) * g["pos"].view(1, P, H)
        x = x + torch.tanh(g["pos_gate"]) * g["pos_tile"][aspect_ratio_id].view(nt, P, H)
        x = F.layer_norm(x, (H,), g["ln_pre_w"], g["ln_pre_b"], 1e-5)
        pad = (8 - P % 8) % 8
        x = F.pad(x, (0, 0, 0, pad))
        Pp = P + pad
        # padding tiles and padding patches neither attend nor are attended to (among themselves they are left alone)
        live = torch.zeros(nt, Pp, dtype=torch.float32, device=self.device)
        live[:num_tiles] = 1
        live[:, P:] = 0
        dead = (1 - live).reshape(nt * Pp, 1)
        mask = (dead @ dead.t() * torch.finfo(self.dtype).min).to(self.dtype)[None, None]
        x = x.reshape(1, nt * Pp, H)
        inter = []
        for i, l in enumerate(g["local"]):
            x = self._vision_layer(x, l, mask, False)
            if i in v.intermediate_layers_indices:
                inter.append(x)
        x = F.layer_norm(x, (H,), g["ln_post_w"], g["ln_post_b"], 1e-5)
        x = x.reshape(nt, Pp, H) + (g["post_tile"][aspect_ratio_id].view(nt, 1, H) * torch.tanh(g["post_tile_gate"]))
        x = x.reshape(1, nt * Pp, H)
        for l in g["global"]:
            x = self._vision_layer(x, l, mask, True)
        x = x.reshape(nt, Pp, H)[:, :P]
        inter = torch.stack(inter, -1).reshape(nt, Pp, -1)[:, :P]
        x = torch.cat([x, inter], -1)                                                                   # [tiles, P, vision_output_dim]
        return F.linear(x, g["proj_w"], g["proj_b"]).reshape(nt * P, -1)

    # ------------------------------------------------------------------ step 3: text model
    def encode(self, ids: Sequence[int], images: Sequence[Tuple[torch.Tensor, int, int]] = ()) -> MllamaState:
        """A request's state: the cross-attention keys / values of its images; the prompt itself runs in the first
        `decode_step`."""
        t = self.config.text
        st = MllamaState(ids)
        st.spans = cross_attention_spans(list(ids), self.config.image_token_index)
        if images:
            if len(images) != len(st.spans):
                raise ValueError(f"the prompt has {len(st.spans)} image tokens and {len(images)} images")
            states = torch.cat([self.vision_features(*im) for im in images], 0)                         # [images * tiles * P, hidden]
            st.tiles = [im[2] for im in images]
            nkv, d = t.num_key_value_heads, t.head_dim
            for li, L in enumerate(self.tw["layers"]):
                if L["cross"]:
                    k = F.linear(states, L["k"]).view(-1, nkv, d).transpose(0, 1)
                    st.cross_k[li] = _rms(k, L["k_norm"], t.rms_norm_eps)
                    st.cross_v[li] = F.linear(states, L["v"]).view(-1, nkv, d).transpose(0, 1)
        return st

    def _cross_mask(self, st: MllamaState, positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Additive mask [tokens, vision tokens] and the per-token switch of the cross-attention MLP branch."""
        v = self.config.vision
        per_image = v.max_num_tiles * v.num_patches
        n_vis = per_image * len(st.tiles)
        allow = torch.zeros(positions.shape[0], n_vis, dtype=torch.bool, device=self.device)
        for i, ((a, b), nt) in enumerate(zip(st.spans, st.tiles)):
            rows = (positions >= a) & ((positions < b) if b >= 0 else torch.ones_like(positions, dtype=torch.bool))
            allow[rows, i * per_image: i * per_image + nt * v.num_patches] = True
        row_ok = allow.any(-1)
        mask = torch.zeros(positions.shape[0], n_vis, dtype=self.dtype, device=self.device)
        mask.masked_fill_(~allow, torch.finfo(self.dtype).min)
        mask[~row_ok] = 0                                  # a token in front of every image: unmasked attention, MLP branch off
        return mask, row_ok.to(self.dtype)

    def _text(self, st: MllamaState, ids: Sequence[int]) -> torch.Tensor:
        """Runs `ids` on top of the request's state; returns the logits of the last token [vocab]."""
        t, tw = self.config.text, self.tw
        nh, nkv, d = t.num_attention_heads, t.num_key_value_heads, t.head_dim
        T = len(ids)
        x = tw["embed"][torch.tensor(list(ids), device=self.device)]
        pos = torch.arange(st.cached, st.cached + T, device=self.device)
        cs = self.cos_sin[pos]
        cos, sin = cs[:, : d // 2], cs[:, d // 2:]
        scale = d ** -0.5
        have_images = bool(st.cross_k)
        if have_images:
            cmask, row_ok = self._cross_mask(st, pos)
        for li, L in enumerate(tw["layers"]):
            if L["cross"]:
                if not have_images:
                    continue
                h = _rms(x, L["in_norm"], t.rms_norm_eps)
                q = _rms(F.linear(h, L["q"]).view(T, nh, d), L["q_norm"], t.rms_norm_eps).transpose(0, 1)              # [nh, T, d]
                k = st.cross_k[li].repeat_interleave(nh // nkv, 0)
                val = st.cross_v[li].repeat_interleave(nh // nkv, 0)
                s = (q.float() @ k.float().transpose(1, 2)) * scale + cmask.float()[None]
                a = (torch.softmax(s, -1) @ val.float()).to(x.dtype).transpose(0, 1).reshape(T, nh * d)
                x = x + torch.tanh(L["gate_attn"]) * F.linear(a, L["o"])
                h = _rms(x, L["post_norm"], t.rms_norm_eps)
                h = F.linear(F.silu(F.linear(h, L["gate"])) * F.linear(h, L["up"]), L["down"])
                x = x + torch.tanh(L["gate_mlp"]) * (h * row_ok[:, None])
                continue
            h = _rms(x, L["in_norm"], t.rms_norm_eps)
            q = ref.apply_rope(F.linear(h, L["q"]).view(T, nh, d), cos, sin, d).transpose(0, 1)
            k = ref.apply_rope(F.linear(h, L["k"]).view(T, nkv, d), cos, sin, d).transpose(0, 1)
            val = F.linear(h, L["v"]).view(T, nkv, d).transpose(0, 1)
            if li in st.k:
                k, val = torch.cat([st.k[li], k], 1), torch.cat([st.v[li], val], 1)
            st.k[li], st.v[li] = k, val
            kk, vv = k.repeat_interleave(nh // nkv, 0), val.repeat_interleave(nh // nkv, 0)
            s = (q.float() @ kk.float().transpose(1, 2)) * scale                                   # [nh, T, keys]
            keys = torch.arange(k.shape[1], device=self.device)
            s = s.masked_fill(keys[None, None, :] > pos[None, :, None], float("-inf"))
            a = (torch.softmax(s, -1) @ vv.float()).to(x.dtype).transpose(0, 1).reshape(T, nh * d)
            x = x + F.linear(a, L["o"])
            h = _rms(x, L["post_norm"], t.rms_norm_eps)
            x = x + F.linear(F.silu(F.linear(h, L["gate"])) * F.linear(h, L["up"]), L["down"])
        st.cached += T
        return F.linear(_rms(x[-1:], tw["norm"], t.rms_norm_eps), tw["lm_head"])[0].float()

    def decode_step(self, states: Sequence[MllamaState]) -> torch.Tensor:
        """One step for every request: the whole prompt on a request's first step, its last token afterwards.  -> [B, vocab]."""
        out = []
        for st in states:
            ids = st.pending if st.pending is not None else [st.last_token]
            out.append(self._text(st, ids))
            st.pending = None
        return torch.stack(out, 0)
