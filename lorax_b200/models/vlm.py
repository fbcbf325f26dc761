"""Vision-language serving: LLaVA-NeXT (CLIP or SigLIP vision tower + two-layer projector + any-resolution tiling) in front of
the paged decoder.

The reference serves LLaVA-NeXT through `VlmCausalLM` (`server/lorax_server/models/vlm_causal_lm.py`, model code
`custom_modeling/llava_next.py`, `clip.py`, `siglip.py`), with the router expanding every image into as many `<image>` tokens as the model
will produce features (`router/src/config.rs:6-190`, `validation.rs:498-638`).  The same three steps here:

1. `num_image_features(height, width)`: how many rows of the prompt an image takes;
2. `pixel_values(image)`: the image resized to the best-fitting grid resolution and cut into tiles of the tower's input size,
   plus the whole image at tile size, normalised;
3. `image_features(tiles, (height, width))`: tower -> hidden state of the chosen layer without the class token -> projector
   -> tiles laid out on their grid, padding cut away, an `image_newline` vector after every row of features -> `[n, hidden]`.

The rows replace the embeddings of the `<image>` placeholders in the decoder's prefill (`PrefillItem.embeds`); everything after
that (paged attention, LoRA on the language model, sampling) is the ordinary decoder path.  The tower runs as PyTorch ops: it is
a few hundred megaflops per tile, once per request.
"""

from __future__ import annotations

import base64
import io
import math
import re
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from ..utils.weights import AbstractWeights
from .decoder import DecoderModel

VLM_TYPES = ("llava_next",)
CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)
IMAGE_MARKDOWN = re.compile(r"!\[\]\(([^)]+)\)")


@dataclass
class ClipVisionConfig:
    hidden_size: int = 1024
    intermediate_size: int = 4096
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    image_size: int = 336
    patch_size: int = 14
    layer_norm_eps: float = 1e-5
    hidden_act: str = "quick_gelu"
    # "clip_vision_model": class token in front of the patches, LayerNorm before the encoder, patch convolution without bias.
    # "siglip_vision_model" (reference: `custom_modeling/siglip.py`): patches only, no LayerNorm in front, biased convolution.
    model_type: str = "clip_vision_model"

    @classmethod
    def from_dict(cls, d: dict) -> "ClipVisionConfig":
        kw = {k: v for k, v in d.items() if k in cls.__dataclass_fields__ and v is not None}
        if kw.get("model_type") == "siglip_vision_model":
            kw.setdefault("layer_norm_eps", 1e-6)
            kw.setdefault("hidden_act", "gelu_pytorch_tanh")
        return cls(**kw)

    @property
    def is_siglip(self) -> bool:
        return self.model_type == "siglip_vision_model"

    @property
    def extra_tokens(self) -> int:
        """Rows the tower emits per tile besides the patches (CLIP's class token)."""
        return 0 if self.is_siglip else 1


@dataclass
class LlavaNextConfig:
    vision: ClipVisionConfig
    text: ModelConfig
    image_token_index: int = 32000
    vision_feature_layer: int = -2
    vision_feature_select_strategy: str = "default"
    image_grid_pinpoints: List[List[int]] = field(default_factory=lambda: [[336, 672], [672, 336], [672, 672], [1008, 336], [336, 1008]])
    projector_hidden_act: str = "gelu"

    @classmethod
    def from_dict(cls, d: dict) -> "LlavaNextConfig":
        tower = d.get("vision_config", {}).get("model_type", "clip_vision_model")
        if tower not in ("clip_vision_model", "siglip_vision_model"):
            raise NotImplementedError(f"vision tower {tower}: CLIP and SigLIP towers are built")
        kw = {k: d[k] for k in ("image_token_index", "vision_feature_layer", "vision_feature_select_strategy", "image_grid_pinpoints",
                                "projector_hidden_act") if d.get(k) is not None}
        if "image_token_index" not in kw and d.get("image_token_id") is not None:
            kw["image_token_index"] = d["image_token_id"]
        return cls(vision=ClipVisionConfig.from_dict(d.get("vision_config", {})), text=ModelConfig.from_dict(d["text_config"]), **kw)


# ------------------------------------------------------------------------------------------------ geometry
def select_best_resolution(size: Tuple[int, int], candidates: Sequence[Sequence[int]]) -> Tuple[int, int]:
    """(height, width) of the candidate that keeps most of the image's pixels after an aspect-preserving resize and, among
    those, wastes the least area."""
    h0, w0 = size
    best, best_eff, best_waste = None, -1, float("inf")
    for h, w in candidates:
        scale = min(w / w0, h / h0)
        eff = min(int(w0 * scale) * int(h0 * scale), w0 * h0)
        waste = w * h - eff
        if eff > best_eff or (eff == best_eff and waste < best_waste):
            best, best_eff, best_waste = (h, w), eff, waste
    return best


def unpadded_grid(size: Tuple[int, int], grid_hw: Tuple[int, int]) -> Tuple[int, int, int, int]:
    """For features laid out on a grid of `grid_hw` rows x columns that covers the padded image: (first row, rows kept, first
    column, columns kept) of the part that shows the image itself."""
    h0, w0 = size
    gh, gw = grid_hw
    if w0 / h0 > gw / gh:
        new_h = int(round(h0 * (gw / w0), 7))
        pad = (gh - new_h) // 2
        return pad, gh - 2 * pad, 0, gw
    new_w = int(round(w0 * (gh / h0), 7))
    pad = (gw - new_w) // 2
    return 0, gh, pad, gw - 2 * pad


class LlavaNextModel:
    def __init__(self, config: LlavaNextConfig, text: DecoderModel):
        self.config = config
        self.text = text
        self.device, self.dtype = text.device, text.dtype
        self.w = {}
        # normalisation of the pixels: CLIP's statistics, 0.5 / 0.5 for SigLIP (the defaults of their image processors)
        self.image_mean, self.image_std = CLIP_MEAN, CLIP_STD

    # ------------------------------------------------------------------ loading
    @classmethod
    def from_weights(cls, config: LlavaNextConfig, w: AbstractWeights, device, dtype, tp=None, max_positions=None) -> "LlavaNextModel":
        # Where the parts live differs between exports (`language_model.model.*` + `vision_tower.*`, `model.language_model.*` +
        # `model.vision_tower.*`, and mixtures of the two): take the prefixes from the tensors that must exist.
        names = w.keys()

        def prefix_of(suffix):
            hits = [k for k in names if k.endswith(suffix)]
            if not hits:
                raise KeyError(f"no tensor ending in {suffix}")
            return min(hits, key=len)[: -len(suffix)]
        lang = _Prefixed(w, {"model.": prefix_of("embed_tokens.weight"), "lm_head.": prefix_of("lm_head.weight") + "lm_head."
                             if any(k.endswith("lm_head.weight") for k in names) else "lm_head."})
        text = DecoderModel.from_weights(config.text, lang, device, dtype, tp, max_positions=max_positions)
        m = cls(config, text)
        vt = prefix_of("embeddings.position_embedding.weight")
        sig = config.vision.is_siglip
        if sig:
            m.image_mean = m.image_std = (0.5, 0.5, 0.5)
            if config.vision_feature_select_strategy == "default":
                raise ValueError("a SigLIP tower has no class token to drop: vision_feature_select_strategy must be 'full'")
        pj = prefix_of("linear_1.weight")
        nl = prefix_of("image_newline") + "image_newline"

        def get(name):
            return w.get_tensor(name).to(dtype).to(m.device).contiguous()
        g = m.w
        g["patch"], g["pos"] = get(vt + "embeddings.patch_embedding.weight"), get(vt + "embeddings.position_embedding.weight")
        if sig:
            g["patch_b"] = get(vt + "embeddings.patch_embedding.bias")
        else:
            g["cls"] = get(vt + "embeddings.class_embedding")
            g["pre_w"], g["pre_b"] = get(vt + "pre_layrnorm.weight"), get(vt + "pre_layrnorm.bias")
        n_layers = config.vision.num_hidden_layers
        last = n_layers + config.vision_feature_layer + 1 if config.vision_feature_layer < 0 else config.vision_feature_layer
        g["layers"] = []
        for i in range(last):                               # layers past the chosen hidden state are never run
            p = vt + f"encoder.layers.{i}."
            g["layers"].append({k: get(p + n) for k, n in (
                ("ln1_w", "layer_norm1.weight"), ("ln1_b", "layer_norm1.bias"), ("ln2_w", "layer_norm2.weight"), ("ln2_b", "layer_norm2.bias"),
                ("q_w", "self_attn.q_proj.weight"), ("q_b", "self_attn.q_proj.bias"), ("k_w", "self_attn.k_proj.weight"),
                ("k_b", "self_attn.k_proj.bias"), ("v_w", "self_attn.v_proj.weight"), ("v_b", "self_attn.v_proj.bias"),
                ("o_w", "self_attn.out_proj.weight"), ("o_b", "self_attn.out_proj.bias"), ("fc1_w", "mlp.fc1.weight"),
                ("fc1_b", "mlp.fc1.bias"), ("fc2_w", "mlp.fc2.weight"), ("fc2_b", "mlp.fc2.bias"))})
        g["p1_w"], g["p1_b"], g["p2_w"], g["p2_b"] = get(pj + "linear_1.weight"), get(pj + "linear_1.bias"), get(pj + "linear_2.weight"), \
            get(pj + "linear_2.bias")
        g["newline"] = get(nl)
        return m

    # ------------------------------------------------------------------ step 1: how many rows
    def num_image_features(self, height: int, width: int) -> int:
        v = self.config.vision
        side = v.image_size // v.patch_size
        base = side * side + v.extra_tokens - (1 if self.config.vision_feature_select_strategy == "default" else 0)
        bh, bw = select_best_resolution((height, width), self.config.image_grid_pinpoints)
        gh, gw = bh // v.image_size * side, bw // v.image_size * side
        _, rows, _, cols = unpadded_grid((height, width), (gh, gw))
        return base + rows * (cols + 1)

    # ------------------------------------------------------------------ step 2: pixels
    def pixel_values(self, image) -> Tuple[torch.Tensor, Tuple[int, int]]:
        """PIL image -> (tiles [1 + n, 3, S, S] normalised fp32, (height, width) of the original)."""
        from PIL import Image
        v = self.config.vision
        S = v.image_size
        image = image.convert("RGB")
        w0, h0 = image.size
        bh, bw = select_best_resolution((h0, w0), self.config.image_grid_pinpoints)
        scale = min(bw / w0, bh / h0)
        if bw / w0 < bh / h0:
            nw, nh = bw, min(math.ceil(h0 * (bw / w0)), bh)
        else:
            nh, nw = bh, min(math.ceil(w0 * (bh / h0)), bw)
        del scale
        resized = image.resize((nw, nh), Image.BICUBIC)
        canvas = Image.new("RGB", (bw, bh), (0, 0, 0))
        canvas.paste(resized, ((bw - nw) // 2, (bh - nh) // 2))
        tiles = [image.resize((S, S), Image.BICUBIC)]
        for y in range(0, bh, S):
            for x in range(0, bw, S):
                tiles.append(canvas.crop((x, y, x + S, y + S)))
        import numpy as np
        arr = torch.from_numpy(np.stack([np.asarray(t, dtype=np.float32) / 255.0 for t in tiles])).permute(0, 3, 1, 2)
        mean = torch.tensor(self.image_mean).view(1, 3, 1, 1)
        std = torch.tensor(self.image_std).view(1, 3, 1, 1)
        return ((arr - mean) / std).contiguous(), (h0, w0)

    # ------------------------------------------------------------------ step 3: features
    def _tower(self, tiles: torch.Tensor) -> torch.Tensor:
        """[n, 3, S, S] -> hidden state of the chosen layer [n, (1 +) patches, hidden]."""
        v, g = self.config.vision, self.w
        x = F.conv2d(tiles.to(self.dtype).to(self.device), g["patch"], g.get("patch_b"), stride=v.patch_size)   # [n, hidden, side, side]
        x = x.flatten(2).transpose(1, 2)
        if "cls" in g:
            x = torch.cat([g["cls"].view(1, 1, -1).expand(x.shape[0], 1, -1), x], 1) + g["pos"][None]
            x = F.layer_norm(x, (v.hidden_size,), g["pre_w"], g["pre_b"], v.layer_norm_eps)
        else:
            x = x + g["pos"][None]
        nh, d = v.num_attention_heads, v.hidden_size // v.num_attention_heads
        for l in g["layers"]:
            h = F.layer_norm(x, (v.hidden_size,), l["ln1_w"], l["ln1_b"], v.layer_norm_eps)
            q = F.linear(h, l["q_w"], l["q_b"]).view(*h.shape[:2], nh, d).transpose(1, 2)
            k = F.linear(h, l["k_w"], l["k_b"]).view(*h.shape[:2], nh, d).transpose(1, 2)
            val = F.linear(h, l["v_w"], l["v_b"]).view(*h.shape[:2], nh, d).transpose(1, 2)
            a = F.scaled_dot_product_attention(q, k, val).transpose(1, 2).reshape(*h.shape[:2], -1)
            x = x + F.linear(a, l["o_w"], l["o_b"])
            h = F.layer_norm(x, (v.hidden_size,), l["ln2_w"], l["ln2_b"], v.layer_norm_eps)
            h = F.linear(h, l["fc1_w"], l["fc1_b"])
            if v.hidden_act == "quick_gelu":
                h = h * torch.sigmoid(1.702 * h)
            else:
                h = F.gelu(h, approximate="tanh" if v.hidden_act in ("gelu_pytorch_tanh", "gelu_new", "gelu_fast") else "none")
            x = x + F.linear(h, l["fc2_w"], l["fc2_b"])
        return x

    def image_features(self, tiles: torch.Tensor, size: Tuple[int, int]) -> torch.Tensor:
        """Tiles of one image (whole image first) and its original (height, width) -> [num_image_features, hidden]."""
        v, g = self.config.vision, self.w
        x = self._tower(tiles)
        if self.config.vision_feature_select_strategy == "default":
            x = x[:, 1:]
        x = F.linear(x, g["p1_w"], g["p1_b"])
        x = F.gelu(x) if self.config.projector_hidden_act == "gelu" else F.silu(x)
        x = F.linear(x, g["p2_w"], g["p2_b"])                                                       # [n, patches, hidden]
        base, rest = x[0], x[1:]
        if rest.shape[0] == 0:
            return torch.cat([base, g["newline"][None]], 0)
        side = v.image_size // v.patch_size
        bh, bw = select_best_resolution(size, self.config.image_grid_pinpoints)
        th, tw = bh // v.image_size, bw // v.image_size
        grid = rest.view(th, tw, side, side, -1).permute(0, 2, 1, 3, 4).reshape(th * side, tw * side, -1)   # rows x columns of features
        r0, nr, c0, nc = unpadded_grid(size, (th * side, tw * side))
        grid = grid[r0:r0 + nr, c0:c0 + nc]
        grid = torch.cat([grid, g["newline"].view(1, 1, -1).expand(nr, 1, -1)], 1)
        return torch.cat([base, grid.reshape(nr * (nc + 1), grid.shape[-1])], 0)


class _Prefixed(AbstractWeights):
    """View of a checkpoint in which the language model's tensors carry the names a plain decoder checkpoint would use."""

    def __init__(self, inner: AbstractWeights, prefixes: dict):
        self.inner, self.prefixes = inner, prefixes
        self.quant = getattr(inner, "quant", None)
        self.keep_packed = getattr(inner, "keep_packed", True)
        self.dtype = getattr(inner, "dtype", None)

    def _map(self, name: str) -> str:
        for short, full in self.prefixes.items():
            if name.startswith(short):
                return full + name[len(short):]
        return name

    def has_tensor(self, name):
        return self.inner.has_tensor(self._map(name))

    def get_tensor(self, name):
        return self.inner.get_tensor(self._map(name))

    def _raw(self, name):
        return self.inner._raw(self._map(name))


# ------------------------------------------------------------------------------------------------ prompt handling
def load_image(ref: str, timeout: float = 10.0):
    """`data:<mime>;base64,<payload>` or an http(s) URL -> PIL image."""
    from PIL import Image
    if ref.startswith("data:"):
        head, _, payload = ref.partition(",")
        if not head.endswith(";base64"):
            raise ValueError("image data URIs must be base64 encoded")
        return Image.open(io.BytesIO(base64.b64decode(payload)))
    if ref.startswith("http://") or ref.startswith("https://"):
        import urllib.request
        with urllib.request.urlopen(ref, timeout=timeout) as r:
            return Image.open(io.BytesIO(r.read()))
    raise ValueError(f"invalid image content: {ref[:40]}")


def split_prompt(text: str) -> List[Tuple[str, str]]:
    """"a ![](uri) b" -> [("text", "a "), ("image", uri), ("text", " b")] (the reference's chunking, validation.rs:498-638)."""
    out, pos = [], 0
    for m in IMAGE_MARKDOWN.finditer(text):
        if m.start() > pos:
            out.append(("text", text[pos:m.start()]))
        out.append(("image", m.group(1)))
        pos = m.end()
    if pos < len(text):
        out.append(("text", text[pos:]))
    return out
