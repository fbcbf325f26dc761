"""Medusa speculation heads as an adapter type.

A Medusa adapter adds `medusa_num_heads` small heads on top of the base model's last hidden state h (after the final norm).
Head i guesses the token i + 2 positions ahead; the guesses of one step are verified by the next forward pass, which scores
[last token, guess 1, guess 2, ...] in one ragged pass and keeps the longest prefix the model agrees with.

Two layouts exist (reference: `server/lorax_server/adapters/medusa.py:102-214`):

* v1  every head is `medusa_num_layers` residual blocks  x <- x + silu(W x + b)  followed by its own vocabulary projection
      (`{i}.{l}.linear.weight / .bias`, `{i}.{L}.weight`);
* v2  one residual block per head and the base model's lm_head shared by all heads: all blocks are one stacked GEMM
      [heads * H, H], and the lm_head runs once over the stacked rows [h, h + r_1, ..., h + r_n].

The checkpoint is `medusa_lm_head.safetensors` (or `.pt`) next to a `config.json` with `medusa_num_heads`,
`medusa_num_layers` and optionally `version`.  A directory that also holds a PEFT LoRA (`adapter_config.json`) is the
reference's Medusa + LoRA combination (`adapters/medusa_lora.py`): both parts load under one adapter index.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch

MEDUSA_FILES = ("medusa_lm_head.safetensors", "medusa_lm_head.pt")


@dataclass
class MedusaConfig:
    base_model_name_or_path: str
    medusa_num_heads: int
    medusa_num_layers: int
    version: float = 1.0

    @classmethod
    def load(cls, config: dict) -> "MedusaConfig":
        return cls(base_model_name_or_path=config.get("base_model_name_or_path", ""), medusa_num_heads=int(config["medusa_num_heads"]),
                   medusa_num_layers=int(config.get("medusa_num_layers", 1)), version=float(config.get("version", 1)))


def is_medusa_dir(path: str) -> bool:
    cfg = os.path.join(path, "config.json")
    if not os.path.exists(cfg) or not any(os.path.exists(os.path.join(path, f)) for f in MEDUSA_FILES):
        return False
    with open(cfg) as f:
        return "medusa_num_heads" in json.load(f)


def load_medusa_adapter(path: str) -> Tuple[MedusaConfig, Dict[str, torch.Tensor]]:
    with open(os.path.join(path, "config.json")) as f:
        cfg = MedusaConfig.load(json.load(f))
    st = os.path.join(path, MEDUSA_FILES[0])
    if os.path.exists(st):
        from safetensors.torch import load_file
        tensors = load_file(st)
    else:
        tensors = torch.load(os.path.join(path, MEDUSA_FILES[1]), map_location="cpu", weights_only=True)
    return cfg, {k: v for k, v in tensors.items()}


class MedusaHeads:
    """The heads of one Medusa adapter on one device.  Replicated on every tensor-parallel rank (heads * H * H elements)."""

    def __init__(self, config: MedusaConfig, tensors: Dict[str, torch.Tensor], device, dtype):
        self.config = config
        n, L = config.medusa_num_heads, config.medusa_num_layers
        self.shared_head = not (L > 1 or f"0.{L}.weight" in tensors)          # v2: the base lm_head serves every head

        def t(name):
            if name not in tensors:
                raise KeyError(f"medusa adapter lacks tensor {name}")
            return tensors[name].to(dtype).to(device).contiguous()
        if self.shared_head:
            # all residual blocks as one GEMM: rows [i * H, (i + 1) * H) belong to head i
            self.w = torch.cat([t(f"{i}.0.linear.weight") for i in range(n)], 0)
            self.b = torch.cat([t(f"{i}.0.linear.bias") for i in range(n)], 0)
        else:
            self.blocks = [[(t(f"{i}.{l}.linear.weight"), t(f"{i}.{l}.linear.bias")) for l in range(L)] for i in range(n)]
            self.out = [t(f"{i}.{L}.weight") for i in range(n)]
        self.num_heads = n
        self.nbytes = sum(v.numel() * v.element_size() for v in tensors.values())

    @property
    def speculative_tokens(self) -> int:
        return self.num_heads

    def hidden_rows(self, h: torch.Tensor) -> Optional[torch.Tensor]:
        """v2 only: [R, H] -> [R * heads, H], the rows the shared lm_head has to score (h + residual of each head)."""
        if not self.shared_head:
            return None
        R, H = h.shape
        y = torch.addmm(self.b.float(), h.float(), self.w.float().t())         # [R, heads * H]
        res = torch.nn.functional.silu(y).view(R, self.num_heads, H)
        return (h.float().unsqueeze(1) + res).to(h.dtype).reshape(R * self.num_heads, H)

    def propose(self, h: torch.Tensor, lm_head: Callable[[torch.Tensor], torch.Tensor]) -> torch.Tensor:
        """Greedy guesses [R, heads] (int64) from last hidden states h [R, H]; `lm_head` maps [M, H] to full-vocabulary
        logits [M, V] (it gathers the vocabulary shards under tensor parallelism)."""
        R = h.shape[0]
        if self.shared_head:
            logits = lm_head(self.hidden_rows(h))
            return logits.float().argmax(-1).view(R, self.num_heads)
        outs = []
        for blocks, out in zip(self.blocks, self.out):
            x = h.float()
            for w, b in blocks:
                x = x + torch.nn.functional.silu(torch.addmm(b.float(), x, w.float().t()))
            outs.append((x @ out.float().t()).argmax(-1))
        return torch.stack(outs, 1)


def random_medusa_tensors(hidden: int, heads: int, layers: int = 1, vocab: int = 0, seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Random heads of the right shapes (tests, benchmarks).  `vocab > 0` adds the per-head projections of the v1 layout."""
    g = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for i in range(heads):
        for l in range(layers):
            out[f"{i}.{l}.linear.weight"] = torch.randn(hidden, hidden, generator=g) * std
            out[f"{i}.{l}.linear.bias"] = torch.randn(hidden, generator=g) * std
        if vocab:
            out[f"{i}.{layers}.weight"] = torch.randn(vocab, hidden, generator=g) * std
    return out
