"""Merging several LoRA adapters into one, per request (`merged_adapters` in the API) or offline.

Strategies and their parameters follow the reference (`server/lorax_server/utils/merges/strategies.py:43-158`,
`utils/merges/utils.py:23-106`, themselves after PEFT's merging utilities):

  linear       weighted sum of the task tensors
  ties         keep the top `density` fraction of each tensor by magnitude, elect a sign per element (by total mass
               or by frequency), average the values that agree with the elected sign
  dare_linear  drop entries at random with probability 1 - density, rescale survivors by 1 / density, weighted sum
  dare_ties    random drop + rescale, then the sign election and disjoint mean of TIES

The sign of TIES / DARE-TIES is elected on the pruned tensors before the weights are applied, as the reference does.
One deliberate difference: the DARE strategies do rescale the survivors by 1 / density, as the DARE method and PEFT
define it; the reference computes that quotient and discards it (`utils/merges/utils.py:51-53`), so its DARE output is
smaller by the factor `density`.

lora_A and lora_B are merged separately per module; ranks are zero-padded to the largest rank; each adapter's
alpha / r is folded into its B first so that adapters with different scales combine correctly.
"""

from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

from .lora import LoraConfig, ModuleMap


def prune_magnitude(t: torch.Tensor, density: float) -> torch.Tensor:
    if density >= 1.0:
        return t
    k = max(int(density * t.numel()), 1)
    flat = t.abs().flatten()
    thresh = torch.topk(flat, k, largest=True).values[-1]
    return torch.where(t.abs() >= thresh, t, torch.zeros_like(t))


def prune_random(t: torch.Tensor, density: float, rescale: bool, generator=None) -> torch.Tensor:
    if density >= 1.0:
        return t
    mask = torch.bernoulli(torch.full_like(t, density, dtype=torch.float32), generator=generator).to(t.dtype)
    out = t * mask
    return out / density if rescale else out


def majority_sign_mask(stacked: torch.Tensor, method: str = "total") -> torch.Tensor:
    """stacked: [n, ...].  True where an entry's sign equals the elected sign of its position."""
    sign = stacked.sign()
    if method == "frequency":
        elected = sign.sum(0)
    else:
        elected = stacked.sum(0)
    elected = torch.where(elected >= 0, torch.ones_like(elected), -torch.ones_like(elected))
    return sign == elected


def disjoint_merge(stacked: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    kept = stacked * mask
    count = mask.sum(0).clamp(min=1)
    return kept.sum(0) / count


def merge_tensors(tensors: Sequence[torch.Tensor], weights: Sequence[float], strategy: str = "linear", density: float = 1.0,
                  majority_sign_method: str = "total", generator=None) -> torch.Tensor:
    w = torch.tensor(list(weights), dtype=torch.float32).view(-1, *([1] * tensors[0].dim()))
    ts = [t.float() for t in tensors]
    if strategy == "linear":
        return (torch.stack(ts) * w).sum(0)
    if strategy == "ties":
        ts = [prune_magnitude(t, density) for t in ts]
    elif strategy in ("dare_linear", "dare_ties"):
        ts = [prune_random(t, density, rescale=True, generator=generator) for t in ts]
    else:
        raise ValueError(f"unknown merge strategy {strategy!r}")
    unweighted = torch.stack(ts)
    stacked = unweighted * w
    if strategy == "dare_linear":
        return stacked.sum(0)
    # the sign is elected on the pruned tensors BEFORE the weights are applied (reference utils/merges/strategies.py:62-66,
    # 93-97), so a negative or a large weight does not change which entries take part
    return disjoint_merge(stacked, majority_sign_mask(unweighted, majority_sign_method))


def _pad_rank(t: torch.Tensor, r: int, dim: int) -> torch.Tensor:
    if t.shape[dim] == r:
        return t
    shape = list(t.shape)
    shape[dim] = r - t.shape[dim]
    return torch.cat([t, torch.zeros(shape, dtype=t.dtype)], dim)


def merge_adapters(adapters: Sequence[Tuple[LoraConfig, ModuleMap]], weights: Sequence[float], strategy: str = "linear",
                   density: float = 1.0, majority_sign_method: str = "total", seed: int = 0) -> Tuple[LoraConfig, ModuleMap]:
    if len(weights) != len(adapters):
        raise ValueError("one weight per adapter is required")
    r = max(c.r for c, _ in adapters)
    gen = torch.Generator().manual_seed(seed)
    modules = sorted(set().union(*[set(mm.keys()) for _, mm in adapters]))
    out: ModuleMap = {}
    for mod in modules:
        As, Bs, ws = [], [], []
        for (cfg, mm), wgt in zip(adapters, weights):
            if mod not in mm:
                continue
            As.append(_pad_rank(mm[mod]["lora_A"].float(), r, 0))
            Bs.append(_pad_rank(mm[mod]["lora_B"].float() * cfg.scale, r, 1))
            ws.append(wgt)
        out[mod] = {"lora_A": merge_tensors(As, ws, strategy, density, majority_sign_method, gen),
                    "lora_B": merge_tensors(Bs, ws, strategy, density, majority_sign_method, gen)}
    targets = sorted(set(t for c, _ in adapters for t in c.target_modules))
    cfg = LoraConfig(r=r, lora_alpha=float(r), target_modules=targets, base_model_name_or_path=adapters[0][0].base_model_name_or_path)
    return cfg, out


def merge_into_base(weight: torch.Tensor, cfg: LoraConfig, ab: Dict[str, torch.Tensor]) -> torch.Tensor:
    """W + scale * B A: the static merge used by `--merge-adapter-weights` (reference `utils/adapter.py:331-399`)."""
    return (weight.float() + cfg.scale * (ab["lora_B"].float() @ ab["lora_A"].float())).to(weight.dtype)
