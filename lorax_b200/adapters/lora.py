"""PEFT LoRA adapters: config, (de)serialisation, rank padding, tensor-parallel sharding and packing into
the single-blob layout the kernels read.

File format (public surface, same as the reference `server/lorax_server/adapters/lora.py:37-84,193-210`):
``adapter_config.json`` with ``r``, ``lora_alpha``, ``target_modules``, ``fan_in_fan_out``, ``use_rslora``,
``base_model_name_or_path`` and ``adapter_model.safetensors`` with keys
``base_model.model.{module}.lora_A.weight`` [r, in] and ``...lora_B.weight`` [out, r].
`peft` itself is not required.

Blob layout.  All matrices of one adapter have sizes proportional to its (padded) rank r, so an adapter is
stored as ONE contiguous bf16 blob of ``r * layout.units`` elements:

    for layer l, group g in (qkv, o, gate_up, down):   A_cat [nparts*r, K_g]  at r * (l*C + offA[g])
                                                       B_cat [N_g, r]         at r * (l*C + offB[g])
    lm_head (optional)                                 A [r, H], B [V_local, r] after the last layer

A single blob means adapter exchange between the pinned host tier and HBM is one `cudaMemcpyAsync`, and
the kernels find any matrix from (slot base, slot rank) with two multiplications.  The LoRA scale
(alpha / r, or alpha / sqrt(r) for rsLoRA) is folded into B; ranks are zero-padded to 8 or a multiple of 16.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
from safetensors.torch import load_file, save_file

GROUP_ORDER = ("qkv", "o", "gate_up", "down")
LM_HEAD = "lm_head"


def pad_rank(r: int) -> int:
    """The next multiple of 16: one K step of a bf16 tensor-core instruction, so that the LoRA delta can be added by
    UMMAs inside the base GEMM (the reference pads to 8*world_size or a multiple of 16, `utils/punica.py:46-76`)."""
    return max(16, (r + 15) // 16 * 16)


@dataclass
class LoraConfig:
    r: int
    lora_alpha: float
    target_modules: List[str]
    base_model_name_or_path: str = ""
    fan_in_fan_out: bool = False
    use_rslora: bool = False
    bias: str = "none"
    peft_type: str = "LORA"
    task_type: str = "CAUSAL_LM"
    extra: dict = field(default_factory=dict)

    @property
    def scale(self) -> float:
        return self.lora_alpha / math.sqrt(self.r) if self.use_rslora else self.lora_alpha / self.r

    @classmethod
    def from_dict(cls, d: dict) -> "LoraConfig":
        known = {"r", "lora_alpha", "target_modules", "base_model_name_or_path", "fan_in_fan_out", "use_rslora", "bias",
                 "peft_type", "task_type"}
        tm = d.get("target_modules") or []
        if isinstance(tm, str):
            tm = [tm]
        return cls(r=int(d["r"]), lora_alpha=float(d.get("lora_alpha", d["r"])), target_modules=list(tm),
                   base_model_name_or_path=d.get("base_model_name_or_path") or "", fan_in_fan_out=bool(d.get("fan_in_fan_out", False)),
                   use_rslora=bool(d.get("use_rslora", False)), bias=d.get("bias", "none"), peft_type=d.get("peft_type", "LORA"),
                   task_type=d.get("task_type") or "CAUSAL_LM", extra={k: v for k, v in d.items() if k not in known})

    @classmethod
    def load(cls, adapter_dir: os.PathLike) -> "LoraConfig":
        with open(os.path.join(adapter_dir, "adapter_config.json")) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        d = dict(r=self.r, lora_alpha=self.lora_alpha, target_modules=self.target_modules,
                 base_model_name_or_path=self.base_model_name_or_path, fan_in_fan_out=self.fan_in_fan_out,
                 use_rslora=self.use_rslora, bias=self.bias, peft_type=self.peft_type, task_type=self.task_type)
        d.update(self.extra)
        return d


ModuleMap = Dict[str, Dict[str, torch.Tensor]]   # "model.layers.0.self_attn.q_proj" -> {"lora_A": [r,in], "lora_B": [out,r]}


def load_peft_adapter(adapter_dir: os.PathLike) -> Tuple[LoraConfig, ModuleMap]:
    cfg = LoraConfig.load(adapter_dir)
    st_path = os.path.join(adapter_dir, "adapter_model.safetensors")
    if os.path.exists(st_path):
        tensors = load_file(st_path)
    else:
        bin_path = os.path.join(adapter_dir, "adapter_model.bin")
        tensors = torch.load(bin_path, map_location="cpu", weights_only=True)
    return cfg, module_map_from_tensors(tensors, cfg)


def module_map_from_tensors(tensors: Dict[str, torch.Tensor], cfg: Optional[LoraConfig] = None) -> ModuleMap:
    mm: ModuleMap = {}
    for key, t in tensors.items():
        name = key
        if name.startswith("base_model.model."):
            name = name[len("base_model.model."):]
        for tag in ("lora_A", "lora_B"):
            for suffix in (f".{tag}.weight", f".{tag}.default.weight"):
                if name.endswith(suffix):
                    mod = name[: -len(suffix)]
                    if cfg is not None and cfg.fan_in_fan_out:
                        t = t.t()
                    mm.setdefault(mod, {})[tag] = t
    bad = [m for m, v in mm.items() if set(v) != {"lora_A", "lora_B"}]
    if bad:
        raise ValueError(f"adapter modules without both lora_A and lora_B: {bad[:3]}")
    return mm


def save_peft_adapter(adapter_dir: os.PathLike, cfg: LoraConfig, mm: ModuleMap):
    os.makedirs(adapter_dir, exist_ok=True)
    with open(os.path.join(adapter_dir, "adapter_config.json"), "w") as f:
        json.dump(cfg.to_dict(), f, indent=1)
    flat = {}
    for mod, ab in mm.items():
        flat[f"base_model.model.{mod}.lora_A.weight"] = ab["lora_A"].contiguous()
        flat[f"base_model.model.{mod}.lora_B.weight"] = ab["lora_B"].contiguous()
    save_file(flat, os.path.join(adapter_dir, "adapter_model.safetensors"), metadata={"format": "pt"})


def random_adapter(model_config, r: int, alpha: float, target_modules: Sequence[str], seed: int, std_a: float = 0.02,
                   std_b: float = 0.02, dtype=torch.float32, layer_prefix: str = "model.layers") -> Tuple[LoraConfig, ModuleMap]:
    """A random PEFT-shaped adapter for the given base architecture (benchmarks and tests)."""
    c = model_config
    g = torch.Generator(device="cpu").manual_seed(seed)
    dims = {
        "q_proj": (c.hidden_size, c.q_size), "k_proj": (c.hidden_size, c.kv_size), "v_proj": (c.hidden_size, c.kv_size),
        "o_proj": (c.q_size, c.hidden_size), "gate_proj": (c.hidden_size, c.intermediate_size),
        "up_proj": (c.hidden_size, c.intermediate_size), "down_proj": (c.intermediate_size, c.hidden_size),
    }
    mm: ModuleMap = {}
    for l in range(c.num_hidden_layers):
        for t in target_modules:
            if t == "lm_head":
                continue
            fin, fout = dims[t]
            sub = "self_attn" if t in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
            mm[f"{layer_prefix}.{l}.{sub}.{t}"] = {
                "lora_A": (torch.randn(r, fin, generator=g) * std_a).to(dtype),
                "lora_B": (torch.randn(fout, r, generator=g) * std_b).to(dtype),
            }
    if "lm_head" in target_modules:
        mm["lm_head"] = {"lora_A": (torch.randn(r, c.hidden_size, generator=g) * std_a).to(dtype),
                         "lora_B": (torch.randn(c.vocab_size, r, generator=g) * std_b).to(dtype)}
    cfg = LoraConfig(r=r, lora_alpha=alpha, target_modules=list(target_modules))
    return cfg, mm


# ------------------------------------------------------------------------------------------------ layout
@dataclass
class GroupInfo:
    K: int
    parts: List[int]
    names: List[str]
    shard: str
    offA: int = 0
    offB: int = 0

    @property
    def N(self):
        return sum(self.parts)

    @property
    def bounds(self):
        n0 = self.parts[0]
        n1 = n0 + (self.parts[1] if len(self.parts) > 1 else 0)
        N = self.N
        return (n0 if len(self.parts) > 1 else N), (n1 if len(self.parts) > 2 else N)


class BlobLayout:
    """Offsets (in elements per unit rank) of every LoRA matrix of one adapter on one TP rank."""

    def __init__(self, model, with_lm_head: bool = True):
        self.num_layers = model.config.num_hidden_layers
        self.groups: Dict[str, GroupInfo] = {}
        off = 0
        for name, g in model.group_shapes().items():
            gi = GroupInfo(K=g["K"], parts=list(g["parts"]), names=list(g["names"]), shard=g["shard"])
            gi.offA = off
            off += len(gi.parts) * gi.K
            gi.offB = off
            off += gi.N
            self.groups[name] = gi
        self.layer_units = off
        self.has_lm_head = with_lm_head
        total = self.layer_units * self.num_layers
        if with_lm_head:
            gi = GroupInfo(K=model.hidden, parts=[model.lm_head.shape[0] if model.lm_head is not None else model.vocab_local],
                           names=["lm_head"], shard="col")
            gi.offA = total
            gi.offB = total + gi.K
            total += gi.K + gi.N
            self.groups[LM_HEAD] = gi
        self.units = total
        self.tp_rank = model.tp.rank
        self.tp_world = model.tp.world_size
        c = model.config
        self.full = dict(nh=c.num_attention_heads, nkv=c.num_key_value_heads, d=c.head_dim, hidden=c.hidden_size,
                         inter=c.intermediate_size, vocab=c.vocab_size)
        self.local = dict(nh=model.nh, nkv=model.nkv, kv_replicas=model.kv_replicas, vocab_local=model.vocab_local,
                          vocab_start=model.vocab_start)
        self.layer_prefixes = ["model.layers", "transformer.h", "gpt_neox.layers", "model.decoder.layers"]

    def unit_off(self, group: str, layer: int, which: str) -> int:
        gi = self.groups[group]
        base = 0 if group == LM_HEAD else layer * self.layer_units
        return base + (gi.offA if which == "A" else gi.offB)

    def blob_elems(self, rank_padded: int) -> int:
        return rank_padded * self.units

    # -------------------------------------------------------------- packing
    def _module_name(self, mm: ModuleMap, layer: int, proj: str) -> Optional[str]:
        sub = "self_attn" if proj in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
        for pre in self.layer_prefixes:
            n = f"{pre}.{layer}.{sub}.{proj}"
            if n in mm:
                return n
        return None

    def _shard_rows(self, t: torch.Tensor, proj: str) -> torch.Tensor:
        """Output-feature (dim 0 of lora_B) shard of a column-parallel projection."""
        ws, rk = self.tp_world, self.tp_rank
        if ws == 1:
            return t
        d = self.full["d"]
        if proj == "q_proj":
            b = t.shape[0] // ws
            return t[rk * b:(rk + 1) * b]
        if proj in ("k_proj", "v_proj"):
            nkv_l, rep = self.local["nkv"], self.local["kv_replicas"]
            kv_rank = rk // rep if self.full["nkv"] < ws else rk
            return t[kv_rank * nkv_l * d:(kv_rank + 1) * nkv_l * d]
        if proj in ("gate_proj", "up_proj"):
            b = t.shape[0] // ws
            return t[rk * b:(rk + 1) * b]
        if proj == "lm_head":
            v0, vl = self.local["vocab_start"], self.local["vocab_local"]
            out = torch.zeros(vl, t.shape[1], dtype=t.dtype)
            n = max(min(t.shape[0] - v0, vl), 0)
            out[:n] = t[v0:v0 + n]
            return out
        raise KeyError(proj)

    def _shard_cols(self, t: torch.Tensor) -> torch.Tensor:
        """Input-feature (dim 1 of lora_A) shard of a row-parallel projection."""
        ws, rk = self.tp_world, self.tp_rank
        if ws == 1:
            return t
        b = t.shape[1] // ws
        return t[:, rk * b:(rk + 1) * b]

    def pack(self, cfg: LoraConfig, mm: ModuleMap, dtype=torch.bfloat16, pin: bool = False) -> Tuple[torch.Tensor, int]:
        """-> (blob [r_pad * units], r_pad).  Projections the adapter does not target stay zero."""
        r = cfg.r
        rp = pad_rank(r)
        blob = torch.zeros(self.blob_elems(rp), dtype=dtype)
        if pin and torch.cuda.is_available():
            blob = blob.pin_memory()
        scale = cfg.scale

        def put(group: str, layer: int, gi: GroupInfo, part: int, proj: str, A: torch.Tensor, B: torch.Tensor):
            A = A.float()
            B = B.float() * scale
            if gi.shard == "row":
                A = self._shard_cols(A)
            else:
                B = self._shard_rows(B, proj)
            nparts = len(gi.parts)
            a0 = rp * self.unit_off(group, layer, "A")
            Av = blob[a0: a0 + nparts * rp * gi.K].view(nparts * rp, gi.K)
            Av[part * rp: part * rp + r] = A.to(dtype)
            b0 = rp * self.unit_off(group, layer, "B")
            Bv = blob[b0: b0 + gi.N * rp].view(gi.N, rp)
            n_start = sum(gi.parts[:part])
            Bv[n_start: n_start + gi.parts[part], :r] = B.to(dtype)

        for layer in range(self.num_layers):
            for gname in GROUP_ORDER:
                gi = self.groups.get(gname)
                if gi is None:
                    continue
                for part, proj in enumerate(gi.names):
                    mod = self._module_name(mm, layer, proj)
                    if mod is None:
                        continue
                    put(gname, layer, gi, part, proj, mm[mod]["lora_A"], mm[mod]["lora_B"])
        if self.has_lm_head and "lm_head" in mm:
            put(LM_HEAD, 0, self.groups[LM_HEAD], 0, "lm_head", mm["lm_head"]["lora_A"], mm["lm_head"]["lora_B"])
        return blob, rp


def check_architecture(cfg: LoraConfig, mm: ModuleMap, model_config) -> None:
    """Reject adapters whose matrices do not fit the base model (reference: `utils/adapter.py:115-148`)."""
    c = model_config
    dims = {
        "q_proj": (c.hidden_size, c.q_size), "k_proj": (c.hidden_size, c.kv_size), "v_proj": (c.hidden_size, c.kv_size),
        "o_proj": (c.q_size, c.hidden_size), "gate_proj": (c.hidden_size, c.intermediate_size),
        "up_proj": (c.hidden_size, c.intermediate_size), "down_proj": (c.intermediate_size, c.hidden_size),
        "lm_head": (c.hidden_size, c.vocab_size),
    }
    for mod, ab in mm.items():
        proj = mod.split(".")[-1]
        if proj not in dims:
            continue
        fin, fout = dims[proj]
        if ab["lora_A"].shape[1] != fin or ab["lora_B"].shape[0] != fout:
            raise ValueError(
                f"adapter module {mod} has shape A{tuple(ab['lora_A'].shape)} B{tuple(ab['lora_B'].shape)}, "
                f"which does not match the base model ({fin} -> {fout}); base_model_name_or_path={cfg.base_model_name_or_path!r}")
