"""Checkpoint access: tensor-name -> file routing over safetensors shards, lazy handles, and the
tensor-parallel slicing helpers the model loaders use.

Behavioural counterpart of `server/lorax_server/utils/weights.py:43-407` in the reference (`get_tensor`,
`get_sharded`, `get_partial_sharded` with block = size // world_size, packed QKV handling, and an
in-memory variant for adapters).  `.bin` checkpoints are converted once to safetensors next to the
source (`utils/convert.py:62-114`).
"""

from __future__ import annotations

import json
import os
import struct
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence

import torch
from safetensors import safe_open
from safetensors.torch import load_file, save_file


class AbstractWeights:
    # GPTQ / AWQ checkpoints: {"quant_method", "bits", "group_size", "zero_offset"} (see `checkpoint_quantization`); a linear
    # layer stored as `<name>.qweight / .qzeros / .scales [/ .g_idx]` is then visible under `<name>.weight`, either in the
    # packed resident form (`keep_packed`) or expanded to the loader's dtype
    quant: Optional[dict] = None
    keep_packed: bool = True

    def get_tensor(self, name: str) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError

    def has_tensor(self, name: str) -> bool:  # pragma: no cover - interface
        raise NotImplementedError

    def _raw(self, name: str) -> Optional[torch.Tensor]:  # pragma: no cover - interface
        """The stored tensor without any conversion, or None."""
        raise NotImplementedError

    def _quant_base(self, name: str) -> Optional[str]:
        if self.quant is None or not name.endswith(".weight"):
            return None
        base = name[: -len("weight")]
        return base if self._raw_exists(base + "qweight") else None

    def _raw_exists(self, name: str) -> bool:
        return self._raw(name) is not None

    def get_quantized_linear(self, name: str):
        """`<name>` ends in `.weight`: the packed `GroupQuantWeight` of that layer when its groups are contiguous and
        `keep_packed` is set, else the dense [out, in] matrix."""
        from .quant_formats import from_checkpoint
        base = self._quant_base(name)
        q = self.quant
        tensors = {k: self._raw(base + k) for k in ("qweight", "qzeros", "scales")}
        g = self._raw(base + "g_idx")
        if g is not None:
            tensors["g_idx"] = g
        dt = getattr(self, "dtype", None) or torch.float32
        packed, dense = from_checkpoint(tensors, q.get("quant_method", "gptq"), int(q.get("bits", 4)), int(q.get("group_size", 128)),
                                        int(q.get("zero_offset", 1)), dtype=dt, want_dense=not self.keep_packed)
        if packed is not None and self.keep_packed:
            return packed
        return dense

    def get_shape(self, name: str):
        return tuple(self.get_tensor(name).shape)


class Weights(AbstractWeights):
    def __init__(self, filenames: Sequence[os.PathLike], device="cpu", dtype: Optional[torch.dtype] = None,
                 rank: int = 0, world_size: int = 1, aliases: Optional[Dict[str, List[str]]] = None, prefix: str = ""):
        self.routing: Dict[str, str] = {}
        for fn in filenames:
            with safe_open(str(fn), framework="pt") as f:
                for k in f.keys():
                    if k in self.routing:
                        raise RuntimeError(f"key {k} found in {fn} and {self.routing[k]}")
                    self.routing[k] = str(fn)
        self.aliases = aliases or {}
        self.device = torch.device(device)
        self.dtype = dtype
        self.rank = rank
        self.world_size = world_size
        self.prefix = prefix
        self._handles: Dict[str, object] = {}

    # ---------------------------------------------------------------- routing
    def _handle(self, filename: str):
        h = self._handles.get(filename)
        if h is None:
            h = self._handles[filename] = safe_open(filename, framework="pt")
        return h

    def _resolve(self, name: str):
        for cand in [self.prefix + name, name] + self.aliases.get(name, []):
            fn = self.routing.get(cand)
            if fn is not None:
                return fn, cand
        raise KeyError(f"weight {name} does not exist")

    def has_tensor(self, name: str) -> bool:
        try:
            self._resolve(name)
            return True
        except KeyError:
            return self._quant_base(name) is not None

    def _raw(self, name: str) -> Optional[torch.Tensor]:
        try:
            fn, key = self._resolve(name)
        except KeyError:
            return None
        return self._handle(fn).get_tensor(key)

    def _raw_exists(self, name: str) -> bool:
        try:
            self._resolve(name)
            return True
        except KeyError:
            return False

    def _slice(self, name: str):
        fn, key = self._resolve(name)
        return self._handle(fn).get_slice(key)

    def get_shape(self, name: str):
        return tuple(self._slice(name).get_shape())

    def keys(self):
        return list(self.routing.keys())

    def _finish(self, t: torch.Tensor) -> torch.Tensor:
        if self.dtype is not None and t.dtype.is_floating_point and t.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
            t = t.to(self.dtype)
        return t.to(self.device)

    def _dequant_fp8(self, name: str, t: torch.Tensor, row0: int = 0, col0: int = 0) -> torch.Tensor:
        """Block-scaled fp8 checkpoints (`<name>` in e4m3 next to `<name>_scale_inv`, one fp32 scale per 128 x 128 block):
        return the slice starting at (row0, col0) in the loader's dtype.  The model re-quantises for its own kernels."""
        if t.dtype != torch.float8_e4m3fn or not self.has_tensor(name + "_scale_inv"):
            return t
        if row0 % 128 or col0 % 128:
            raise ValueError(f"{name}: an fp8 shard must start on a 128-element block boundary (got {row0}, {col0})")
        fn, key = self._resolve(name + "_scale_inv")
        scale = self._handle(fn).get_tensor(key).float()
        r, c = t.shape
        s = scale[row0 // 128: row0 // 128 + (r + 127) // 128, col0 // 128: col0 // 128 + (c + 127) // 128]
        s = s.repeat_interleave(128, 0)[:r].repeat_interleave(128, 1)[:, :c]
        return (t.float() * s).to(self.dtype or torch.bfloat16)

    # ---------------------------------------------------------------- getters
    def get_tensor(self, name: str) -> torch.Tensor:
        try:
            fn, key = self._resolve(name)
        except KeyError:
            if self._quant_base(name) is None:
                raise
            t = self.get_quantized_linear(name)
            return t if not isinstance(t, torch.Tensor) else self._finish(t)
        return self._finish(self._dequant_fp8(name, self._handle(fn).get_tensor(key)))

    def get_partial_sharded(self, name: str, dim: int) -> torch.Tensor:
        """This rank's contiguous block of `dim` (block = size // world_size; the tail goes to the last rank's
        neighbour by the same rule as the reference: start = rank * block)."""
        sl = self._slice(name)
        size = sl.get_shape()[dim]
        block = size // self.world_size
        start, stop = self.rank * block, (self.rank + 1) * block
        if dim == 0:
            t = self._dequant_fp8(name, sl[start:stop], row0=start)
        elif dim == 1:
            t = self._dequant_fp8(name, sl[:, start:stop], col0=start)
        else:
            raise NotImplementedError("only dims 0 and 1 are sharded")
        return self._finish(t)

    def get_sharded(self, name: str, dim: int) -> torch.Tensor:
        size = self.get_shape(name)[dim]
        if size % self.world_size != 0:
            raise ValueError(f"{name}: dim {dim} of size {size} is not divisible by {self.world_size} shards")
        return self.get_partial_sharded(name, dim)

    def get_rows(self, name: str, start: int, stop: int) -> torch.Tensor:
        return self._finish(self._dequant_fp8(name, self._slice(name)[start:stop], row0=start))

    def get_multi_sharded(self, names: Iterable[str], dim: int) -> torch.Tensor:
        """Concatenate the per-rank shards of several tensors (fused QKV / gate_up)."""
        return torch.cat([self.get_sharded(n, dim) for n in names], dim=0 if dim == 0 else dim)


class InMemoryWeights(AbstractWeights):
    """Tensors already in memory (adapter module maps)."""

    def __init__(self, tensors: Dict[str, torch.Tensor], device="cpu", dtype=None, rank: int = 0, world_size: int = 1):
        self.tensors = tensors
        self.device = torch.device(device)
        self.dtype = dtype
        self.rank, self.world_size = rank, world_size

    def has_tensor(self, name):
        return name in self.tensors or self._quant_base(name) is not None

    def _raw(self, name):
        return self.tensors.get(name)

    def keys(self):
        return list(self.tensors.keys())

    def get_tensor(self, name):
        if name not in self.tensors and self._quant_base(name) is not None:
            t = self.get_quantized_linear(name)
            return t if not isinstance(t, torch.Tensor) else self.get_tensor_from(t)
        t = self.tensors[name]
        if self.dtype is not None and t.dtype.is_floating_point:
            t = t.to(self.dtype)
        return t.to(self.device)

    def get_partial_sharded(self, name, dim):
        t = self.tensors[name]
        block = t.shape[dim] // self.world_size
        t = t.narrow(dim, self.rank * block, block)
        return self.get_tensor_from(t)

    get_sharded = get_partial_sharded

    def get_tensor_from(self, t):
        if self.dtype is not None and t.dtype.is_floating_point:
            t = t.to(self.dtype)
        return t.to(self.device)


class MergedWeights(AbstractWeights):
    """A checkpoint with one LoRA adapter folded into it: every `<module>.weight` the adapter targets comes back as
    W + scale * B A (`--merge-adapter-weights`; the reference writes such a checkpoint to disk first, `utils/adapter.py:331-399`)."""

    def __init__(self, inner: AbstractWeights, lora_config, module_map):
        self.inner, self.cfg, self.mm = inner, lora_config, module_map
        self.quant = getattr(inner, "quant", None)
        self.keep_packed = False                            # the sum needs the dense matrix
        self.dtype = getattr(inner, "dtype", None)
        self.merged = 0

    def has_tensor(self, name):
        return self.inner.has_tensor(name)

    def keys(self):
        return self.inner.keys()

    def _raw(self, name):
        return self.inner._raw(name)

    def get_tensor(self, name):
        keep, self.inner.keep_packed = getattr(self.inner, "keep_packed", True), False
        try:
            t = self.inner.get_tensor(name)
        finally:
            self.inner.keep_packed = keep
        mod = name[: -len(".weight")] if name.endswith(".weight") else None
        if mod in self.mm:
            from ..adapters.merges import merge_into_base
            self.merged += 1
            return merge_into_base(t, self.cfg, {k: v.to(t.device) for k, v in self.mm[mod].items()})
        return t


def checkpoint_quantization(model_dir: os.PathLike, config: Optional[dict] = None) -> Optional[dict]:
    """How the checkpoint's linear layers are stored, from `config.json` (`quantization_config`), AutoGPTQ's
    `quantize_config.json` or AutoAWQ's `quant_config.json`; None for a dense (or block-fp8) checkpoint.  The reference reads
    the same files in `Weights._set_gptq_params` (utils/weights.py:409-447)."""
    d = Path(model_dir)
    qc = dict((config or {}).get("quantization_config") or {})
    if not qc:
        for fn in ("quantize_config.json", "quant_config.json"):
            if (d / fn).exists():
                qc = json.loads((d / fn).read_text())
                break
    if not qc:
        return None
    method = qc.get("quant_method") or ("awq" if "w_bit" in qc else "gptq")
    if method not in ("gptq", "awq"):
        return None
    bits = int(qc.get("bits", qc.get("w_bit", 4)))
    group = int(qc.get("group_size", qc.get("q_group_size", 128)))
    v2 = qc.get("checkpoint_format") == "gptq_v2"
    return {"quant_method": method, "bits": bits, "group_size": group, "zero_offset": 0 if (v2 or method == "awq") else 1,
            "desc_act": bool(qc.get("desc_act", False))}


# -------------------------------------------------------------------------------------------- files
def safetensors_header(path: os.PathLike) -> dict:
    """Parse the JSON header of a safetensors file without reading tensor data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        return json.loads(f.read(n))


def safetensors_nbytes(path: os.PathLike) -> int:
    """Sum of the tensor byte sizes recorded in the header (`utils/sources/source.py:75-130` of the reference
    uses the same figure as the adapter's memory cost)."""
    total = 0
    for k, v in safetensors_header(path).items():
        if k == "__metadata__":
            continue
        a, b = v["data_offsets"]
        total += b - a
    return total


def weight_files(model_dir: os.PathLike, extension: str = ".safetensors") -> List[Path]:
    d = Path(model_dir)
    files = sorted(p for p in d.glob(f"*{extension}") if not p.name.startswith("adapter_") and "training_args" not in p.name)
    if not files and extension == ".safetensors":
        bins = sorted(p for p in d.glob("*.bin") if "training_args" not in p.name and not p.name.startswith("adapter_"))
        if bins:
            return convert_files(bins)
    if not files:
        raise FileNotFoundError(f"no {extension} weights under {d}")
    return files


def convert_file(pt_file: Path, sf_file: Path, discard_names: Sequence[str] = ()):
    """torch pickle -> safetensors, dropping tied duplicates and checking for NaN/Inf and round-trip equality."""
    loaded = torch.load(str(pt_file), map_location="cpu", weights_only=True)
    if "state_dict" in loaded:
        loaded = loaded["state_dict"]
    seen, out = {}, {}
    for k, v in sorted(loaded.items()):
        if not isinstance(v, torch.Tensor) or k in discard_names:
            continue
        key = (v.data_ptr(), tuple(v.shape), v.dtype)
        if key in seen:                       # shared storage (tied weights): keep the first name only
            continue
        seen[key] = k
        if v.dtype.is_floating_point and not torch.isfinite(v).all():
            raise ValueError(f"{pt_file}: tensor {k} has NaN/Inf values")
        out[k] = v.contiguous()
    sf_file.parent.mkdir(parents=True, exist_ok=True)
    save_file(out, str(sf_file), metadata={"format": "pt"})
    back = load_file(str(sf_file))
    for k, v in out.items():
        if not torch.equal(v, back[k]):
            raise RuntimeError(f"{k} changed in the safetensors round trip")


def convert_files(pt_files: Sequence[Path], discard_names: Sequence[str] = ()) -> List[Path]:
    outs = []
    for p in pt_files:
        sf = p.with_name(p.stem.replace("pytorch_model", "model") + ".safetensors")
        if not sf.exists():
            convert_file(p, sf, discard_names)
        outs.append(sf)
    return outs
