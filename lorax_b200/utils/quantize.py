"""Offline weight quantisation: `lorax-b200 quantize <model> <out_dir> --method fp8`.

The reference's `quantize` sub-command runs GPTQ calibration (`server/lorax_server/cli.py:189-230`,
`utils/gptq/quantize.py`).  Here the supported scheme is the one the B200 kernels serve: e4m3 weights with one fp32
scale per 128 x 128 block, computed from the checkpoint alone (no calibration data).  The output directory is a
normal safetensors checkpoint in which every quantised `*.weight` is stored as float8_e4m3fn next to a
`*.weight_scale_inv` tensor (the name DeepSeek-style block-fp8 checkpoints use), plus the config with a
`quantization_config` entry, so the loader can tell it apart from a bf16 checkpoint.
"""

from __future__ import annotations

import json
import shutil
from pathlib import Path
from typing import Dict, Iterable

import torch

from ..ops.reference import dequantize_weight_fp8_block128, quantize_weight_fp8_block128

# projections of the decoder blocks; embeddings, norms and the lm_head stay in the checkpoint's dtype
QUANT_SUFFIXES = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "gate_proj.weight", "up_proj.weight",
                  "down_proj.weight", "qkv_proj.weight", "gate_up_proj.weight", "query_key_value.weight", "dense.weight",
                  "dense_h_to_4h.weight", "dense_4h_to_h.weight", "c_attn.weight", "c_proj.weight", "c_fc.weight", "w1.weight",
                  "w2.weight", "w3.weight")


def should_quantize(name: str, t: torch.Tensor) -> bool:
    return t.dim() == 2 and name.endswith(QUANT_SUFFIXES) and min(t.shape) >= 128


def quantize_state_dict(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for name, t in sd.items():
        if should_quantize(name, t):
            q, scale = quantize_weight_fp8_block128(t)
            out[name] = q
            out[name + "_scale_inv"] = scale
        else:
            out[name] = t
    return out


def dequantize_state_dict(sd: Dict[str, torch.Tensor], dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    out = {}
    for name, t in sd.items():
        if name.endswith("_scale_inv"):
            continue
        if t.dtype == torch.float8_e4m3fn and name + "_scale_inv" in sd:
            out[name] = dequantize_weight_fp8_block128(t, sd[name + "_scale_inv"]).to(dtype)
        else:
            out[name] = t
    return out


def quantize_checkpoint(model_dir: str, out_dir: str, method: str = "fp8", files: Iterable[str] = ()) -> Dict[str, int]:
    """Quantise every safetensors shard of `model_dir` into `out_dir`.  Returns counts for the log line."""
    if method != "fp8":
        raise ValueError(f"unsupported quantisation method {method!r}: this build quantises to block-scaled fp8 "
                         f"(GPTQ / AWQ checkpoints are loaded, not produced)")
    from safetensors.torch import load_file, save_file
    src, dst = Path(model_dir), Path(out_dir)
    dst.mkdir(parents=True, exist_ok=True)
    shards = [src / f for f in files] if files else sorted(src.glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no .safetensors files under {src}")
    n_q = n_all = 0
    for shard in shards:
        sd = load_file(str(shard))
        q = quantize_state_dict(sd)
        n_all += len(sd)
        n_q += sum(1 for k in q if k.endswith("_scale_inv"))
        save_file(q, str(dst / shard.name), metadata={"format": "pt"})
    for extra in src.iterdir():
        if extra.suffix in (".json", ".model", ".txt") and extra.name != "model.safetensors.index.json":
            shutil.copy(extra, dst / extra.name)
    cfg_path = dst / "config.json"
    if cfg_path.exists():
        cfg = json.loads(cfg_path.read_text())
        cfg["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128],
                                      "activation_scheme": "dynamic"}
        cfg_path.write_text(json.dumps(cfg, indent=2))
    return {"tensors": n_all, "quantized": n_q}
