"""Offline weight quantisation: `lorax-server quantize <model> <out_dir> --scheme fp8|gptq`.

The reference's `quantize` sub-command runs GPTQ calibration (`server/lorax_server/cli.py:189-230`,
`utils/gptq/quantize.py`).  Two schemes are written here:

* `fp8`   e4m3 weights with one fp32 scale per 128 x 128 block, computed from the checkpoint alone.  Every quantised
          `*.weight` is stored as float8_e4m3fn next to a `*.weight_scale_inv` tensor (the name DeepSeek-style block-fp8
          checkpoints use).
* `gptq`  4- or 8-bit groups with Hessian-compensated rounding (`quant_formats.gptq_quantize`).  The Hessians of every
          projection's inputs are collected in one pass of calibration text (or random token ids when no text is given)
          through the dense model; the result is written in the AutoGPTQ layout (`qweight / qzeros / scales / g_idx`),
          which this loader and other GPTQ runtimes read.

Both mark the config with a `quantization_config` entry, so the loader can tell the result from a dense checkpoint.
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


def quantize_checkpoint(model_dir: str, out_dir: str, method: str = "fp8", files: Iterable[str] = (), **gptq_args) -> Dict[str, int]:
    """Quantise every safetensors shard of `model_dir` into `out_dir`.  Returns counts for the log line."""
    if method == "gptq":
        return gptq_quantize_checkpoint(model_dir, out_dir, **gptq_args)
    if method != "fp8":
        raise ValueError(f"unsupported quantisation scheme {method!r}: fp8 and gptq checkpoints are written")
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


def _copy_side_files(src: Path, dst: Path):
    for extra in src.iterdir():
        if extra.suffix in (".json", ".model", ".txt") and extra.name != "model.safetensors.index.json":
            shutil.copy(extra, dst / extra.name)


def collect_hessians(model, token_batches) -> Dict[tuple, torch.Tensor]:
    """Run `token_batches` (lists of token ids) through the dense model and return, per (layer, projection group), the sum of
    x x^T over every token that entered that group's GEMM, in fp32.  The four groups are the model's fused projections: qkv, o,
    gate_up, down."""
    from ..runtime.kv_cache import KVCache
    from ..runtime.runner import ModelRunner, PrefillItem
    hess: Dict[tuple, torch.Tensor] = {}
    inner = model._linear

    def spy(x, w, b, group, layer, inp, *a, **k):
        xf = x.detach().float()
        key = (layer, group)
        h = xf.t() @ xf
        hess[key] = h if key not in hess else hess[key] + h
        return inner(x, w, b, group, layer, inp, *a, **k)
    longest = max(len(t) for t in token_batches)
    blocks = (longest + 15) // 16 + 2
    kv = KVCache(model.config.num_hidden_layers, blocks, model.nkv, model.d, model.dtype, model.device)
    runner = ModelRunner(model, kv, max_batch=1, max_seq_tokens=longest + 16, max_prefill_tokens=longest + 16, use_graphs=False)
    model._linear = spy
    try:
        for ids in token_batches:
            runner.prefill([PrefillItem(list(ids), 0, list(range(1, (len(ids) + 15) // 16 + 1)))])
    finally:
        model._linear = inner
    return hess


def gptq_quantize_checkpoint(model_dir: str, out_dir: str, bits: int = 4, group: int = 128, nsamples: int = 32, seqlen: int = 256,
                             dataset: str = "", device: str = "", damp: float = 0.01, seed: int = 0, act_order: bool = False) -> Dict[str, int]:
    """GPTQ over every decoder projection of the checkpoint.  `act_order` quantises the input channels of every layer from the
    most to the least active one (largest diagonal entry of the Hessian first; `--act-order` of the reference's quantize
    command, cli.py:145-176) and records the order in `g_idx`, which the loader serves packed.  `dataset` is a UTF-8 text file (one sample per line, cut to
    `seqlen` tokens); without it the calibration inputs are random token ids, which still yields the correlations between a
    layer's input channels but not the token statistics of real text."""
    from safetensors.torch import load_file, save_file

    from ..config import ModelConfig
    from ..models.decoder import DecoderModel
    from ..models.loading import NAME_MAPS
    from .quant_formats import gptq_pack, gptq_quantize
    from .weights import Weights, weight_files
    src, dst = Path(model_dir), Path(out_dir)
    dst.mkdir(parents=True, exist_ok=True)
    mc = ModelConfig.from_pretrained(str(src))
    nm = NAME_MAPS.get(mc.model_type)
    if nm is None or nm.get("conv1d"):
        raise NotImplementedError(f"GPTQ calibration is not wired for model_type={mc.model_type}")
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    files = weight_files(str(src))
    model = DecoderModel.from_weights(mc, Weights(files, device="cpu", dtype=dt), dev, dt, max_positions=max(seqlen + 64, 512))
    gen = torch.Generator().manual_seed(seed)
    if dataset:
        from ..server.runtime import load_tokenizer
        tok = load_tokenizer(str(src))
        if tok is None:
            raise FileNotFoundError(f"{src} has no tokenizer.json to encode the calibration text with")
        lines = [ln for ln in Path(dataset).read_text(encoding="utf-8").splitlines() if ln.strip()][:nsamples]
        batches = [tok.encode(ln).ids[:seqlen] for ln in lines]
        batches = [b for b in batches if len(b) >= 2]
    else:
        batches = [torch.randint(0, mc.vocab_size, (seqlen,), generator=gen).tolist() for _ in range(nsamples)]
    hess = collect_hessians(model, batches)
    del model
    # checkpoint tensor name -> (layer, group)
    owner: Dict[str, tuple] = {}
    for i in range(mc.num_hidden_layers):
        L = nm["layer"].format(i=i)
        for key, grp in (("q", "qkv"), ("k", "qkv"), ("v", "qkv"), ("qkv", "qkv"), ("o", "o"), ("gate", "gate_up"), ("up", "gate_up"),
                         ("gate_up", "gate_up"), ("down", "down")):
            if nm.get(key):
                owner[L + nm[key] + ".weight"] = (i, grp)
    prefixes = tuple(nm.get("prefixes", [""]))
    n_q = n_all = 0
    for shard in files:
        sd = load_file(str(shard))
        out = {}
        for name, t in sd.items():
            n_all += 1
            bare = next((name[len(p):] for p in prefixes if p and name.startswith(p) and name[len(p):] in owner), name)
            key = owner.get(bare)
            g = group if group > 0 else t.shape[1]
            if key is None or key not in hess or t.dim() != 2 or t.shape[1] % g or t.shape[0] % (32 // bits):
                out[name] = t
                continue
            H = hess[key].to(dev)
            W = t.to(dev).float()
            perm = None
            if act_order:
                perm = torch.argsort(torch.diag(H), descending=True, stable=True)
                W, H = W[:, perm], H[perm][:, perm]
            Q, sc, zp = gptq_quantize(W, H, bits=bits, group=group, damp=damp)
            g_idx = None
            if perm is not None:                 # back to the checkpoint's column order; column perm[i] belongs to group i // g
                inv = torch.argsort(perm)
                Q = Q[:, inv]
                g_idx = (inv // g).to(torch.int32).cpu()
            tensors = gptq_pack(Q.cpu(), sc.cpu(), zp.cpu(), bits, g)
            if g_idx is not None:
                tensors["g_idx"] = g_idx
            for suffix, v in tensors.items():
                out[name[: -len("weight")] + suffix] = v.contiguous()
            n_q += 1
        save_file(out, str(dst / Path(shard).name), metadata={"format": "pt"})
    _copy_side_files(src, dst)
    qcfg = {"quant_method": "gptq", "bits": bits, "group_size": group, "desc_act": bool(act_order), "sym": False, "damp_percent": damp,
            "checkpoint_format": "gptq"}
    cfg_path = dst / "config.json"
    if cfg_path.exists():
        cfg = json.loads(cfg_path.read_text())
        cfg["quantization_config"] = qcfg
        cfg_path.write_text(json.dumps(cfg, indent=2))
    (dst / "quantize_config.json").write_text(json.dumps(qcfg, indent=2))
    return {"tensors": n_all, "quantized": n_q}
