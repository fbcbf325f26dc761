"""Typed configuration objects.

Two dataclasses replace the import-time environment globals of the reference
(`server/lorax_server/utils/state.py:12-38`, `utils/dist.py:8-14`,
`utils/graph.py:29-31`):

* :class:`ModelConfig` is the parsed HuggingFace ``config.json`` of the base model.
* :class:`EngineConfig` is every serving knob (launcher flags + environment),
  resolved once and passed explicitly.  Public flag names follow the reference
  launcher (`launcher/src/main.rs:273-655`).
"""

from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

# Architectures handled by the single config-driven decoder (models/decoder.py).
DECODER_MODEL_TYPES = (
    "llama", "mistral", "mixtral", "qwen2", "qwen", "gemma", "gemma2", "phi3", "phi",
    "cohere", "solar", "granite", "gpt2", "gpt_neox", "falcon", "RefinedWeb",
    "RefinedWebModel", "gpt_bigcode", "dbrx",
)


@dataclass
class ModelConfig:
    model_type: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    max_position_embeddings: int = 4096
    sliding_window: Optional[int] = None
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    # MoE (mixtral / dbrx)
    num_local_experts: int = 0
    num_experts_per_tok: int = 0
    # gemma-family quirks
    norm_weight_offset: float = 0.0          # gemma stores (w - 1)
    embedding_multiplier: float = 1.0        # gemma scales embeddings by sqrt(hidden)
    attn_logit_softcapping: Optional[float] = None
    final_logit_softcapping: Optional[float] = None
    query_pre_attn_scalar: Optional[float] = None
    # granite / cohere multipliers
    residual_multiplier: float = 1.0
    attention_multiplier: Optional[float] = None
    logits_scaling: float = 1.0
    logit_scale: float = 1.0
    # layer norm style: "rms" or "layernorm" (gpt2/neox/falcon/phi)
    norm_type: str = "rms"
    # rotary fraction (phi / neox partial rotary)
    partial_rotary_factor: float = 1.0
    # parallel attention+mlp blocks (falcon, neox, phi, cohere)
    parallel_residual: bool = False
    # learned absolute positions (gpt2, bigcode, opt); OPT's table starts at position_offset = 2
    learned_positions: bool = False
    position_offset: int = 0
    # ALiBi instead of any position embedding (bloom, mpt): bias -slope_h * distance on the attention scores
    alibi: bool = False
    alibi_bias_max: float = 8.0
    # LayerNorm right after the embedding lookup (bloom)
    embed_norm: bool = False
    # clamp of the fused QKV projection's output (mpt, dbrx)
    clip_qkv: Optional[float] = None
    eos_token_id: Any = None
    bos_token_id: Any = None
    pad_token_id: Any = None
    torch_dtype: str = "bfloat16"
    quantization_config: Optional[Dict[str, Any]] = None
    extra: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads

    # ------------------------------------------------------------------ sizes
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def is_moe(self) -> bool:
        return self.num_local_experts > 0

    @property
    def attn_scale(self) -> float:
        if self.attention_multiplier is not None:
            return float(self.attention_multiplier)
        if self.query_pre_attn_scalar is not None:
            return float(self.query_pre_attn_scalar) ** -0.5
        return float(self.head_dim) ** -0.5

    # ------------------------------------------------------------------ io
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        d = dict(d)
        mt = d.get("model_type", "llama")
        known = {f.name for f in dataclasses.fields(cls)}
        kw: Dict[str, Any] = {k: v for k, v in d.items() if k in known}
        extra = {k: v for k, v in d.items() if k not in known}
        # key aliases used by the older architectures
        alias = {
            "n_embd": "hidden_size", "n_layer": "num_hidden_layers", "n_head": "num_attention_heads",
            "n_positions": "max_position_embeddings", "n_inner": "intermediate_size",
            "layer_norm_epsilon": "rms_norm_eps", "layer_norm_eps": "rms_norm_eps",
            "num_kv_heads": "num_key_value_heads", "n_head_kv": "num_key_value_heads",
            "rotary_emb_base": "rope_theta", "rotary_pct": "partial_rotary_factor",
        }
        for src, dst in alias.items():
            if src in d and d[src] is not None and dst not in kw:
                kw[dst] = d[src]
        if kw.get("intermediate_size") is None:
            kw["intermediate_size"] = 4 * kw.get("hidden_size", 4096)
        if mt in ("gemma", "gemma2"):
            kw.setdefault("norm_weight_offset", 1.0)
            kw.setdefault("embedding_multiplier", float(kw.get("hidden_size", 4096)) ** 0.5)
            kw.setdefault("hidden_act", d.get("hidden_activation") or d.get("hidden_act", "gelu_pytorch_tanh"))
            kw.setdefault("tie_word_embeddings", True)
        if mt in ("gpt2", "gpt_bigcode"):
            kw.update(norm_type="layernorm", learned_positions=True, hidden_act=d.get("activation_function", "gelu_new"),
                      attention_bias=True, mlp_bias=True, tie_word_embeddings=True)
            if mt == "gpt_bigcode" and d.get("multi_query", True):
                kw["num_key_value_heads"] = 1
        if mt in ("gpt_neox",):
            kw.update(norm_type="layernorm", parallel_residual=d.get("use_parallel_residual", True),
                      attention_bias=True, mlp_bias=True, hidden_act=d.get("hidden_act", "gelu"))
        if mt in ("falcon", "RefinedWeb", "RefinedWebModel"):
            kw.update(norm_type="layernorm", parallel_residual=d.get("parallel_attn", True),
                      hidden_act="gelu", attention_bias=d.get("bias", False), mlp_bias=d.get("bias", False))
            # key/value heads: the 40b layout (new_decoder_architecture; "RefinedWeb" checkpoints imply it) names them, the
            # 7b layout has one shared head when multi_query is set, falcon-rw has as many as query heads
            new_arch = bool(d.get("new_decoder_architecture", mt == "RefinedWeb"))
            nh = kw.get("num_attention_heads", 32)
            if new_arch:
                kw["num_key_value_heads"] = d.get("num_kv_heads") or d.get("n_head_kv") or nh
            else:
                kw["num_key_value_heads"] = 1 if d.get("multi_query", True) else nh
            if d.get("alibi", False):
                raise NotImplementedError("falcon with ALiBi (falcon-rw): its bias is scaled with the scores, unlike bloom's")
            kw["rms_norm_eps"] = d.get("layer_norm_epsilon", 1e-5)
        if mt == "phi":
            kw.update(norm_type="layernorm", parallel_residual=True, attention_bias=True, mlp_bias=True,
                      hidden_act=d.get("hidden_act", "gelu_new"))
        if mt == "cohere":
            kw.update(norm_type="layernorm_nobias", parallel_residual=True, tie_word_embeddings=True)
        if mt == "qwen2":
            kw.setdefault("attention_bias", True)
        if mt == "granite":
            kw.setdefault("embedding_multiplier", d.get("embedding_multiplier", 1.0))
        if mt == "bloom":
            kw.update(norm_type="layernorm", alibi=True, embed_norm=True, attention_bias=True, mlp_bias=True, hidden_act="gelu_tanh",
                      tie_word_embeddings=True, hidden_size=d.get("hidden_size", d.get("n_embed", 4096)))
            kw["intermediate_size"] = 4 * kw["hidden_size"]
            kw.setdefault("max_position_embeddings", d.get("seq_length", 2048))
        if mt == "mpt":
            attn = d.get("attn_config", {}) or {}
            no_bias = d.get("no_bias", True)
            kw.update(hidden_size=d["d_model"], num_hidden_layers=d["n_layers"], num_attention_heads=d["n_heads"],
                      intermediate_size=int(d.get("expansion_ratio", 4) * d["d_model"]), max_position_embeddings=d.get("max_seq_len", 2048),
                      norm_type="layernorm_nobias" if no_bias else "layernorm", attention_bias=not no_bias, mlp_bias=not no_bias,
                      hidden_act="gelu", alibi=bool(attn.get("alibi", True)), alibi_bias_max=float(attn.get("alibi_bias_max", 8)),
                      clip_qkv=attn.get("clip_qkv"), learned_positions=not attn.get("alibi", True), tie_word_embeddings=True,
                      rms_norm_eps=d.get("layer_norm_epsilon", 1e-5))
            if attn.get("qk_ln"):
                raise NotImplementedError("mpt with qk_ln")
            ls = d.get("logit_scale")
            kw["logit_scale"] = 1.0 if ls is None else (float(d["d_model"]) ** -0.5 if ls == "inv_sqrt_d_model" else float(ls))
        if mt == "opt":
            if d.get("word_embed_proj_dim", d["hidden_size"]) != d["hidden_size"] or not d.get("do_layer_norm_before", True):
                raise NotImplementedError("opt with a projected embedding or post-layer-norm blocks (opt-350m)")
            kw.update(norm_type="layernorm", learned_positions=True, position_offset=2, attention_bias=d.get("enable_bias", True),
                      mlp_bias=d.get("enable_bias", True), hidden_act=d.get("activation_function", "relu"), intermediate_size=d["ffn_dim"],
                      tie_word_embeddings=d.get("tie_word_embeddings", True))
        if mt == "qwen":
            # first-generation Qwen: intermediate_size counts both halves of the gated MLP; fused c_attn with bias
            kw.update(intermediate_size=d["intermediate_size"] // 2, attention_bias=True, head_dim=d.get("kv_channels"),
                      max_position_embeddings=d.get("seq_length", d.get("max_position_embeddings", 8192)),
                      tie_word_embeddings=d.get("tie_word_embeddings", False))
        if mt == "dbrx":
            ffn = d.get("ffn_config", {})
            attn = d.get("attn_config", {})
            kw.update(hidden_size=d["d_model"], num_hidden_layers=d["n_layers"], num_attention_heads=d["n_heads"],
                      num_key_value_heads=attn.get("kv_n_heads", d["n_heads"]),
                      intermediate_size=ffn.get("ffn_hidden_size", 4 * d["d_model"]),
                      num_local_experts=ffn.get("moe_num_experts", 0), num_experts_per_tok=ffn.get("moe_top_k", 0),
                      rope_theta=attn.get("rope_theta", 10000.0), norm_type="layernorm_nobias", clip_qkv=attn.get("clip_qkv"),
                      max_position_embeddings=d.get("max_seq_len", 2048))
        kw["model_type"] = mt
        kw["extra"] = extra
        return cls(**kw)

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        d = dataclasses.asdict(self)
        d.update(d.pop("extra"))
        return d


def mistral_7b() -> ModelConfig:
    """Mistral-7B-v0.1 architecture (the headline benchmark model)."""
    return ModelConfig(model_type="mistral", vocab_size=32000, hidden_size=4096, intermediate_size=14336,
                       num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=32768, sliding_window=4096)


def llama3_8b() -> ModelConfig:
    return ModelConfig(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                       num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192)


def llama3_70b() -> ModelConfig:
    return ModelConfig(model_type="llama", vocab_size=128256, hidden_size=8192, intermediate_size=28672,
                       num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                       rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192)


def mixtral_8x7b() -> ModelConfig:
    return ModelConfig(model_type="mixtral", vocab_size=32000, hidden_size=4096, intermediate_size=14336,
                       num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       rms_norm_eps=1e-5, rope_theta=1e6, max_position_embeddings=32768,
                       num_local_experts=8, num_experts_per_tok=2)


def tiny_llama(vocab_size: int = 32000) -> ModelConfig:
    """The CPU plumbing model: 2 layers, hidden 256, 4 heads, 2 KV heads, intermediate 688."""
    return ModelConfig(model_type="llama", vocab_size=vocab_size, hidden_size=256, intermediate_size=688,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                       rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=2048, torch_dtype="float32")


def _env(name: str, default, cast=None):
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    if cast is bool:
        return v.lower() in ("1", "true", "yes", "on")
    return (cast or type(default))(v)


@dataclass
class EngineConfig:
    """Serving knobs.  Defaults follow `launcher/src/main.rs:413-560` of the reference."""

    model_id: str = ""
    revision: Optional[str] = None
    source: str = "hub"
    adapter_source: str = "hub"
    default_adapter_source: Optional[str] = None
    dtype: Optional[str] = None
    quantize: Optional[str] = None
    kv_cache_dtype: Optional[str] = None            # "fp8": e4m3 pages with per-layer k / v scales (None: the model's dtype)
    num_shard: int = 1
    max_concurrent_requests: int = 1024
    max_best_of: int = 2
    max_stop_sequences: int = 4
    max_input_length: int = 1024
    max_total_tokens: int = 2048
    max_batch_prefill_tokens: int = 4096
    max_batch_total_tokens: Optional[int] = None
    waiting_served_ratio: float = 1.2
    max_waiting_tokens: int = 20
    # in-process engine, saturated queue: let this many rows drain (for at most that many decode steps) before new prompts
    # interrupt the running batch, so that one prefill pass serves several prompts and most steps stay pure decode graphs
    prefill_min_rows: int = 8
    prefill_max_wait_steps: int = 8
    max_active_adapters: int = 1024
    adapter_cycle_time_s: int = 2
    adapter_memory_fraction: float = 0.1
    eager_prefill: bool = True
    prefix_caching: bool = False
    chunked_prefill: bool = False
    speculative_tokens: int = 0
    speculation_max_batch_size: int = 32
    compile: bool = True                      # CUDA-graph the decode step
    compile_max_batch_size: int = 256
    compile_max_rank: int = 64
    cuda_memory_fraction: float = 1.0
    memory_wiggle_room: float = 0.9
    block_size: int = 32                      # KV page size in tokens
    host_adapter_cache_gb: float = 16.0       # pinned host tier for adapter exchange
    preloaded_adapter_ids: List[str] = field(default_factory=list)
    preloaded_adapter_source: Optional[str] = None
    merge_adapter_weights: bool = False
    port: int = 3000
    hostname: str = "0.0.0.0"
    shard_uds_path: str = "/tmp/lorax-server"
    master_addr: str = "127.0.0.1"
    master_port: int = 29500
    otlp_endpoint: Optional[str] = None
    json_output: bool = False
    cors_allow_origin: List[str] = field(default_factory=list)
    watermark_gamma: float = 0.5
    watermark_delta: float = 2.0
    profiler_dir: Optional[str] = None
    tokenizer_config_path: Optional[str] = None
    fused_collectives: bool = True            # in-kernel NVLink collectives (False = NCCL baseline mode)

    @classmethod
    def from_env(cls, **overrides) -> "EngineConfig":
        c = cls()
        c.model_id = _env("MODEL_ID", c.model_id)
        c.num_shard = _env("NUM_SHARD", c.num_shard)
        c.quantize = _env("QUANTIZE", c.quantize, str)
        c.kv_cache_dtype = _env("KV_CACHE_DTYPE", c.kv_cache_dtype, str)
        c.dtype = _env("DTYPE", c.dtype, str)
        c.max_input_length = _env("MAX_INPUT_LENGTH", c.max_input_length)
        c.max_total_tokens = _env("MAX_TOTAL_TOKENS", c.max_total_tokens)
        c.max_batch_prefill_tokens = _env("MAX_BATCH_PREFILL_TOKENS", c.max_batch_prefill_tokens)
        c.max_batch_total_tokens = _env("MAX_BATCH_TOTAL_TOKENS", c.max_batch_total_tokens, int)
        c.waiting_served_ratio = _env("WAITING_SERVED_RATIO", c.waiting_served_ratio)
        c.max_waiting_tokens = _env("MAX_WAITING_TOKENS", c.max_waiting_tokens)
        c.max_active_adapters = _env("MAX_ACTIVE_ADAPTERS", c.max_active_adapters)
        c.adapter_cycle_time_s = _env("ADAPTER_CYCLE_TIME_S", c.adapter_cycle_time_s)
        c.adapter_memory_fraction = _env("ADAPTER_MEMORY_FRACTION", c.adapter_memory_fraction)
        c.prefix_caching = _env("PREFIX_CACHING", c.prefix_caching, bool)
        c.chunked_prefill = _env("CHUNKED_PREFILL", c.chunked_prefill, bool)
        c.speculative_tokens = _env("SPECULATIVE_TOKENS", c.speculative_tokens)
        c.speculation_max_batch_size = _env("LORAX_SPECULATION_MAX_BATCH_SIZE", c.speculation_max_batch_size)
        c.compile = _env("LORAX_COMPILE", c.compile, bool)
        c.compile_max_batch_size = _env("LORAX_COMPILE_MAX_BATCH_SIZE", c.compile_max_batch_size)
        c.compile_max_rank = _env("LORAX_COMPILE_MAX_RANK", c.compile_max_rank)
        c.cuda_memory_fraction = _env("CUDA_MEMORY_FRACTION", c.cuda_memory_fraction)
        c.memory_wiggle_room = _env("MEMORY_WIGGLE_ROOM", c.memory_wiggle_room)
        c.watermark_gamma = _env("WATERMARK_GAMMA", c.watermark_gamma)
        c.watermark_delta = _env("WATERMARK_DELTA", c.watermark_delta)
        c.profiler_dir = _env("LORAX_PROFILER_DIR", c.profiler_dir, str)
        c.master_addr = _env("MASTER_ADDR", c.master_addr)
        c.master_port = _env("MASTER_PORT", c.master_port)
        c.port = _env("PORT", c.port)
        for k, v in overrides.items():
            if v is not None:
                if not hasattr(c, k):
                    raise KeyError(f"unknown engine option {k!r}")
                setattr(c, k, v)
        return c
