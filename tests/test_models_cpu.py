"""Architecture coverage on CPU: the config-driven decoder against HuggingFace implementations with the same
weights (Mixtral MoE, Qwen2 with QKV bias, Gemma with offset norms / tied embeddings), and merge strategies."""
import pytest
import torch

from lorax_b200.config import ModelConfig
from lorax_b200.models.decoder import DecoderModel
from lorax_b200.models.loading import export_hf_state_dict
from lorax_b200.runtime.kv_cache import KVCache
from lorax_b200.runtime.runner import ModelRunner, PrefillItem


def _logits(model, ids):
    kv = KVCache(model.config.num_hidden_layers, 16, model.nkv, model.d, model.dtype, model.device)
    r = ModelRunner(model, kv, max_batch=2, max_seq_tokens=128, max_prefill_tokens=256, use_graphs=False)
    return r.prefill([PrefillItem(ids, 0, [1, 2, 3], all_logprobs=True)])[2]


def test_mixtral_matches_hf():
    from transformers import MixtralConfig, MixtralForCausalLM
    cfg = ModelConfig(model_type="mixtral", vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=16, rope_theta=1e4, max_position_embeddings=256,
                      num_local_experts=4, num_experts_per_tok=2, torch_dtype="float32")
    m = DecoderModel.random_init(cfg, "cpu", torch.float32, seed=1, std=0.1)
    hc = MixtralConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=16, rope_theta=1e4, max_position_embeddings=256, num_local_experts=4,
                       num_experts_per_tok=2, rms_norm_eps=cfg.rms_norm_eps, sliding_window=None, tie_word_embeddings=False)
    hc._attn_implementation = "eager"
    hf = MixtralForCausalLM(hc).eval()
    sd = export_hf_state_dict(m)
    hsd = hf.state_dict()
    mapped = {}
    for k, v in sd.items():
        if k in hsd:
            mapped[k] = v
    # newer transformers fuse the experts into 3-D tensors: [E, 2I, H] (gate|up) and [E, H, I]
    for i in range(2):
        pre = f"model.layers.{i}.block_sparse_moe." if f"model.layers.{i}.block_sparse_moe.gate.weight" in hsd else f"model.layers.{i}.mlp."
        if pre + "experts.gate_up_proj" in hsd:
            mapped[pre + "experts.gate_up_proj"] = m.layers[i].experts_w13
            mapped[pre + "experts.down_proj"] = m.layers[i].experts_w2
            mapped[pre + "gate.weight"] = m.layers[i].router_w
    missing = [k for k in hsd if k not in mapped and "rotary" not in k]
    if missing:
        pytest.skip(f"this transformers version lays Mixtral out differently: {missing[:3]}")
    hf.load_state_dict(mapped, strict=False)
    ids = torch.randint(0, 300, (23,), generator=torch.Generator().manual_seed(0)).tolist()
    with torch.no_grad():
        want = hf(torch.tensor([ids])).logits[0]
    got = _logits(m, ids)
    assert torch.allclose(got, want, atol=2e-3, rtol=1e-3), (got - want).abs().max()


def test_qwen2_bias_matches_hf():
    from transformers import Qwen2Config, Qwen2ForCausalLM
    cfg = ModelConfig.from_dict(dict(model_type="qwen2", vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                     num_attention_heads=4, num_key_value_heads=2, rope_theta=1e4, max_position_embeddings=256,
                                     rms_norm_eps=1e-6, torch_dtype="float32"))
    assert cfg.attention_bias
    m = DecoderModel.random_init(cfg, "cpu", torch.float32, seed=2, std=0.1)
    hc = Qwen2Config(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     rope_theta=1e4, max_position_embeddings=256, rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False)
    hc._attn_implementation = "eager"
    hf = Qwen2ForCausalLM(hc).eval()
    missing, _ = hf.load_state_dict(export_hf_state_dict(m), strict=False)
    assert not [k for k in missing if "rotary" not in k], missing
    ids = torch.randint(0, 300, (19,), generator=torch.Generator().manual_seed(0)).tolist()
    with torch.no_grad():
        want = hf(torch.tensor([ids])).logits[0]
    assert torch.allclose(_logits(m, ids), want, atol=2e-3, rtol=1e-3)


def test_gemma_matches_hf():
    from transformers import GemmaConfig, GemmaForCausalLM
    cfg = ModelConfig.from_dict(dict(model_type="gemma", vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                     num_attention_heads=4, num_key_value_heads=1, head_dim=16, rope_theta=1e4,
                                     max_position_embeddings=256, rms_norm_eps=1e-6, hidden_act="gelu_pytorch_tanh", torch_dtype="float32"))
    m = DecoderModel.random_init(cfg, "cpu", torch.float32, seed=3, std=0.1)
    hc = GemmaConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                     head_dim=16, rope_theta=1e4, max_position_embeddings=256, rms_norm_eps=1e-6, hidden_activation="gelu_pytorch_tanh")
    hc._attn_implementation = "eager"
    hf = GemmaForCausalLM(hc).eval()
    missing, _ = hf.load_state_dict(export_hf_state_dict(m), strict=False)
    assert not [k for k in missing if "rotary" not in k and "lm_head" not in k], missing
    ids = torch.randint(0, 300, (21,), generator=torch.Generator().manual_seed(0)).tolist()
    with torch.no_grad():
        want = hf(torch.tensor([ids])).logits[0]
    assert torch.allclose(_logits(m, ids), want, atol=3e-3, rtol=1e-3)


def test_merge_strategies():
    from lorax_b200.adapters.merges import merge_tensors
    a = torch.tensor([[1.0, -2.0, 0.1], [0.0, 3.0, -0.2]])
    b = torch.tensor([[-1.0, -1.0, 0.3], [2.0, -3.0, 0.2]])
    lin = merge_tensors([a, b], [0.5, 0.5], "linear")
    assert torch.allclose(lin, (a + b) / 2)
    ties = merge_tensors([a, b], [1.0, 1.0], "ties", density=1.0)
    # sign election by total mass, then mean of the agreeing entries
    assert ties[0, 1].item() == pytest.approx(-1.5) and ties[1, 1].item() in (3.0, -3.0) and ties[0, 0].item() in (1.0, -1.0)
    pruned = merge_tensors([a], [1.0], "ties", density=0.34)
    assert (pruned != 0).sum().item() == 2
    torch.manual_seed(0)
    big = torch.ones(1000)
    dare = merge_tensors([big], [1.0], "dare_linear", density=0.5, generator=torch.Generator().manual_seed(0))
    assert 0.8 < dare.mean().item() < 1.2 and set(dare.unique().tolist()) <= {0.0, 2.0}
