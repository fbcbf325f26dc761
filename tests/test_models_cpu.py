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
    # the sign is elected before the weights are applied: a negative weight flips the contribution, not the election
    t1, t2 = torch.tensor([2.0, -1.0]), torch.tensor([-1.0, -3.0])
    got = merge_tensors([t1, t2], [1.0, -2.0], "ties", density=1.0)
    # position 0: unweighted sum +1 elects "+", only t1 agrees -> 2.0; position 1: both negative -> mean(-1, +6) = 2.5
    assert got.tolist() == pytest.approx([2.0, 2.5])
    pruned = merge_tensors([a], [1.0], "ties", density=0.34)
    assert (pruned != 0).sum().item() == 2
    torch.manual_seed(0)
    big = torch.ones(1000)
    dare = merge_tensors([big], [1.0], "dare_linear", density=0.5, generator=torch.Generator().manual_seed(0))
    assert 0.8 < dare.mean().item() < 1.2 and set(dare.unique().tolist()) <= {0.0, 2.0}


def test_repetition_penalty_reaches_token_zero_in_padded_batches():
    """Rows with shorter histories are padded with id 0 / mask False; that padding must not hide a real token 0."""
    from lorax_b200.sampling.chooser import HeterogeneousNextTokenChooser, NextTokenParams
    ch = HeterogeneousNextTokenChooser([NextTokenParams(repetition_penalty=2.0), NextTokenParams(repetition_penalty=2.0)], "cpu", 8)
    hist = torch.tensor([[0, 3, 0, 0, 0], [5, 6, 7, 1, 2]])
    mask = torch.tensor([[True, True, False, False, False], [True] * 5])
    scores = torch.ones(2, 8)
    out = ch.warp(hist, mask, scores.clone())
    assert out[0, 0].item() == 0.5 and out[0, 3].item() == 0.5 and out[0, 1].item() == 1.0
    assert out[1, 0].item() == 1.0 and out[1, 5].item() == 0.5


def test_fp8_block128_quantiser_roundtrip(tmp_path):
    """128 x 128 block scales: the round trip stays within e4m3 precision even with an outlier block, and the
    checkpoint quantiser writes fp8 tensors plus `_scale_inv` tensors and marks the config."""
    import json
    import torch
    from safetensors.torch import load_file, save_file
    from lorax_b200.ops import reference as ref
    from lorax_b200.utils.quantize import dequantize_state_dict, quantize_checkpoint

    torch.manual_seed(0)
    w = torch.randn(300, 520) * 0.05
    w[:128, :128] *= 50.0                      # an outlier block must not cost the others their precision
    q, s = ref.quantize_weight_fp8_block128(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (3, 5)
    back = ref.dequantize_weight_fp8_block128(q, s)
    rel = ((back - w).abs() / w.abs().clamp_min(1e-3))
    assert rel[200:, 300:].median().item() < 0.04 and (back - w).abs().max().item() <= w.abs().max().item() * 0.07
    x = torch.randn(5, 520).to(torch.bfloat16)
    y = ref.gemm_fp8(x, q, s)
    want = x.float() @ w.t()
    assert ((y.float() - want).norm() / want.norm()).item() < 0.05

    src, dst = tmp_path / "m", tmp_path / "q"
    src.mkdir()
    sd = {"model.layers.0.self_attn.q_proj.weight": torch.randn(256, 256).to(torch.bfloat16),
          "model.layers.0.input_layernorm.weight": torch.ones(256).to(torch.bfloat16),
          "model.embed_tokens.weight": torch.randn(512, 256).to(torch.bfloat16)}
    save_file(sd, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps({"model_type": "llama"}))
    stats = quantize_checkpoint(str(src), str(dst))
    assert stats == {"tensors": 3, "quantized": 1}
    out = load_file(str(dst / "model.safetensors"))
    assert out["model.layers.0.self_attn.q_proj.weight"].dtype == torch.float8_e4m3fn
    assert out["model.layers.0.self_attn.q_proj.weight_scale_inv"].shape == (2, 2)
    assert out["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert json.loads((dst / "config.json").read_text())["quantization_config"]["weight_block_size"] == [128, 128]
    deq = dequantize_state_dict(out)
    err = (deq["model.layers.0.self_attn.q_proj.weight"].float() - sd["model.layers.0.self_attn.q_proj.weight"].float()).abs().max()
    assert err.item() < 0.3


def test_encoders_match_hf():
    """BERT / RoBERTa embeddings (first-token hidden state) and DistilBERT token classification against HuggingFace,
    ragged batch of three sequences."""
    from transformers import BertConfig, BertModel, DistilBertConfig, DistilBertForTokenClassification, RobertaConfig, RobertaModel
    from lorax_b200.models.encoder import EncoderConfig, EncoderModel, random_encoder_state_dict
    from lorax_b200.utils.weights import InMemoryWeights

    torch.manual_seed(0)
    seqs = [[5, 9, 77, 3, 12], [101, 7, 8], [4, 4, 250, 17, 90, 33, 2, 6]]

    # ---- BERT
    hc = BertConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                    max_position_embeddings=64, type_vocab_size=2)
    hc._attn_implementation = "eager"
    cfg = EncoderConfig.from_dict(hc.to_dict())
    sd = random_encoder_state_dict(cfg, seed=1)
    hf = BertModel(hc, add_pooling_layer=False).eval()
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not missing and not unexpected
    ours = EncoderModel.from_weights(cfg, InMemoryWeights(sd), "cpu", torch.float32)
    got = torch.tensor(ours.embed(seqs))
    with torch.no_grad():
        want = torch.stack([hf(torch.tensor([s])).last_hidden_state[0, 0] for s in seqs])
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()

    # ---- RoBERTa (positions start at pad_token_id + 1)
    rc = RobertaConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                       max_position_embeddings=66, type_vocab_size=1, pad_token_id=1)
    rc._attn_implementation = "eager"
    cfg = EncoderConfig.from_dict(rc.to_dict())
    sd = random_encoder_state_dict(cfg, seed=2)
    hf = RobertaModel(rc, add_pooling_layer=False).eval()
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not missing and not unexpected
    ours = EncoderModel.from_weights(cfg, InMemoryWeights({"roberta." + k: v for k, v in sd.items()}), "cpu", torch.float32)
    got = torch.tensor(ours.embed(seqs))
    with torch.no_grad():
        want = torch.stack([hf(torch.tensor([s])).last_hidden_state[0, 0] for s in seqs])
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()

    # ---- DistilBERT token classification
    dc = DistilBertConfig(vocab_size=300, dim=64, n_layers=2, n_heads=4, hidden_dim=128, max_position_embeddings=64, num_labels=5,
                          id2label={i: f"T{i}" for i in range(5)}, label2id={f"T{i}": i for i in range(5)})
    dc._attn_implementation = "eager"
    cfg = EncoderConfig.from_dict(dc.to_dict())
    sd = random_encoder_state_dict(cfg, seed=3, num_labels=5)
    hf = DistilBertForTokenClassification(dc).eval()
    missing, unexpected = hf.load_state_dict({("distilbert." + k if not k.startswith("classifier") else k): v for k, v in sd.items()},
                                             strict=False)
    assert not missing and not unexpected
    ours = EncoderModel.from_weights(cfg, InMemoryWeights({("distilbert." + k if not k.startswith("classifier") else k): v
                                                           for k, v in sd.items()}), "cpu", torch.float32)
    labels, scores = ours.classify(seqs)
    for s, lab, sc in zip(seqs, labels, scores):
        with torch.no_grad():
            p = torch.softmax(hf(torch.tensor([s])).logits[0], -1)
        conf, pred = p.max(-1)
        assert lab == [f"T{i}" for i in pred.tolist()]
        assert torch.allclose(torch.tensor(sc), conf, atol=2e-4)


def _from_hf(hf, max_positions=None, **over):
    """Our decoder loaded from a HuggingFace model's own state dict and config."""
    from lorax_b200.utils.weights import InMemoryWeights
    d = hf.config.to_dict()
    d.update(over)
    cfg = ModelConfig.from_dict(d)
    cfg.torch_dtype = "float32"
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    return DecoderModel.from_weights(cfg, InMemoryWeights(sd, dtype=torch.float32), "cpu", torch.float32, max_positions=max_positions)


def _check_against_hf(hf, model, vocab, n=23, tol=2e-3):
    torch.manual_seed(1)
    ids = torch.randint(0, vocab, (n,)).tolist()
    with torch.no_grad():
        want = hf(torch.tensor([ids])).logits[0]
    got = _logits(model, ids)
    assert got.shape == want.shape
    assert (got - want).abs().max().item() < tol * max(1.0, want.abs().max().item()), (got - want).abs().max()


def test_bloom_alibi_matches_hf():
    """ALiBi bias in the attention scores, LayerNorm on the embeddings, interleaved fused QKV, 6 heads (not a power of two)."""
    from transformers import BloomConfig, BloomForCausalLM
    torch.manual_seed(0)
    hc = BloomConfig(vocab_size=200, hidden_size=96, n_layer=2, n_head=6, layer_norm_epsilon=1e-5)
    hc._attn_implementation = "eager"
    hf = BloomForCausalLM(hc).eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.08)
    m = _from_hf(hf)
    assert m.alibi_slopes is not None and m.embed_norm is not None and m.alibi_slopes.shape[0] == 6
    _check_against_hf(hf, m, 200)


def test_mpt_alibi_matches_hf():
    from transformers import MptConfig, MptForCausalLM
    torch.manual_seed(0)
    hc = MptConfig(d_model=64, n_heads=4, n_layers=2, expansion_ratio=4, max_seq_len=128, vocab_size=180, no_bias=True)
    hc._attn_implementation = "eager"
    hf = MptForCausalLM(hc).eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.08)
    m = _from_hf(hf)
    assert m.alibi_slopes is not None and m.pos_embed is None
    _check_against_hf(hf, m, 180)


def test_opt_matches_hf():
    """Learned positions with OPT's offset of two, ReLU MLP, biased projections."""
    from transformers import OPTConfig, OPTForCausalLM
    torch.manual_seed(0)
    hc = OPTConfig(vocab_size=190, hidden_size=64, ffn_dim=160, num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=96,
                   word_embed_proj_dim=64, do_layer_norm_before=True)
    hc._attn_implementation = "eager"
    hf = OPTForCausalLM(hc).eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.08)
    m = _from_hf(hf)
    assert m.pos_embed.shape[0] == 98 and m.config.hidden_act == "relu"
    _check_against_hf(hf, m, 190)


def test_qwen_v1_names_load_like_qwen2():
    """First-generation Qwen checkpoints (fused c_attn with bias, mlp.w2 = gate, mlp.w1 = up) against a Qwen2 model holding the
    same weights under its own names."""
    from transformers import Qwen2Config, Qwen2ForCausalLM
    from lorax_b200.utils.weights import InMemoryWeights
    torch.manual_seed(0)
    hc = Qwen2Config(vocab_size=210, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
                     max_position_embeddings=128, rope_theta=1e4, rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False)
    hc._attn_implementation = "eager"
    hf = Qwen2ForCausalLM(hc).eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.08)
    sd = hf.state_dict()
    q1 = {"transformer.wte.weight": sd["model.embed_tokens.weight"], "transformer.ln_f.weight": sd["model.norm.weight"],
          "lm_head.weight": sd["lm_head.weight"]}
    for i in range(2):
        a, b = f"model.layers.{i}.", f"transformer.h.{i}."
        q1[b + "ln_1.weight"] = sd[a + "input_layernorm.weight"]
        q1[b + "ln_2.weight"] = sd[a + "post_attention_layernorm.weight"]
        q1[b + "attn.c_attn.weight"] = torch.cat([sd[a + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0)
        q1[b + "attn.c_attn.bias"] = torch.cat([sd[a + f"self_attn.{n}_proj.bias"] for n in "qkv"], 0)
        q1[b + "attn.c_proj.weight"] = sd[a + "self_attn.o_proj.weight"]
        q1[b + "mlp.w2.weight"] = sd[a + "mlp.gate_proj.weight"]
        q1[b + "mlp.w1.weight"] = sd[a + "mlp.up_proj.weight"]
        q1[b + "mlp.c_proj.weight"] = sd[a + "mlp.down_proj.weight"]
    cfg = ModelConfig.from_dict({"model_type": "qwen", "vocab_size": 210, "hidden_size": 64, "intermediate_size": 224, "num_hidden_layers": 2,
                                 "num_attention_heads": 4, "kv_channels": 16, "layer_norm_epsilon": 1e-6, "rotary_emb_base": 1e4,
                                 "seq_length": 128, "torch_dtype": "float32"})
    assert cfg.intermediate_size == 112 and cfg.attention_bias
    m = DecoderModel.from_weights(cfg, InMemoryWeights({k: v.detach().clone() for k, v in q1.items()}, dtype=torch.float32), "cpu", torch.float32)
    _check_against_hf(hf, m, 210)


def test_dbrx_names_load_like_mixtral():
    """DBRX checkpoints (fused clamped Wqkv, LayerNorm without bias, experts stacked along rows as w1 / v1 / w2 of shape
    [E * I, H]) against the same weights under Mixtral's per-expert names in a model with the same switches.  (The DBRX class of
    the installed transformers multiplies by the untransposed expert matrices and only runs with I == H, so it is no oracle.)"""
    from lorax_b200.utils.weights import InMemoryWeights
    E, I, H = 4, 96, 64
    base = dict(vocab_size=170, hidden_size=H, intermediate_size=I, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                head_dim=16, rope_theta=1e4, max_position_embeddings=128, num_local_experts=E, num_experts_per_tok=2, torch_dtype="float32",
                norm_type="layernorm_nobias", clip_qkv=0.6)
    mix = DecoderModel.random_init(ModelConfig(model_type="mixtral", **base), "cpu", torch.float32, seed=3, std=0.1)
    sd = export_hf_state_dict(mix)
    dsd = {"transformer.wte.weight": sd["model.embed_tokens.weight"], "transformer.norm_f.weight": sd["model.norm.weight"],
           "lm_head.weight": sd["lm_head.weight"]}
    for i in range(2):
        a, b = f"model.layers.{i}.", f"transformer.blocks.{i}."
        dsd[b + "norm_attn_norm.norm_1.weight"] = sd[a + "input_layernorm.weight"]
        dsd[b + "norm_attn_norm.norm_2.weight"] = sd[a + "post_attention_layernorm.weight"]
        dsd[b + "norm_attn_norm.attn.Wqkv.weight"] = torch.cat([sd[a + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0)
        dsd[b + "norm_attn_norm.attn.out_proj.weight"] = sd[a + "self_attn.o_proj.weight"]
        dsd[b + "ffn.router.layer.weight"] = sd[a + "block_sparse_moe.gate.weight"]
        ex = a + "block_sparse_moe.experts."
        dsd[b + "ffn.experts.mlp.w1"] = torch.cat([sd[ex + f"{e}.w1.weight"] for e in range(E)], 0)
        dsd[b + "ffn.experts.mlp.v1"] = torch.cat([sd[ex + f"{e}.w3.weight"] for e in range(E)], 0)
        dsd[b + "ffn.experts.mlp.w2"] = torch.cat([sd[ex + f"{e}.w2.weight"].t() for e in range(E)], 0)
    cfg = ModelConfig.from_dict({"model_type": "dbrx", "d_model": H, "n_heads": 4, "n_layers": 2, "max_seq_len": 128, "vocab_size": 170,
                                 "attn_config": {"kv_n_heads": 2, "clip_qkv": 0.6, "rope_theta": 1e4},
                                 "ffn_config": {"ffn_hidden_size": I, "moe_num_experts": E, "moe_top_k": 2}, "torch_dtype": "float32"})
    assert cfg.clip_qkv == 0.6 and cfg.num_local_experts == E and cfg.norm_type == "layernorm_nobias"
    dbrx = DecoderModel.from_weights(cfg, InMemoryWeights(dsd, dtype=torch.float32), "cpu", torch.float32)
    ids = list(range(7, 40))
    a, b = _logits(mix, ids), _logits(dbrx, ids)
    assert torch.allclose(a, b, atol=1e-5)
    # the clamp is live: without it the logits move
    mix.config.clip_qkv = None
    assert not torch.allclose(_logits(mix, ids), b, atol=1e-4)


@pytest.mark.parametrize("ff,tied", [("relu", True), ("gated-gelu", False)])
def test_t5_matches_hf(ff, tied):
    """Encoder-decoder path: greedy tokens and first-step logits against T5ForConditionalGeneration (both feed-forward variants,
    tied and separate lm_head)."""
    from transformers import T5Config, T5ForConditionalGeneration
    from lorax_b200.models.seq2seq import Seq2SeqConfig, Seq2SeqModel
    from lorax_b200.utils.weights import InMemoryWeights
    torch.manual_seed(0)
    hc = T5Config(vocab_size=150, d_model=48, d_kv=12, d_ff=96, num_layers=2, num_decoder_layers=3, num_heads=4,
                  relative_attention_num_buckets=8, relative_attention_max_distance=20, feed_forward_proj=ff, tie_word_embeddings=tied,
                  decoder_start_token_id=0, eos_token_id=1, pad_token_id=0)
    hf = T5ForConditionalGeneration(hc).eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.3)
    d = hc.to_dict()
    d["tie_word_embeddings"] = tied          # as the checkpoint's config.json says it (transformers rewrites the attribute to True)
    cfg = Seq2SeqConfig.from_dict(d)
    assert cfg.num_decoder_layers == 3 and cfg.feed_forward_proj == ff
    m = Seq2SeqModel.from_weights(cfg, InMemoryWeights({k: v.detach().clone() for k, v in hf.state_dict().items()}, dtype=torch.float32),
                                  "cpu", torch.float32)
    ids = torch.randint(2, 150, (1, 37))
    with torch.no_grad():
        want_logits = hf(input_ids=ids, decoder_input_ids=torch.tensor([[0]])).logits[0, 0]
        want, dec = [], [0]
        for _ in range(10):                                  # greedy by re-running the decoder over the whole prefix (no cache)
            tok = int(hf(input_ids=ids, decoder_input_ids=torch.tensor([dec]), use_cache=False).logits[0, -1].argmax())
            want.append(tok)
            dec.append(tok)
            if tok == 1:
                break
    st = m.encode(ids[0].tolist())
    got_logits = m.decode_step([st])[0]
    assert (got_logits - want_logits).abs().max().item() < 2e-3 * max(1.0, want_logits.abs().max().item())
    got = m.generate(ids[0].tolist(), max_new_tokens=10)
    assert got == want
    # two requests of different lengths stepped together equal the same requests stepped alone
    a, b = m.encode(ids[0, :9].tolist()), m.encode(ids[0].tolist())
    for _ in range(3):
        lg = m.decode_step([a, b])
        for s, row in zip((a, b), lg):
            s.last_token, s.position = int(row.argmax()), s.position + 1
    assert [b.last_token] == got[2:3]


def _family(name):
    """A two-layer HuggingFace model of one architecture variant, with every parameter (biases and norm weights
    included) drawn at random so that a tensor the loader drops or misplaces shows in the logits."""
    import transformers as T
    common = dict(vocab_size=200, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=128)
    llama = dict(common, intermediate_size=96, num_key_value_heads=2)
    table = {
        "llama3_rope": (T.LlamaForCausalLM, T.LlamaConfig, dict(llama, rope_theta=5e5, rope_scaling=dict(
            rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=32))),
        "llama_yarn": (T.LlamaForCausalLM, T.LlamaConfig, dict(llama, rope_scaling=dict(
            rope_type="yarn", factor=4.0, original_max_position_embeddings=32))),
        "llama_linear": (T.LlamaForCausalLM, T.LlamaConfig, dict(llama, rope_scaling=dict(rope_type="linear", factor=2.0))),
        "llama_dynamic_ntk": (T.LlamaForCausalLM, T.LlamaConfig, dict(llama, max_position_embeddings=16,
                                                                       rope_scaling=dict(rope_type="dynamic", factor=2.0))),
        "llama_biases": (T.LlamaForCausalLM, T.LlamaConfig, dict(llama, attention_bias=True, mlp_bias=True)),
        "mistral_window": (T.MistralForCausalLM, T.MistralConfig, dict(llama, sliding_window=8)),
        "phi3": (T.Phi3ForCausalLM, T.Phi3Config, dict(llama, pad_token_id=0)),
        "phi3_longrope": (T.Phi3ForCausalLM, T.Phi3Config, dict(
            llama, pad_token_id=0, original_max_position_embeddings=16, rope_scaling=dict(
                type="longrope", short_factor=[1.0 + 0.1 * i for i in range(8)], long_factor=[2.0 + 0.3 * i for i in range(8)]))),
        "gemma2": (T.Gemma2ForCausalLM, T.Gemma2Config, dict(llama, head_dim=16, sliding_window=8, query_pre_attn_scalar=24,
                                                             attn_logit_softcapping=20.0, final_logit_softcapping=10.0)),
        "cohere": (T.CohereForCausalLM, T.CohereConfig, dict(llama, logit_scale=0.25)),
        "granite": (T.GraniteForCausalLM, T.GraniteConfig, dict(llama, embedding_multiplier=3.0, logits_scaling=2.0,
                                                                residual_multiplier=0.5, attention_multiplier=0.1)),
        "gpt2": (T.GPT2LMHeadModel, T.GPT2Config, dict(vocab_size=200, n_embd=64, n_layer=2, n_head=4, n_positions=128)),
        "gpt_bigcode": (T.GPTBigCodeForCausalLM, T.GPTBigCodeConfig, dict(vocab_size=200, n_embd=64, n_layer=2, n_head=4,
                                                                          n_positions=128, multi_query=True)),
        "gpt_neox_parallel": (T.GPTNeoXForCausalLM, T.GPTNeoXConfig, dict(common, intermediate_size=160, rotary_pct=0.25,
                                                                          use_parallel_residual=True)),
        "gpt_neox_sequential": (T.GPTNeoXForCausalLM, T.GPTNeoXConfig, dict(common, intermediate_size=160, rotary_pct=0.5,
                                                                            use_parallel_residual=False)),
        "falcon_7b": (T.FalconForCausalLM, T.FalconConfig, dict(common, multi_query=True, parallel_attn=True, bias=False,
                                                                new_decoder_architecture=False, alibi=False)),
        "falcon_40b": (T.FalconForCausalLM, T.FalconConfig, dict(common, num_kv_heads=2, parallel_attn=True, bias=False,
                                                                 new_decoder_architecture=True, alibi=False)),
        "falcon_rw": (T.FalconForCausalLM, T.FalconConfig, dict(common, multi_query=False, parallel_attn=False, bias=True,
                                                                new_decoder_architecture=False, alibi=False)),
        "phi": (T.PhiForCausalLM, T.PhiConfig, dict(common, intermediate_size=160, partial_rotary_factor=0.5)),
    }
    cls, cfg_cls, kw = table[name]
    torch.manual_seed(0)
    hc = cfg_cls(**kw)
    hc._attn_implementation = "eager"
    hf = cls(hc).eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.08)
    return hf


@pytest.mark.parametrize("name", ["llama3_rope", "llama_yarn", "llama_linear", "llama_dynamic_ntk", "llama_biases", "mistral_window", "phi3",
                                  "phi3_longrope", "gemma2", "cohere", "granite", "gpt2", "gpt_bigcode", "gpt_neox_parallel",
                                  "gpt_neox_sequential", "falcon_7b", "falcon_40b", "falcon_rw", "phi"])
def test_decoder_family_matches_hf(name):
    """Every decoder architecture the registry names that has no test of its own above, loaded from a HuggingFace model's own
    state dict and config: prompt logits over 23 tokens equal HuggingFace's eager implementation.  The variants pin the RoPE
    scalings (llama3, YaRN, linear, dynamic NTK, LongRoPE), sliding windows (every layer for mistral, alternate layers for
    gemma2), both soft caps of gemma2, the multipliers of granite and cohere, fused and interleaved QKV packings, and the three
    falcon block layouts."""
    hf = _family(name)
    # dynamic NTK stretches the rotary base with the table length; HuggingFace stretches it with the sequence length
    m = _from_hf(hf, max_positions=23 if name == "llama_dynamic_ntk" else None)
    _check_against_hf(hf, m, 200)
