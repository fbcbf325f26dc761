"""CPU plumbing slice: tiny Llama, 4 random PEFT LoRA adapters, a heterogeneous batch of 8 requests decoded
greedily through the engine, checked token-exactly against HuggingFace `LlamaForCausalLM` with every adapter
merged by hand (W + alpha/r * B A) and every request run alone."""
import pytest
import torch

from lorax_b200.adapters.lora import load_peft_adapter, random_adapter, save_peft_adapter
from lorax_b200.adapters.manager import AdapterManager
from lorax_b200.config import EngineConfig, tiny_llama
from lorax_b200.models.decoder import DecoderModel
from lorax_b200.models.loading import export_hf_state_dict
from lorax_b200.runtime.engine import Engine, GenRequest


def _hf_model(cfg, sd):
    from transformers import LlamaConfig, LlamaForCausalLM
    hc = LlamaConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                     num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
                     num_key_value_heads=cfg.num_key_value_heads, rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta,
                     max_position_embeddings=cfg.max_position_embeddings, tie_word_embeddings=False, attention_bias=False)
    hc._attn_implementation = "eager"
    m = LlamaForCausalLM(hc).to(torch.float32).eval()
    missing, unexpected = m.load_state_dict(sd, strict=False)
    assert not [k for k in missing if "rotary" not in k], missing
    return m


def _merge(sd, cfg_a, mm):
    out = dict(sd)
    for mod, ab in mm.items():
        key = mod + ".weight"
        out[key] = out[key] + cfg_a.scale * (ab["lora_B"].float() @ ab["lora_A"].float())
    return out


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    torch.manual_seed(0)
    cfg = tiny_llama()
    model = DecoderModel.random_init(cfg, "cpu", torch.float32, seed=0)
    mgr = AdapterManager(model, arena_bytes=64 << 20, host_bytes=256 << 20)
    adapters = []
    root = tmp_path_factory.mktemp("adapters")
    for i in range(4):
        # B is drawn larger than the 0.02 of the benchmark config so that adapters visibly change the tokens
        c, mm = random_adapter(cfg, r=8, alpha=16, target_modules=["q_proj", "v_proj"], seed=100 + i, std_a=0.05, std_b=0.05)
        save_peft_adapter(root / f"a{i}", c, mm)
        c2, mm2 = load_peft_adapter(root / f"a{i}")
        mgr.register(f"a{i}", c2, mm2)
        assert mgr.load(i + 1, f"a{i}")
        adapters.append((c2, mm2))
    return cfg, model, mgr, adapters


def test_heterogeneous_batch_matches_hf(setup):
    cfg, model, mgr, adapters = setup
    g = torch.Generator().manual_seed(1)
    prompts = []
    for i in range(8):
        n = int(torch.randint(16, 65, (1,), generator=g))
        prompts.append(torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist())
    adapter_idx = [i % 5 for i in range(8)]
    eng = Engine(model, EngineConfig(max_total_tokens=256, max_batch_prefill_tokens=1024), num_blocks=128, max_batch=8)
    outs = eng.generate(prompts, max_new_tokens=32, adapter_indices=adapter_idx)
    base_sd = export_hf_state_dict(model)
    n_diff_from_base = 0
    hf_base = _hf_model(cfg, base_sd)
    for i, (p, a) in enumerate(zip(prompts, adapter_idx)):
        hf = hf_base if a == 0 else _hf_model(cfg, _merge(base_sd, *adapters[a - 1]))
        with torch.no_grad():
            ref = hf.generate(torch.tensor([p]), max_new_tokens=32, do_sample=False, pad_token_id=0, eos_token_id=None)[0, len(p):].tolist()
            if a != 0:
                base_out = hf_base.generate(torch.tensor([p]), max_new_tokens=32, do_sample=False, pad_token_id=0, eos_token_id=None)[0, len(p):].tolist()
                n_diff_from_base += int(base_out != ref)
        assert outs[i] == ref, (i, a, outs[i], ref)
    assert n_diff_from_base >= 3      # the adapters matter


def test_logits_close_to_hf(setup):
    cfg, model, mgr, adapters = setup
    from lorax_b200.runtime.kv_cache import KVCache
    from lorax_b200.runtime.runner import ModelRunner, PrefillItem
    kv = KVCache(cfg.num_hidden_layers, 16, model.nkv, model.d, torch.float32, "cpu")
    runner = ModelRunner(model, kv, max_batch=4, max_seq_tokens=128, max_prefill_tokens=256)
    g = torch.Generator().manual_seed(2)
    p = torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist()
    _, _, logits = runner.prefill([PrefillItem(p, 0, [1, 2], adapter_index=2, all_logprobs=True)])
    hf = _hf_model(cfg, _merge(export_hf_state_dict(model), *adapters[1]))
    with torch.no_grad():
        want = hf(torch.tensor([p])).logits[0]
    assert torch.allclose(logits, want, atol=2e-4, rtol=1e-4)


def test_fp8_kv_cache_stays_close_to_the_full_precision_cache(setup):
    """`kv_cache_dtype="fp8"`: e4m3 pages with a K and a V scale per layer.  Prefill over a cached prefix and a decode step read
    the quantised pages; the logits stay within the quantisation error of the full-precision cache, and half the bytes per block
    are planned."""
    cfg, model, mgr, adapters = setup
    from lorax_b200.config import EngineConfig
    from lorax_b200.runtime.kv_cache import KVCache, kv_dtype_of
    from lorax_b200.runtime.runner import ModelRunner, PrefillItem
    ecfg = EngineConfig(kv_cache_dtype="fp8")
    saved = model.kv_scales
    try:
        assert kv_dtype_of(model, ecfg) == torch.float8_e4m3fn and len(model.kv_scales) == cfg.num_hidden_layers
        model.kv_scales = [(0.05, 0.03)] * cfg.num_hidden_layers
        g = torch.Generator().manual_seed(4)
        p = torch.randint(0, cfg.vocab_size, (50,), generator=g).tolist()
        outs = []
        for dtype in (torch.float32, torch.float8_e4m3fn):
            kv = KVCache(cfg.num_hidden_layers, 16, model.nkv, model.d, dtype, "cpu")
            runner = ModelRunner(model, kv, max_batch=4, max_seq_tokens=128, max_prefill_tokens=256)
            runner.prefill([PrefillItem(p[:33], 0, [1, 2], want_logits=False)])
            _, _, logits = runner.prefill([PrefillItem(p[33:], 33, [1, 2], all_logprobs=True)])      # reads the cached prefix
            outs.append(logits.float())
        assert KVCache.bytes_per_block(2, 4, 64, torch.float8_e4m3fn) * 4 == KVCache.bytes_per_block(2, 4, 64, torch.float32)
        err = (outs[0] - outs[1]).norm() / outs[0].norm()
        assert 0 < err < 0.1, err
        assert (outs[0].argmax(-1) == outs[1].argmax(-1)).float().mean() > 0.8
    finally:
        model.kv_scales = saved


def test_prefill_riding_on_decode_steps_gives_same_tokens(setup):
    """Requests that arrive while others decode are prefilled in the same forward pass as the decode rows (one pass
    over the weights for both).  Tokens must equal those of the run where prefill and decode are separate passes."""
    cfg, model, mgr, adapters = setup
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab_size, (int(torch.randint(8, 40, (1,), generator=g)),), generator=g).tolist() for _ in range(7)]
    adapter_idx = [(i * 2) % 5 for i in range(7)]
    new_tokens = [12, 1, 9, 14, 6, 10, 8]

    def run(mixed: bool):
        from lorax_b200.runtime.engine import GenRequest
        eng = Engine(model, EngineConfig(max_total_tokens=128, max_batch_prefill_tokens=512, waiting_served_ratio=0.0), num_blocks=128,
                     max_batch=8)
        eng.mixed_steps = mixed
        arrivals = {0: [0, 1, 2], 2: [3], 3: [4, 5], 7: [6]}
        step, n_mixed = 0, 0
        while step < 200 and (step <= 7 or not eng.idle):
            for i in arrivals.get(step, []):
                eng.add_request(GenRequest(i + 1, prompts[i], new_tokens[i], adapter_idx[i]))
            before = eng.runner.steps
            had_running = bool(eng.running)
            will_prefill = bool(eng.waiting)
            eng.step()
            n_mixed += int(mixed and had_running and will_prefill)
            step += 1
        assert eng.idle
        return [eng.finished[i + 1].output_ids for i in range(7)], n_mixed

    sep, _ = run(False)
    mix, n_mixed = run(True)
    assert n_mixed >= 2
    assert [len(o) for o in mix] == new_tokens
    assert mix == sep


def test_adapter_exchange_under_memory_pressure():
    """Six adapters, an HBM arena that holds two: the engine loads on demand and evicts the least recently used idle
    adapter.  Tokens equal the run in which every adapter is resident."""
    from lorax_b200.runtime.engine import GenRequest
    cfg = tiny_llama()
    model = DecoderModel.random_init(cfg, "cpu", torch.float32, seed=0)
    ads = [random_adapter(cfg, r=8, alpha=16, target_modules=["q_proj", "v_proj"], seed=200 + i, std_a=0.05, std_b=0.05) for i in range(6)]
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab_size, (int(torch.randint(6, 20, (1,), generator=g)),), generator=g).tolist() for _ in range(12)]
    which = [1, 2, 3, 1, 4, 5, 6, 2, 0, 3, 6, 1]

    def run(arena_adapters):
        mgr = AdapterManager(model, arena_bytes=64 << 20, host_bytes=256 << 20)
        for i, (c, mm) in enumerate(ads):
            mgr.register(f"x{i}", c, mm)
        one = mgr.host.get("x0").blob.numel()
        mgr2 = AdapterManager(model, arena_bytes=int(one * 4 * arena_adapters * 1.05) + 4096, host_bytes=256 << 20)   # fp32 blobs
        for i, (c, mm) in enumerate(ads):
            mgr2.register(f"x{i}", c, mm)
        eng = Engine(model, EngineConfig(max_total_tokens=64, max_batch_prefill_tokens=256, waiting_served_ratio=0.0), num_blocks=64, max_batch=3)
        for i in range(6):
            eng.register_adapter(i + 1, f"x{i}")
        for i, p in enumerate(prompts):
            eng.add_request(GenRequest(i + 1, p, 6, which[i]))
        eng.run(max_steps=500)
        assert eng.idle
        return [eng.finished[i + 1].output_ids for i in range(12)], eng.stats, mgr2

    full, _, _ = run(6)
    tight, stats, mgr = run(2)
    assert tight == full
    assert stats.get("adapter_evictions", 0) >= 3 and len(mgr.resident) <= 2
    # with room for one adapter more than the batch can use, adapters of queued requests are brought in ahead of their turn
    roomy, stats3, _ = run(4)
    assert roomy == full and stats3.get("adapter_prefetches", 0) >= 1


def test_vocabulary_parallel_sampling_equals_sampling_from_the_full_row():
    """Tensor-parallel ranks keep their vocabulary shard, exchange 128 candidates plus (max, sum exp) per row and the best
    (noisy score, log-probability, id) triple: the drawn ids equal those of the sampler that sees the whole row, for
    temperature-only rows, top-k rows with and without top-p, and greedy rows that only carry penalties."""
    from lorax_b200.sampling import device as ds
    from lorax_b200.sampling.chooser import NextTokenParams
    torch.manual_seed(3)
    V, ws = 1000, 4
    pad = 1024                                   # the head is padded to a multiple of the ranks' shard: columns >= V must never win
    params = [NextTokenParams(do_sample=True, temperature=0.8, seed=11), NextTokenParams(do_sample=True, temperature=1.3, top_k=40, seed=5),
              NextTokenParams(do_sample=True, temperature=0.9, top_k=100, top_p=0.7, seed=9), NextTokenParams(do_sample=False, repetition_penalty=1.4, frequency_penalty=0.2),
              NextTokenParams(do_sample=True, temperature=0.5, top_k=3, top_p=0.95, seed=2, presence_penalty=0.5)]
    assert all(ds.tp_eligible(p) for p in params)
    assert not ds.tp_eligible(NextTokenParams(do_sample=True, top_p=0.9)) and not ds.tp_eligible(NextTokenParams(do_sample=True, top_k=500))
    assert not ds.tp_eligible(NextTokenParams(do_sample=True, top_k=10, typical_p=0.5))
    rows = [0, 2, 3, 5, 6]
    B = 8
    for trial in range(6):
        logits = torch.randn(B, pad) * 3
        logits[:, V:] = 50.0                      # padding columns carry junk
        hist = {i: torch.randint(0, 3, (V,)).float() for i in range(len(rows))}
        steps = [trial + 4 * i for i in range(len(rows))]
        full = ds.RowSampler("cpu")
        store_a = {k: v.clone() for k, v in hist.items()}
        full.bind(rows, params, list(range(len(rows))), store_a)
        want_ids, want_lp = full(logits[:, :V], steps)
        shard = pad // ws
        samplers, stores = [], []
        for r in range(ws):
            sm = ds.RowSampler("cpu")
            st = {k: v.clone() for k, v in hist.items()}
            sm.bind(rows, params, list(range(len(rows))), st)
            samplers.append(sm)
            stores.append(st)
        phase1 = [sm.tp_candidates(logits[:, r * shard:(r + 1) * shard], r * shard, V) for r, sm in enumerate(samplers)]
        payloads = torch.stack([p for _, p in phase1])
        assert payloads.shape == (ws, len(rows), ds.TP_CANDIDATES + 2)
        bests = []
        for r, sm in enumerate(samplers):
            tau, logz = sm.tp_cutoff(payloads)
            bests.append(sm.tp_local_best(phase1[r][0], tau, logz, steps, r * shard))
        bests = torch.stack(bests)
        for sm in samplers:
            ids, lp = sm.tp_finish(bests)
            assert torch.equal(ids, want_ids), (trial, ids, want_ids)
            assert torch.allclose(lp, want_lp, atol=1e-4)
            assert int(ids.max()) < V
        for sm in samplers:
            sm.release()
        full.release()
        for st in stores:                         # every rank bumped the same histogram entries as the full sampler
            for k in st:
                assert torch.equal(st[k], store_a[k])


def test_device_sampler_distribution_and_filters():
    """The exponential-noise draw follows the warped distribution; top-k / top-p / typical-p keep exactly the reference's sets;
    the noise depends on (seed, step) only."""
    from lorax_b200.sampling import device as ds
    torch.manual_seed(0)
    V = 12
    logits = torch.randn(1, V) * 2
    t = torch.tensor
    # filters against the per-row warpers of the host chooser's definitions
    x = ds.warp(logits, t([0.7]), t([5]), t([0.8]), t([1.0]))
    scaled = logits[0] / 0.7
    top5 = scaled.topk(5).indices
    p = torch.softmax(scaled[top5], -1)
    keep = top5[: int(((p.cumsum(0) - p) < 0.8).sum())]
    assert set(torch.isfinite(x[0]).nonzero()[:, 0].tolist()) == set(keep.tolist())
    off = ds.warp(logits, t([1.0]), t([0]), t([1.0]), t([1.0]))
    assert torch.allclose(off, logits.float())
    typ = ds.warp(logits, t([1.0]), t([0]), t([1.0]), t([0.5]))
    logp = torch.log_softmax(logits[0], -1)
    ent = -(logp.exp() * logp).sum()
    order = (-logp - ent).abs().argsort()
    mass = logp.exp()[order]
    n_keep = int(((mass.cumsum(0) - mass) < 0.5).sum())
    assert set(torch.isfinite(typ[0]).nonzero()[:, 0].tolist()) == set(order[:n_keep].tolist())
    # the draw: empirical frequencies over many steps match softmax
    R = 20000
    scores = logits.expand(R, V).contiguous()
    ids, lp = ds.draw(scores, torch.full((R,), 1234, dtype=torch.int64), torch.arange(R, dtype=torch.int64))
    freq = torch.bincount(ids, minlength=V).float() / R
    assert (freq - torch.softmax(logits[0], -1)).abs().max().item() < 0.012
    assert torch.allclose(lp, torch.log_softmax(logits[0], -1)[ids])
    # determinism: same (seed, step) -> same noise whatever the row; different seeds differ
    a = ds.uniform_noise(t([7, 9, 7]), t([3, 3, 3]), 1000)
    assert torch.equal(a[0], a[2]) and not torch.equal(a[0], a[1]) and 0 < a.min() and a.max() < 1
    assert abs(a.mean().item() - 0.5) < 0.02


def test_engine_samples_on_device_reproducibly(setup):
    """Sampling requests in the in-process engine: a request's tokens depend on its seed only (not on its neighbours or its
    decode row), greedy requests in the same batch are untouched, and unsupported parameters are refused."""
    from lorax_b200.sampling.chooser import NextTokenParams
    cfg, model, mgr, _ = setup
    g = torch.Generator().manual_seed(21)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 17, 12, 30)]

    def run(order, params):
        eng = Engine(model, EngineConfig(max_input_length=64, max_total_tokens=128, max_batch_prefill_tokens=256, compile=False), num_blocks=64)
        for rid in order:
            eng.add_request(GenRequest(rid, prompts[rid], max_new_tokens=10, params=params[rid]))
        eng.run()
        return {rid: eng.finished[rid].output_ids for rid in order}
    sample = NextTokenParams(temperature=1.3, top_k=50, top_p=0.95, do_sample=True, seed=11)
    params = {0: NextTokenParams(), 1: sample, 2: NextTokenParams(temperature=0.8, do_sample=True, seed=5), 3: NextTokenParams()}
    a = run([0, 1, 2, 3], params)
    b = run([3, 2, 1], params)                              # other neighbours, other rows
    greedy = run([0, 3], params)
    assert a[1] == b[1] and a[2] == b[2]
    assert a[0] == greedy[0] and a[3] == greedy[3] == b[3]
    c = run([1], {1: NextTokenParams(temperature=1.3, top_k=50, top_p=0.95, do_sample=True, seed=12)})
    assert c[1] != a[1]                                     # another seed, another continuation
    assert all(len(v) == 10 for v in a.values())
    with pytest.raises(ValueError):
        run([0], {0: NextTokenParams(do_sample=True, watermark=True)})


def test_engine_penalties_on_device_match_the_host_chooser(setup):
    """Repetition, frequency and presence penalties in the in-process engine, whose history is a histogram on the device: a
    greedy request with penalties yields the tokens of a step-by-step oracle (full forward pass over prompt + output, the
    served path's host-side chooser over the whole history, arg-max), whatever shares its batch; a sampling request with
    penalties is reproducible from its seed."""
    from lorax_b200.runtime.kv_cache import KVCache
    from lorax_b200.runtime.runner import ModelRunner, PrefillItem
    from lorax_b200.sampling.chooser import HeterogeneousNextTokenChooser, NextTokenParams
    from lorax_b200.sampling import device as ds
    cfg, model, mgr, _ = setup
    g = torch.Generator().manual_seed(33)
    # prompts over a small alphabet so that tokens repeat and the penalties bite
    prompts = [torch.randint(0, 40, (n,), generator=g).tolist() for n in (14, 25, 11)]
    pen = NextTokenParams(repetition_penalty=1.8, frequency_penalty=0.7, presence_penalty=0.4)
    assert ds.supported(pen) and ds.needs_device_step(pen) and not pen.plain
    n_new = 12

    def oracle(prompt):
        kv = KVCache(cfg.num_hidden_layers, 16, model.nkv, model.d, model.dtype, model.device)
        r = ModelRunner(model, kv, max_batch=2, max_seq_tokens=128, max_prefill_tokens=256, use_graphs=False)
        chooser = HeterogeneousNextTokenChooser([pen], "cpu", cfg.vocab_size)
        ids = list(prompt)
        for _ in range(n_new):
            logits = r.prefill([PrefillItem(ids, 0, [1, 2, 3, 4], all_logprobs=True)])[2][-1:].float()
            hist = torch.tensor([ids])
            ids.append(int(chooser.warp(hist, torch.ones_like(hist, dtype=torch.bool), logits.clone()).argmax(-1)))
        return ids[len(prompt):]

    def run(order, params):
        eng = Engine(model, EngineConfig(max_input_length=64, max_total_tokens=128, max_batch_prefill_tokens=256, compile=False), num_blocks=64)
        for rid in order:
            eng.add_request(GenRequest(rid, prompts[rid], max_new_tokens=n_new, params=params[rid]))
        eng.run()
        assert not eng._hist or all(k in eng.running for k in eng._hist)
        return {rid: eng.finished[rid].output_ids for rid in order}
    sample = NextTokenParams(temperature=1.1, top_k=30, do_sample=True, seed=4, repetition_penalty=1.5, presence_penalty=0.5)
    params = {0: pen, 1: NextTokenParams(), 2: sample}
    a = run([0, 1, 2], params)
    b = run([2, 0], params)
    plain = run([0, 1], {0: NextTokenParams(), 1: NextTokenParams()})
    assert a[0] == oracle(prompts[0]) == b[0]
    assert a[0] != plain[0] and a[1] == plain[1]            # the penalties change the tokens; the greedy neighbour is untouched
    assert a[2] == b[2]
