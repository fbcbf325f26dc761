"""Speculative decoding in the shard runtime (prompt-lookup proposals verified by one ragged pass per step): the tokens
must equal plain greedy decoding whatever the proposals are, and good proposals must shorten the number of steps."""
import torch

from lorax_b200.adapters.lora import random_adapter
from lorax_b200.config import EngineConfig, tiny_llama
from lorax_b200.models.decoder import DecoderModel
from lorax_b200.server import runtime as rt_mod
from lorax_b200.server.runtime import ShardRuntime


def _run(rt, prompts, adapters, new_tokens):
    pb = rt.pb
    reqs = []
    for i, (p, a) in enumerate(zip(prompts, adapters)):
        reqs.append(pb.Request(id=i, tokenized_inputs=pb.TokenizedInputs(ids=p), truncate=256, adapter_index=a,
                               blocks=list(range(1 + 6 * i, 7 + 6 * i)),
                               parameters=pb.NextTokenChooserParameters(temperature=1.0, top_p=1.0, typical_p=1.0, repetition_penalty=1.0),
                               stopping_parameters=pb.StoppingCriteriaParameters(max_new_tokens=new_tokens[i], ignore_eos_token=True)))
    resp = rt.prefill(pb.PrefillRequest(batch=pb.Batch(id=1, requests=reqs, size=len(reqs), max_tokens=512)))
    out = {g.request_id: list(g.next_tokens.ids) for g in resp.generations}
    steps = 0
    cached = resp.batch if resp.HasField("batch") else None
    while cached is not None and steps < 200:
        d = rt.decode(pb.DecodeRequest(batches=[cached]))
        steps += 1
        for g in d.generations:
            out[g.request_id] += list(g.next_tokens.ids)
            if g.HasField("generated_text"):
                assert g.generated_text.generated_tokens == len(out[g.request_id])
        cached = d.batch if d.HasField("batch") else None
    return out, steps


def _runtime(model, spec):
    cfg = EngineConfig(max_input_length=128, max_total_tokens=192, max_batch_prefill_tokens=512, compile=False, speculative_tokens=spec)
    return ShardRuntime(model, None, cfg, num_blocks=64, max_batch=8, adapter_arena_bytes=64 << 20)


def test_speculative_decoding_matches_greedy(monkeypatch):
    torch.manual_seed(0)
    cfg = tiny_llama()
    model = DecoderModel.random_init(cfg, "cpu", torch.float32, seed=0)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (12, 30, 21)]
    new_tokens = [17, 9, 24]
    base_rt = _runtime(model, 0)
    c, mm = random_adapter(cfg, r=8, alpha=16, target_modules=["q_proj", "v_proj"], seed=5, std_a=0.05, std_b=0.05)
    base_rt.adapters.register("a", c, mm)
    assert base_rt.adapters.load(1, "a")
    adapters = [0, 1, 0]
    want, base_steps = _run(base_rt, prompts, adapters, new_tokens)
    assert [len(want[i]) for i in range(3)] == new_tokens and base_steps == max(new_tokens) - 1

    # 1. real prompt-lookup proposals (they rarely match a random model): same tokens
    spec_rt = _runtime(model, 3)
    spec_rt.adapters = base_rt.adapters
    model.adapters = base_rt.adapters
    got, _ = _run(spec_rt, prompts, adapters, new_tokens)
    assert got == want

    # 2. an oracle proposer that knows the continuation: every proposal is accepted, 4 tokens per row and step
    full = {i: prompts[i] + want[i] for i in range(3)}

    def oracle(history, lengths, last_ids, n_spec):
        h = history[0, : lengths[0]].tolist()
        i = next(k for k, f in full.items() if f[: len(h)] == h)
        nxt = full[i][len(h): len(h) + n_spec]
        return torch.tensor([nxt + [0] * (n_spec - len(nxt))])

    monkeypatch.setattr(rt_mod, "ngram_speculate", oracle)
    spec_rt2 = _runtime(model, 3)
    spec_rt2.adapters = base_rt.adapters
    model.adapters = base_rt.adapters
    got2, steps2 = _run(spec_rt2, prompts, adapters, new_tokens)
    assert got2 == want
    assert steps2 <= (max(new_tokens) - 1 + 3) // 4 + 1
    assert spec_rt2.spec_stats["tokens"] / spec_rt2.spec_stats["steps"] > 2.5


def test_medusa_heads_math_and_loading(tmp_path):
    """Both Medusa layouts against the formulas: v1 = residual blocks + own projection per head, v2 = one residual block per
    head and the base lm_head over the stacked rows (reference: adapters/medusa.py:102-214)."""
    import json
    from safetensors.torch import save_file
    from lorax_b200.adapters.medusa import MedusaConfig, MedusaHeads, is_medusa_dir, load_medusa_adapter, random_medusa_tensors
    H, V, R = 32, 50, 5
    g = torch.Generator().manual_seed(1)
    h = torch.randn(R, H, generator=g)
    lm = torch.randn(V, H, generator=g)
    silu = torch.nn.functional.silu
    # v2
    t2 = random_medusa_tensors(H, heads=3, layers=1, seed=2, std=0.3)
    heads2 = MedusaHeads(MedusaConfig("base", 3, 1, 2), t2, "cpu", torch.float32)
    assert heads2.shared_head
    got = heads2.propose(h, lambda x: x @ lm.t())
    want = torch.stack([((h + silu(h @ t2[f"{i}.0.linear.weight"].t() + t2[f"{i}.0.linear.bias"])) @ lm.t()).argmax(-1) for i in range(3)], 1)
    assert torch.equal(got, want)
    # v1 with two blocks per head
    t1 = random_medusa_tensors(H, heads=2, layers=2, vocab=V, seed=3, std=0.3)
    heads1 = MedusaHeads(MedusaConfig("base", 2, 2, 1), t1, "cpu", torch.float32)
    assert not heads1.shared_head
    cols = []
    for i in range(2):
        x = h
        for l in range(2):
            x = x + silu(x @ t1[f"{i}.{l}.linear.weight"].t() + t1[f"{i}.{l}.linear.bias"])
        cols.append((x @ t1[f"{i}.2.weight"].t()).argmax(-1))
    assert torch.equal(heads1.propose(h, None), torch.stack(cols, 1))
    # directory layout
    d = tmp_path / "medusa"
    d.mkdir()
    save_file(t2, str(d / "medusa_lm_head.safetensors"))
    (d / "config.json").write_text(json.dumps({"base_model_name_or_path": "base", "medusa_num_heads": 3, "medusa_num_layers": 1, "version": 2}))
    assert is_medusa_dir(str(d)) and not is_medusa_dir(str(tmp_path))
    cfg, tensors = load_medusa_adapter(str(d))
    assert cfg.medusa_num_heads == 3 and cfg.version == 2 and set(tensors) == set(t2)


def test_medusa_speculation_matches_greedy_and_follows_the_heads(tmp_path):
    """Medusa heads as the proposer of the speculative path: whatever they guess the emitted tokens equal plain greedy decoding,
    the guesses come from the hidden state of the last accepted position, per-request heads override the default ones, and
    heads that know the continuation cut the number of steps."""
    import json
    from safetensors.torch import save_file
    from lorax_b200.adapters.medusa import MedusaConfig, random_medusa_tensors
    torch.manual_seed(0)
    cfg = tiny_llama()
    model = DecoderModel.random_init(cfg, "cpu", torch.float32, seed=0)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (10, 26)]
    new_tokens = [15, 11]
    base_rt = _runtime(model, 0)
    want, _ = _run(base_rt, prompts, [0, 0], new_tokens)

    rt = _runtime(model, 0)
    rt.load_medusa(0, MedusaConfig("m", 3, 1, 2), random_medusa_tensors(cfg.hidden_size, 3, seed=7, std=0.2))
    assert rt.cfg.speculative_tokens == 3 and model.keep_hidden
    seen = []
    inner = rt._medusa_guess

    def spy(seqs, hidden):
        inner(seqs, hidden)
        seen.extend(len(s.spec_next) for s in seqs)
    rt._medusa_guess = spy
    got, _ = _run(rt, prompts, [0, 0], new_tokens)
    assert got == want and seen and set(seen) == {3}

    # heads addressed by a request's adapter index, arriving through the adapter RPCs from a local directory
    d = tmp_path / "heads"
    d.mkdir()
    save_file(random_medusa_tensors(cfg.hidden_size, 2, seed=9, std=0.2), str(d / "medusa_lm_head.safetensors"))
    (d / "config.json").write_text(json.dumps({"medusa_num_heads": 2, "medusa_num_layers": 1, "version": 2}))
    pb = rt.pb
    params = pb.AdapterParameters(adapter_ids=[str(d)])
    r = rt.download_adapter(pb.DownloadAdapterRequest(adapter_parameters=params, adapter_source=2))
    assert r.downloaded
    assert rt.load_adapter(pb.LoadAdapterRequest(adapter_parameters=params, adapter_source=2, adapter_index=5)).loaded
    assert rt.medusa[5].num_heads == 2
    seen.clear()
    got5, _ = _run(rt, prompts, [5, 0], new_tokens)
    assert got5 == want and {2, 3} <= set(seen)          # LoRA-free adapter index: base model tokens, its own two heads
    assert rt.offload_adapter(pb.OffloadAdapterRequest(adapter_parameters=params, adapter_source=2, adapter_index=5)).offloaded
    assert 5 not in rt.medusa

    # heads that know the continuation: every guess is accepted
    full = {i: prompts[i] + want[i] for i in range(2)}

    rt2 = _runtime(model, 0)
    rt2.load_medusa(0, MedusaConfig("m", 3, 1, 2), random_medusa_tensors(cfg.hidden_size, 3, seed=7))
    rt2._medusa_guess = lambda seqs, hidden: None
    verify = rt2._decode_speculative

    def clairvoyant(seqs, n_spec):                       # guesses as perfect heads would have left them after the last pass
        for s in seqs:
            h = s.prompt_ids + s.output_ids
            i = next(k for k, f in full.items() if f[: len(h)] == h)
            s.spec_next = full[i][len(h): len(h) + 3]
        return verify(seqs, n_spec)
    rt2._decode_speculative = clairvoyant
    got2, steps2 = _run(rt2, prompts, [0, 0], new_tokens)
    assert got2 == want and steps2 <= (max(new_tokens) - 1 + 3) // 4 + 1
    model.keep_hidden = False


def test_preloaded_adapters_are_loaded_and_announced(tmp_path):
    """`--preloaded-adapter-ids`: adapters are fetched in parallel at start-up, sit under indices 1..n and are listed in Info, so
    the router can address them without a load on demand."""
    from lorax_b200.adapters.lora import save_peft_adapter
    cfg = tiny_llama()
    model = DecoderModel.random_init(cfg, "cpu", torch.float32, seed=0)
    rt = _runtime(model, 0)
    dirs = []
    for i in range(3):
        c, mm = random_adapter(cfg, r=8, alpha=16, target_modules=["q_proj", "v_proj"], seed=40 + i, std_a=0.05, std_b=0.05)
        save_peft_adapter(tmp_path / f"ad{i}", c, mm)
        dirs.append(str(tmp_path / f"ad{i}"))
    rt.preload_adapters(dirs[:2], source=2)
    rt.load_default_adapter(dirs[2], source=2)
    info = rt.info()
    got = {p.adapter_parameters.adapter_ids[0]: (p.adapter_index, p.adapter_source) for p in info.preloaded_adapters}
    assert got == {dirs[0]: (1, 2), dirs[1]: (2, 2), dirs[2]: (3, 2)}
    assert all(rt.adapters.is_loaded(i) for i in (1, 2, 3))
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, cfg.vocab_size, (11,), generator=g).tolist()] * 3
    out, _ = _run(rt, prompts, [0, 1, 3], [6, 6, 6])
    assert len({tuple(v) for v in out.values()}) >= 2          # the adapters change the continuation
    model.adapters = None
