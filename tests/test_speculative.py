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
