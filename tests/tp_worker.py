"""Worker for the tensor-parallel tests (launched with torch.distributed.run; rank 0 prints one JSON line).

Checks, on every rank: (1) the TP=k forward of a tiny Llama with LoRA adapters equals the TP=1 forward of the same
model (same seed -> same full weights), which is the rank-consistency requirement for the LoRA sharding scheme;
(2) on GPUs, the fused GEMM + reduce-scatter + all-gather kernel and the vocabulary-parallel greedy head against
fp32 references assembled with NCCL collectives, twice in a row (the counters are cumulative across launches)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lorax_b200.adapters.lora import random_adapter  # noqa: E402
from lorax_b200.adapters.manager import AdapterManager  # noqa: E402
from lorax_b200.config import tiny_llama  # noqa: E402
from lorax_b200.models.decoder import DecoderModel  # noqa: E402
from lorax_b200.parallel.tp import TensorParallel  # noqa: E402
from lorax_b200.runtime.kv_cache import KVCache  # noqa: E402
from lorax_b200.runtime.runner import ModelRunner, PrefillItem  # noqa: E402

TARGETS = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


def build(cfg, device, dtype, tp):
    model = DecoderModel.random_init(cfg, device, dtype, seed=0, tp=tp)
    mgr = AdapterManager(model, arena_bytes=64 << 20, host_bytes=128 << 20)
    for i in range(2):
        c, mm = random_adapter(cfg, r=8 * (i + 1), alpha=16, target_modules=TARGETS, seed=20 + i, std_a=0.05, std_b=0.05)
        mgr.register(f"a{i}", c, mm)
        assert mgr.load(i + 1, f"a{i}")
    return model


def run_model(model, prompts, ads, n_decode, graphs):
    cfg = model.config
    kv = KVCache(cfg.num_hidden_layers, 64, model.nkv, model.d, model.dtype, model.device)
    r = ModelRunner(model, kv, max_batch=8, max_seq_tokens=256, max_prefill_tokens=1024, use_graphs=graphs)
    blocks = [[1 + 4 * i + j for j in range(4)] for i in range(len(prompts))]
    ids, _, logits = r.prefill([PrefillItem(p, 0, blocks[i], adapter_index=ads[i]) for i, p in enumerate(prompts)])
    outs = [logits.float().cpu().clone()]
    rows = [r.state.take_row(i) for i in range(len(prompts))]
    r.install(rows, ids.tolist(), [len(p) for p in prompts], blocks, ads)
    r.resort()
    toks = [ids.tolist()]
    for _ in range(n_decode):
        k, b, logits = r.decode(need_logits=False)
        idp, _ = r.wait(k)
        toks.append(idp[:len(prompts)].tolist())
    return outs, toks


def run_sampled(model, prompts, ads, shards: bool, n_decode: int = 4):
    """Sampled decoding (top-k with temperature, top-k + top-p, temperature only) through the device sampler: from vocabulary
    shards with candidates exchanged, or from the gathered logits."""
    from lorax_b200.sampling.chooser import NextTokenParams
    from lorax_b200.sampling.device import RowSampler
    cfg = model.config
    kv = KVCache(cfg.num_hidden_layers, 64, model.nkv, model.d, model.dtype, model.device)
    r = ModelRunner(model, kv, max_batch=8, max_seq_tokens=256, max_prefill_tokens=1024, use_graphs=True)
    blocks = [[1 + 4 * i + j for j in range(4)] for i in range(len(prompts))]
    ids, _, _ = r.prefill([PrefillItem(p, 0, blocks[i], adapter_index=ads[i]) for i, p in enumerate(prompts)])
    rows = [r.state.take_row(i) for i in range(len(prompts))]
    r.install(rows, ids.tolist(), [len(p) for p in prompts], blocks, ads)
    mapping = r.resort()
    params = [NextTokenParams(do_sample=True, temperature=0.9, top_k=20, seed=3), NextTokenParams(do_sample=True, temperature=1.2, top_k=50, top_p=0.8, seed=4),
              NextTokenParams(do_sample=True, temperature=0.7, seed=5)]
    rs = RowSampler(model.device)
    live = sorted(mapping[x] for x in rows)
    rs.bind(live, params)
    toks, used_shards = [], []
    tp = model.tp
    for step in range(n_decode):
        def hook(logits, st, step=step):
            local = logits.shape[1] != model.vocab
            used_shards.append(bool(local))
            if local:
                got, lp = rs.call_tp(logits, [step] * len(live), model.vocab_start, model.vocab, tp.all_gather_stack)
            else:
                got, lp = rs(logits, [step] * len(live))
            g32 = got.to(st.next_ids.dtype)
            st.next_ids.index_copy_(0, rs.rows, g32)
            st.logprobs.index_copy_(0, rs.rows, lp.to(st.logprobs.dtype))
            st.input_ids.index_copy_(0, rs.rows, g32)
        k, b, _ = r.decode(sampler=hook, sampler_takes_shards=shards)
        idp, _ = r.wait(k)
        toks.append(idp[:len(prompts)].tolist())
    return toks, used_shards


def main():
    tp = TensorParallel.init_from_env()
    dev = tp.device
    cuda = dev.type == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    out = {"world": tp.world_size, "device": dev.type}
    cfg = tiny_llama()
    if tp.world_size > 2:          # shapes that still split over 4 and 8 ranks (heads, K shards that are multiples of 8)
        cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads = 512, 1024, 8, 2
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (20, 33, 47)]
    ads = [1, 0, 2]
    # ---- TP=k model vs TP=1 model
    full = build(cfg, dev, dtype, TensorParallel.single())
    ref_logits, ref_toks = run_model(full, prompts, ads, 4, graphs=False)
    for mode in (["nccl", "fused"] if cuda else ["gloo"]):
        shard = build(cfg, dev, dtype, tp)
        if mode == "fused":
            from lorax_b200.parallel import fused
            fused.enable(tp, shard).max_fused_tokens = 256       # exercise the fused kernel for every batch size
        else:
            tp.fused = None
        got_logits, got_toks = run_model(shard, prompts, ads, 4, graphs=cuda)
        err = ((got_logits[0] - ref_logits[0]).norm() / ref_logits[0].norm()).item()
        out[f"model_{mode}_logits_relerr"] = err
        out[f"model_{mode}_first_tokens_equal"] = got_toks[0] == ref_toks[0]
        out[f"model_{mode}_decode_tokens_equal"] = sum(a == b for a, b in zip(got_toks, ref_toks)) / len(ref_toks)
        if mode == "fused":
            tp.fused.check()
            out["fused_calls"] = tp.fused.calls
            # sampling from vocabulary shards (candidates exchanged) draws what sampling from the gathered logits draws
            a, used_a = run_sampled(shard, prompts, ads, shards=True)
            b, used_b = run_sampled(shard, prompts, ads, shards=False)
            out["sampled_from_shards_equals_gathered"] = a == b
            out["sampled_shards_path_taken"] = all(used_a) and not any(used_b)
            tp.fused.check()
    # ---- kernels
    if cuda:
        from lorax_b200.parallel import fused as fz
        fc = tp.fused
        errs, eq = [], []
        for it, (T, N, K) in enumerate([(5, 256, 128), (64, 256, 512), (200, 256, 192), (17, 256, 64)]):
            gen = torch.Generator(device=dev).manual_seed(100 * it + tp.rank)
            x = torch.randn(T, K, device=dev, dtype=dtype, generator=gen)
            w = torch.randn(N, K, device=dev, dtype=dtype, generator=gen) / K ** 0.5
            add = torch.randn(T, N, device=dev, dtype=dtype, generator=gen) * 0.1
            res = fc.gemm_allreduce(x, w, None, add).clone()
            part = x.float() @ w.float().t() + add.float()
            dist.all_reduce(part)
            torch.cuda.synchronize()
            errs.append(((res.float() - part).norm() / part.norm()).item())
            gathered = [torch.empty_like(res) for _ in range(tp.world_size)]
            dist.all_gather(gathered, res)
            eq.append(all(torch.equal(gathered[0], t) for t in gathered))      # every rank holds the same bits
        fc.check()
        # 7B-sized output width with the K shards of the O and down projections: both token-tile regimes and the K-split variants
        fc_big = fz.FusedCollectives(tp, n_max=4096, max_rows=512)
        for it, (T, N, K) in enumerate([(32, 4096, 4096 // tp.world_size), (256, 4096, 14336 // tp.world_size), (100, 4096, 512)]):
            gen = torch.Generator(device=dev).manual_seed(500 + 100 * it + tp.rank)
            x = torch.randn(T, K, device=dev, dtype=dtype, generator=gen)
            w = torch.randn(N, K, device=dev, dtype=dtype, generator=gen) / K ** 0.5
            res = fc_big.gemm_allreduce(x, w, None, None).clone()
            part = x.float() @ w.float().t()
            dist.all_reduce(part)
            torch.cuda.synchronize()
            errs.append(((res.float() - part).norm() / part.norm()).item())
            gathered = [torch.empty_like(res) for _ in range(tp.world_size)]
            dist.all_gather(gathered, res)
            eq.append(all(torch.equal(gathered[0], t) for t in gathered))
        fc_big.check()
        out["gemm_allreduce_relerr"] = max(errs)
        out["gemm_allreduce_ranks_identical"] = all(eq)
        # two-shot all-reduce kernel against an fp32 sum of the ranks' inputs
        if fc.all_reduce_input(1, cfg.hidden_size) is not None:
            errs, eq = [], []
            for it, T in enumerate([1, 7, 64, 300]):
                gen = torch.Generator(device=dev).manual_seed(900 + 10 * it + tp.rank)
                x = torch.randn(T, cfg.hidden_size, device=dev, dtype=dtype, generator=gen)
                want = x.float()
                dist.all_reduce(want)
                got = fc.all_reduce(x.clone() if it % 2 else fc.all_reduce_input(T, cfg.hidden_size).copy_(x)).clone()
                torch.cuda.synchronize()
                errs.append(((got.float() - want).norm() / want.norm()).item())
                gathered = [torch.empty_like(got) for _ in range(tp.world_size)]
                dist.all_gather(gathered, got)
                eq.append(all(torch.equal(gathered[0], t) for t in gathered))
            fc.check()
            out["allreduce_sym_relerr"] = max(errs)
            out["allreduce_sym_ranks_identical"] = all(eq)
        # vocabulary-parallel greedy head
        ok = []
        for it, T in enumerate([3, 40]):
            gen = torch.Generator(device=dev).manual_seed(7 + it)           # same full logits on every rank
            full_logits = torch.randn(T, 1000 * tp.world_size, device=dev, dtype=dtype, generator=gen)
            local = full_logits[:, tp.rank * 1000:(tp.rank + 1) * 1000].contiguous()
            ids = torch.empty(T, dtype=torch.int32, device=dev)
            lps = torch.empty(T, dtype=torch.float32, device=dev)
            fc.argmax_tp(local, tp.rank * 1000, ids, lps)
            torch.cuda.synchronize()
            want = full_logits.float().argmax(-1)
            wlp = torch.log_softmax(full_logits.float(), -1).gather(1, want[:, None])[:, 0]
            ok.append(bool(torch.equal(ids.long(), want)) and bool(torch.allclose(lps, wlp, atol=2e-3)))
        fc.check()
        out["argmax_tp_ok"] = all(ok)
    flags = torch.tensor([1.0], device=dev if cuda else "cpu")
    dist.all_reduce(flags)
    if tp.rank == 0:
        print("RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
