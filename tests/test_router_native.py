"""C++ router components through their C ABI: allocator, radix trie, adapter exchange policy, JSON, and the
batching loop against a fake shard (including failure injection on the host)."""
import json

import pytest

from lorax_b200.router import native as rn


def test_simple_allocator_reserves_block_zero_and_recycles():
    a = rn.BlockAllocator(num_blocks=9, block_size=16)
    assert a.free_blocks == 8
    x = a.allocate(40)
    assert len(x.blocks) == 3 and 0 not in x.blocks and len(x.slots) == 40
    assert x.slots[0] == x.blocks[0] * 16 and x.slots[16] == x.blocks[1] * 16
    y = a.allocate(16 * 5)
    assert y is not None and a.free_blocks == 0
    assert a.allocate(1) is None
    a.free(x)
    assert a.free_blocks == 3


def test_sliding_window_allocation_cycles_slots():
    a = rn.BlockAllocator(num_blocks=64, block_size=16, window=32)
    x = a.allocate(100)
    assert len(x.blocks) == 3            # ceil(32/16) + 1
    assert len(x.slots) == 100
    assert x.slots[48] == x.slots[0]     # slot list wraps around the window's blocks


def test_radix_prefix_reuse_and_adapter_isolation():
    a = rn.BlockAllocator(num_blocks=32, block_size=4, prefix_caching=True)
    prompt = list(range(10))
    x = a.allocate(16, adapter_index=1, prompt=prompt)
    assert x.prefix_len == 0
    free_before = a.free_blocks
    a.free(x, adapter_index=1, all_tokens=prompt + [100, 101])      # 12 tokens -> 3 whole blocks cached
    assert a.free_blocks == free_before + 1                          # 4 allocated, 3 adopted by the trie
    y = a.allocate(16, adapter_index=1, prompt=prompt)
    assert y.prefix_len == 8 and y.blocks[:2] == x.blocks[:2]        # never the whole prompt: last block is recomputed
    z = a.allocate(16, adapter_index=2, prompt=prompt)
    assert z.prefix_len == 0                                         # same text, other adapter: different KV
    w = a.allocate(16, adapter_index=1, prompt=prompt[:5] + [77] * 5)
    assert w.prefix_len == 4                                         # partial overlap: one shared block


def test_radix_evicts_lru_unreferenced_leaves():
    a = rn.BlockAllocator(num_blocks=9, block_size=4, prefix_caching=True)    # 8 usable blocks
    p1, p2 = [1] * 8, [2] * 8
    x = a.allocate(8, prompt=p1); a.free(x, all_tokens=p1)
    y = a.allocate(8, prompt=p2); a.free(y, all_tokens=p2)
    assert a.free_blocks == 4
    z = a.allocate(9, prompt=p2 + [9])         # touches p2 (now most recent) and takes 1 more block
    assert z.prefix_len == 8
    big = a.allocate(20, prompt=[3] * 20)      # needs 5 blocks: must evict p1 (LRU, unreferenced), not p2 (referenced)
    assert big is not None
    again = a.allocate(4, prompt=p1 + [5])
    assert again is None or again.prefix_len == 0


def test_radix_split_of_a_referenced_node_keeps_blocks_evictable():
    """A live allocation points at the deepest node it matched.  When a second request shares only a shorter prefix the
    node is split; both parts must lose their reference when the requests end, or the blocks are stuck for good."""
    a = rn.BlockAllocator(num_blocks=9, block_size=4, prefix_caching=True)       # 8 usable blocks
    prompt = list(range(100, 117))                                               # 17 tokens
    first = a.allocate(17, prompt=prompt); a.free(first, all_tokens=prompt)      # 4 whole blocks cached
    x = a.allocate(17, prompt=prompt)                                            # references the 16-token node
    assert x.prefix_len == 16
    y = a.allocate(12, prompt=prompt[:8] + [7, 7, 7, 7])                         # shares 8 tokens: splits that node
    assert y.prefix_len == 8
    a.free(x, all_tokens=prompt); a.free(y, all_tokens=prompt[:8] + [7, 7, 7, 7])
    big = a.allocate(32, prompt=[9] * 32)                                        # needs every block: all must be evictable
    assert big is not None and len(big.blocks) == 8


def test_json_parser_roundtrip_and_errors():
    s = '{"a": [1, 2.5, true, null, "x\\n\\u00e9\\ud83d\\ude00"], "b": {"c": -3}}'
    out = json.loads(rn.json_roundtrip(s))
    assert out == json.loads(s)
    assert rn.json_roundtrip('{"a": }').startswith("ERROR")
    assert rn.json_roundtrip('[1, 2').startswith("ERROR")


def test_adapter_exchange_policy():
    ops = [
        ["append", 1, 0.0], ["append", 2, 0.1], ["append", 3, 0.2],
        ["downloaded", 1, 0.3], ["downloaded", 2, 0.3], ["downloaded", 3, 0.3],
        ["update", [], 0.5],                 # 2 slots: adapters 1 and 2 are admitted, 3 waits
        ["next", 0.5],                       # nothing is Ready yet
        ["ready", 1], ["ready", 2],
        ["next", 0.6], ["next", 0.6],        # oldest first: request of adapter 1, then adapter 2
        ["update", [1], 0.7],                # adapter 2 idle and 3 pending -> 2 is offloaded, 3 admitted
        ["ready", 3], ["next", 0.8],
    ]
    t = rn.queues_script(ops, max_active=2, cycle_s=100.0)
    assert t[6]["load"] == [1, 2] and t[6]["offload"] == []
    assert t[7] is None
    assert t[10] == 1 and t[11] == 2
    assert t[12]["offload"] == [2] and t[12]["load"] == [3]
    assert t[14] == 3


def test_adapter_time_slice_rotation():
    ops = [
        ["append", 1, 0.0], ["append", 1, 0.0], ["append", 2, 0.1],
        ["downloaded", 1, 0.6], ["downloaded", 2, 0.6],
        ["update", [], 0.0], ["ready", 1],
        ["update", [], 5.0],                 # adapter 1 exceeded its 2 s slice while adapter 2 waits (budget 1.0 fits one)
    ]
    t = rn.queues_script(ops, max_active=4, cycle_s=2.0)
    assert t[5]["load"] == [1]
    assert t[7]["offload"] == [1] and t[7]["load"] == [2]


def test_batching_loop_heterogeneous_adapters():
    reqs = [{"inputs": f"hello world {i}", "adapter_id": ["", "a1", "a2", "a3"][i % 4] or None, "max_new_tokens": 3 + i % 5} for i in range(24)]
    for r in reqs:
        if r["adapter_id"] is None:
            del r["adapter_id"]
    out = rn.infer_fake_run(reqs, max_active_adapters=8)
    assert all(r["ok"] for r in out["results"]), out["results"]
    assert [r["tokens"] for r in out["results"]] == [3 + i % 5 for i in range(24)]
    log = out["log"]
    assert sorted(l for l in log if l.startswith("download")) == ["download a1", "download a2", "download a3"]
    assert sum(l.startswith("load") for l in log) == 3
    assert "lorax_batch_inference_count" in out["metrics"]


def test_adapter_failure_is_isolated():
    reqs = [{"inputs": "a b c", "adapter_id": "missing-one", "max_new_tokens": 4},
            {"inputs": "a b c", "adapter_id": "good", "max_new_tokens": 4},
            {"inputs": "a b c", "max_new_tokens": 4}]
    out = rn.infer_fake_run(reqs)
    r = out["results"]
    assert not r[0]["ok"] and "missing-one" in r[0]["error"]
    assert r[1]["ok"] and r[2]["ok"]


def test_decode_failure_fails_batch_and_clears_cache():
    reqs = [{"inputs": "x y", "max_new_tokens": 10} for _ in range(4)]
    out = rn.infer_fake_run(reqs, fail_decode_after=2)
    assert all((not r["ok"]) and r["error_type"] == "generation" for r in out["results"])
    assert "clear" in out["log"]


def test_validation_errors():
    out = rn.infer_fake_run([{"inputs": "", "max_new_tokens": 4}, {"inputs": "a", "max_new_tokens": 5000},
                             {"inputs": "a", "max_new_tokens": 2, "top_p": 1.5}])
    assert [r.get("status") for r in out["results"]] == [422, 422, 422]


@pytest.mark.parametrize("sanitizer", ["address", "thread"])
def test_host_code_under_sanitizers(sanitizer):
    """The allocator, the queues and the batching loop (36 concurrent requests over 6 adapters against the fake shard, then the
    same with a shard that starts failing) built with AddressSanitizer + UBSan and with ThreadSanitizer: no finding, exit 0."""
    import os
    import subprocess
    from lorax_b200.csrc import build
    try:
        exe = build.build_host_selftest(sanitizer)
    except build.SanitizerUnavailable as e:
        pytest.skip(str(e))
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1", UBSAN_OPTIONS="print_stacktrace=1")
    # real tokenizer pipelines and awkward text for the router's tokenizer under the sanitizer (the files of the tokenizer tests)
    try:
        import tempfile
        import test_router_tokenizer as T
        from tokenizers import pre_tokenizers
        d = tempfile.mkdtemp()
        toks = {"bl": T.byte_level_bpe(pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)), "sp": T.sentencepiece_bpe(True),
                "sp2": T.sentencepiece_bpe(False)}
        try:
            toks["uni"] = T.precompiled_unigram()
        except BaseException:                      # no sentencepiece here
            pass
        paths = []
        for name, tok in toks.items():
            tok.save(os.path.join(d, name + ".json"))
            paths.append(os.path.join(d, name + ".json"))
        with open(os.path.join(d, "text"), "w", encoding="utf-8") as f:
            f.write("\x1e".join(T.SAMPLES + T.HARD_UNICODE))
        env.update(LX_SELFTEST_TOKENIZERS=":".join(paths), LX_SELFTEST_TEXT=os.path.join(d, "text"))
    except ImportError:
        pass
    try:
        import json
        import tempfile
        import test_router_chat_template as C
        reqs = [json.dumps(dict(template=t, messages=m, bos_token="<s>", eos_token="</s>", **({"tools": C.TOOLS} if k % 2 else {})))
                for t in C.TEMPLATES.values() for k, m in enumerate(C.MESSAGES)]
        chat_file = os.path.join(tempfile.mkdtemp(), "chat")
        with open(chat_file, "w", encoding="utf-8") as f:
            f.write("\x1e".join(reqs))
        env["LX_SELFTEST_CHAT"] = chat_file
    except ImportError:
        pass
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
    if "LX_SELFTEST_TOKENIZERS" in env:
        assert "tokenizer files:" in r.stdout and " 0 ids" not in r.stdout
    if "LX_SELFTEST_CHAT" in env:
        assert "chat requests:" in r.stdout and "chat requests: 0 of" not in r.stdout


def test_encoder_batcher_shares_batches_and_contains_failures():
    """Embed / classify inputs from eight caller threads through the router's encoder batcher against the fake shard: every answer is
    the one of the caller's own input, inputs that arrive while a batch is on the shard share the next one, and a batch the shard
    fails answers its own inputs with the error and nobody else's."""
    from lorax_b200.router.native import encoder_batcher_fake_run
    r = encoder_batcher_fake_run(8, 30)
    assert r["wrong"] == 0 and r["ok"] + r["failed"] == 240
    assert 4 <= r["failed"] < 40                       # thread 0 sends four failing inputs; a few neighbours share their batches
    assert max(r["batches"]) > 1 and sum(r["batches"]) < 240          # classify inputs are not counted here
    assert 'lorax_batch_inference_failure{method="embed"}' in r["metrics"] and "lorax_request_queue_duration_bucket" in r["metrics"]
