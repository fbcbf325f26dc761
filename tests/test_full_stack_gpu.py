"""The served path on a B200: C++ router in front of a CUDA shard runtime (bf16 kernels, CUDA graphs, adapters loaded
on demand), driven over HTTP.  Checks that the GPU path produces the engine's tokens for a lone request, that adapters
change the output, that concurrent requests of different adapters complete, and that sampling and streaming work."""
import concurrent.futures
import json
import subprocess
import time
import urllib.request

import pytest
import torch
from safetensors.torch import save_file

from test_full_stack import ROUTER, _free_port, _post

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu_stack(tmp_path_factory):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from lorax_b200.adapters.lora import random_adapter, save_peft_adapter
    from lorax_b200.config import EngineConfig, tiny_llama
    from lorax_b200.csrc import build
    from lorax_b200.models.decoder import DecoderModel
    from lorax_b200.models.loading import export_hf_state_dict
    build.build_host()
    root = tmp_path_factory.mktemp("gstack")
    cfg = tiny_llama(vocab_size=512)
    cfg.eos_token_id = 1
    cfg.torch_dtype = "bfloat16"
    model = DecoderModel.random_init(cfg, "cpu", torch.float32, seed=0)
    mdir = root / "model"
    mdir.mkdir()
    save_file({k: v.to(torch.bfloat16) for k, v in export_hf_state_dict(model).items()}, str(mdir / "model.safetensors"),
              metadata={"format": "pt"})
    d = cfg.to_dict()
    d["architectures"] = ["LlamaForCausalLM"]
    (mdir / "config.json").write_text(json.dumps(d))
    vocab = {f"w{i}": i for i in range(512)}
    vocab["<unk>"] = 0
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(mdir / "tokenizer.json"))
    for i in range(3):
        c, mm = random_adapter(cfg, r=[8, 16, 32][i], alpha=16, target_modules=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"],
                               seed=50 + i, std_a=0.1, std_b=0.1)
        save_peft_adapter(root / f"adapter{i}", c, mm)

    from lorax_b200.server.runtime import build_runtime
    from lorax_b200.server.transport import FramedServer
    ecfg = EngineConfig(max_input_length=64, max_total_tokens=128, max_batch_prefill_tokens=256, compile=True)
    rt = build_runtime(str(mdir), ecfg, device="cuda", dtype=torch.bfloat16, source="local", num_blocks=256, max_batch=16)
    uds = str(root / "shard")
    srv = FramedServer(rt, uds + "-0.lx").start()
    port = _free_port()
    proc = subprocess.Popen([ROUTER, "--port", str(port), "--hostname", "127.0.0.1", "--master-shard-uds-path", uds, "--num-shard", "1",
                             "--max-input-length", "64", "--max-total-tokens", "128", "--max-batch-prefill-tokens", "256",
                             "--model-id", "tiny", "--adapter-source", "local", "--waiting-served-ratio", "0.3"],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    ok = False
    for _ in range(100):
        try:
            with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                ok = r.status == 200
                break
        except Exception:
            time.sleep(0.1)
    if not ok:
        proc.kill()
        raise RuntimeError("router did not come up: " + proc.stdout.read().decode()[-2000:])
    yield dict(port=port, root=root, rt=rt)
    proc.terminate()
    try:
        proc.wait(timeout=10)
    except subprocess.TimeoutExpired:
        proc.kill()
    srv.stop()


def _gen(port, prompt, n=8, **params):
    st, body, _ = _post(port, "/generate", {"inputs": prompt, "parameters": {"max_new_tokens": n, "details": True, "ignore_eos_token": True, **params}})
    assert st == 200, body
    j = json.loads(body)
    assert j["details"]["generated_tokens"] == n
    return [t["id"] for t in j["details"]["tokens"]]


def test_gpu_served_path(gpu_stack):
    port, root, rt = gpu_stack["port"], gpu_stack["root"], gpu_stack["rt"]
    prompt = " ".join(f"w{i}" for i in (5, 17, 200, 33, 8, 91, 44, 301))
    base = _gen(port, prompt)
    outs = [_gen(port, prompt, adapter_id=str(root / f"adapter{i}"), adapter_source="local") for i in range(3)]
    assert any(o != base for o in outs)
    assert _gen(port, prompt) == base                      # deterministic, and unaffected by the adapters now resident
    # oracle for the lone base request: the in-process engine on the same GPU model
    from lorax_b200.config import EngineConfig
    from lorax_b200.runtime.engine import Engine
    saved = rt.model.adapters
    eng = Engine(rt.model, EngineConfig(max_total_tokens=128, max_batch_prefill_tokens=256), num_blocks=64, max_batch=4)
    want = eng.generate([[5, 17, 200, 33, 8, 91, 44, 301]], max_new_tokens=8)[0]
    rt.model.adapters = saved
    assert base == want

    # concurrent heterogeneous load: 24 requests over base + 3 adapters, different lengths
    def one(i):
        params = {} if i % 4 == 0 else {"adapter_id": str(root / f"adapter{i % 4 - 1}"), "adapter_source": "local"}
        p = " ".join(f"w{(7 * i + j) % 500 + 2}" for j in range(4 + i % 9))
        return len(_gen(port, p, n=5 + i % 11, **params)) == 5 + i % 11
    with concurrent.futures.ThreadPoolExecutor(8) as ex:
        assert all(ex.map(one, range(24)))
    # after the storm a lone request still gives the same tokens
    assert _gen(port, prompt) == base

    # sampling with a seed is reproducible; streaming delivers one event per token
    a = _gen(port, prompt, do_sample=True, temperature=0.8, top_k=20, seed=7)
    b = _gen(port, prompt, do_sample=True, temperature=0.8, top_k=20, seed=7)
    assert a == b
    st, body, _ = _post(port, "/generate_stream", {"inputs": prompt, "parameters": {"max_new_tokens": 6, "ignore_eos_token": True}})
    assert st == 200
    events = [json.loads(l[5:]) for l in body.replace("\r", "").split("\n") if l.startswith("data:")]
    assert len(events) == 6 and events[-1]["generated_text"] is not None
    from lorax_b200.ops import native
    native.workspace().check_status()
