"""Tensor parallelism: TP=2 must reproduce TP=1 (CPU ranks over Gloo here; NCCL and the fused NVLink kernels on
GPUs).  The worker is tests/tp_worker.py."""
import json
import os
import subprocess
import sys

import pytest
import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(nproc, port, env_extra=None, timeout=600):
    env = dict(os.environ, PYTHONPATH=REPO, **(env_extra or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(REPO, "tests", "tp_worker.py")]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, timeout=timeout, text=True)
    lines = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")]
    assert lines, p.stdout[-3000:]
    return json.loads(lines[-1][7:])


def test_tp2_matches_tp1_on_cpu_ranks():
    r = _launch(2, 29631, {"CUDA_VISIBLE_DEVICES": ""})
    assert r["world"] == 2 and r["device"] == "cpu"
    assert r["model_gloo_logits_relerr"] < 1e-4
    assert r["model_gloo_first_tokens_equal"] and r["model_gloo_decode_tokens_equal"] == 1.0


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_nccl_and_fused_kernels(world):
    """TP = 2, 4 and 8 against TP = 1 (logits and first tokens, NCCL collectives and the in-kernel NVLink ones), and the fused
    kernels against fp32 sums assembled with NCCL.  NVLS is off: ranks may leave while peers still run."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    r = _launch(world, 29630 + world, {"NCCL_NVLS_ENABLE": "0"})
    assert r["world"] == world
    assert r["model_nccl_logits_relerr"] < 3e-2 and r["model_fused_logits_relerr"] < 3e-2
    assert r["model_fused_first_tokens_equal"]
    assert r["fused_calls"] > 0
    assert r["gemm_allreduce_relerr"] < 6e-3 and r["gemm_allreduce_ranks_identical"]
    assert r["allreduce_sym_relerr"] < 6e-3 and r["allreduce_sym_ranks_identical"]
    assert r["argmax_tp_ok"]
    assert r["sampled_shards_path_taken"] and r["sampled_from_shards_equals_gathered"]
