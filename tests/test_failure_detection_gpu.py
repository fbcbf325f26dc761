"""A wait for another GPU that runs out: the kernel must return, report where it gave up, and leave the context usable.

No second GPU and no fault is involved.  The two-shot all-reduce kernel is launched as rank 0 of a group of two whose
two "peer" pointers both name one local buffer, so the flags that rank 1 would post are simply never written; the wait
budget is shortened to two milliseconds through the library's setting.  Afterwards the flags of the absent rank are
written by the host, and the same launch completes and sums the buffer with itself.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup():
    from lorax_b200.ops import native
    lib = native.load()
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib.lx_allreduce_sym.argtypes = [P, I, I, L, L, L, L, P, P, P]
    lib.lx_allreduce_sym.restype = I
    lib.lx_allreduce_sym_counter_bytes.restype = I
    lib.lx_allreduce_sym_blocks.restype = I
    lib.lx_set_wait_budget_ns.argtypes = [ctypes.c_ulonglong]
    lib.lx_set_wait_budget_ns.restype = None
    lib.lx_get_wait_budget_ns.restype = ctypes.c_ulonglong
    return native, lib


def test_all_reduce_gives_up_on_an_absent_peer_and_recovers():
    native, lib = _setup()
    n = 4096 * 8                                   # bf16 elements to reduce
    area = n * 2
    cnt = lib.lx_allreduce_sym_counter_bytes()
    buf = torch.zeros(2 * area + cnt, dtype=torch.uint8, device="cuda")
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    x = torch.randn(n, device="cuda").to(torch.bfloat16)
    buf[:area].view(torch.bfloat16).copy_(x)
    peers = (ctypes.c_ulonglong * 2)(buf.data_ptr(), buf.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.lx_get_wait_budget_ns() == 2_000_000_000
    lib.lx_set_wait_budget_ns(2_000_000)           # 2 ms
    try:
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        rc = lib.lx_allreduce_sym(ctypes.cast(peers, ctypes.c_void_p), 0, 2, 0, area, 2 * area, n, state.data_ptr(), status.data_ptr(), stream)
        t1.record()
        assert rc == 0
        torch.cuda.synchronize()                   # the kernel returned by itself
        assert t0.elapsed_time(t1) < 500.0
        st = status.tolist()
        blocks = lib.lx_allreduce_sym_blocks()
        assert st[0] == 5 and 4000 <= st[1] < 4000 + blocks, st       # kTimeoutPeerFlag at the first barrier of some block
        assert state.tolist() == [1, 0]            # the launch counter still advanced: the next launch uses fresh flag values
        # the context is usable: an ordinary kernel of the library runs and is right
        a = torch.randn(64, 512, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16) / 16
        got = native.gemm(a, w)
        torch.cuda.synchronize()
        ref = a.float() @ w.float().t()
        assert ((got.float() - ref).norm() / ref.norm()).item() < 6e-3
        # now "rank 1" shows up: the host writes the flags it would have posted (both stages, every block), far ahead of any launch
        status.zero_()
        flags = buf[2 * area:].view(torch.int32).view(2, blocks, 8)
        flags[:, :, 1] = 1 << 30
        torch.cuda.synchronize()
        rc = lib.lx_allreduce_sym(ctypes.cast(peers, ctypes.c_void_p), 0, 2, 0, area, 2 * area, n, state.data_ptr(), status.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0]
        out = buf[area: 2 * area].view(torch.bfloat16)
        # rank 0 reduces the first half of the elements (its slice) from "both" inputs, which are the same buffer
        half = n // 2
        assert torch.equal(out[:half].float(), (x[:half].float() * 2).to(torch.bfloat16).float())
    finally:
        lib.lx_set_wait_budget_ns(0)
    assert lib.lx_get_wait_budget_ns() == 2_000_000_000


def test_status_word_reaches_the_host_with_the_step_result():
    """A kernel that gave up on a wait writes the status word; it travels in the pinned result ring with the step's tokens, so the
    engine fails that step without an extra synchronisation, the word is cleared, and the next request is served."""
    from lorax_b200.config import EngineConfig, tiny_llama
    from lorax_b200.models.decoder import DecoderModel
    from lorax_b200.ops import native
    from lorax_b200.runtime.engine import Engine
    cfg = tiny_llama()
    model = DecoderModel.random_init(cfg, torch.device("cuda", 0), torch.bfloat16, seed=0)
    eng = Engine(model, EngineConfig(max_total_tokens=128, max_batch_prefill_tokens=256), num_blocks=64, max_batch=4)
    want = eng.generate([[5, 6, 7, 8, 9]], max_new_tokens=4)[0]
    ws = native.workspace(model.device)
    ws.status.copy_(torch.tensor([5, 4007], dtype=torch.int32))          # what a timed-out peer wait leaves behind
    with pytest.raises(native.NativeError, match="peer flag timeout.*4007"):
        eng.generate([[5, 6, 7, 8, 9]], max_new_tokens=4)
    assert ws.status.tolist() == [0, 0] and "4007" in eng.runner.device_failed
    # a fresh engine on the same context serves again
    eng2 = Engine(model, EngineConfig(max_total_tokens=128, max_batch_prefill_tokens=256), num_blocks=64, max_batch=4)
    assert eng2.generate([[5, 6, 7, 8, 9]], max_new_tokens=4)[0] == want
