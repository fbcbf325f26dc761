"""The GEMM entry point that allocates nothing, called through its exported C symbol.

Who needs it: a caller that may not allocate device memory at call time (a host that bans cudaMalloc after
start-up, a plugin that must not touch its host framework's allocator) cannot pass the split-K scratch that the
regular entry point wants, so the library carries a fixed scratch array for them.  The test calls the symbol
with ctypes exactly as such a caller would (inputs and outputs are the caller's own buffers), twice in a row
because the second call finds the first call's leftovers in the shared array, and compares with the regular
entry point.  The file name sorts last so that a failure here cannot hide another test's result.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from lorax_b200.ops import native
    lib = native.load()
    f = lib.lx_gemm_bf16_noalloc
    f.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 3 + [ctypes.c_longlong] * 3 + [ctypes.c_int, ctypes.c_void_p]
    f.restype = ctypes.c_int
    lib.lx_gemm_bf16_noalloc_strerror.argtypes = [ctypes.c_int]
    lib.lx_gemm_bf16_noalloc_strerror.restype = ctypes.c_char_p
    lib.lx_gemm_bf16_noalloc_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.lx_gemm_bf16_noalloc_status.restype = ctypes.c_int
    lib.lx_gemm_bf16_noalloc_scratch_bytes.restype = ctypes.c_longlong
    return native, lib


def _call(lib, x, w, out, bias, split):
    T, K = x.shape
    N = w.shape[0]
    return lib.lx_gemm_bf16_noalloc(x.data_ptr(), w.data_ptr(), out.data_ptr(), bias.data_ptr() if bias is not None else None,
                                    T, N, K, x.stride(0), w.stride(0), out.stride(0), split, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("T,N,K,split", [(8, 4096, 4096, 0), (100, 1024, 14336, 4), (256, 512, 2048, 2)])
def test_noalloc_matches_regular_entry_twice(T, N, K, split):
    native, lib = _lib()
    torch.manual_seed(11)
    outs = []
    for call in range(2):       # second call: the static scratch holds the first call's partials and counters
        x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / math.sqrt(K)
        b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
        got = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        rc = _call(lib, x, w, got, b, split)
        assert rc == 0, lib.lx_gemm_bf16_noalloc_strerror(rc)
        st = (ctypes.c_int * 2)()
        assert lib.lx_gemm_bf16_noalloc_status(st, torch.cuda.current_stream().cuda_stream) == 0 and st[0] == 0, list(st)
        want = native.gemm(x, w, bias=b, mode=1, force_split=split)
        torch.cuda.synchronize()
        native.workspace().check_status()
        err = ((got.float() - want.float()).norm() / want.float().norm()).item()
        assert err < 6e-3, (call, err)
        ref = x.float() @ w.float().t() + b.float()
        assert ((got.float() - ref).norm() / ref.norm()).item() < 6e-3
        outs.append(err)


def test_noalloc_on_a_non_blocking_stream():
    """The status read is ordered on the caller's stream, so it is right on streams that do not synchronise with the
    default stream too."""
    native, lib = _lib()
    torch.manual_seed(5)
    s = torch.cuda.Stream()
    x = torch.randn(32, 2048, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(1024, 2048, device="cuda", dtype=torch.bfloat16) / math.sqrt(2048)
    got = torch.empty(32, 1024, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        rc = _call(lib, x, w, got, None, 4)
        assert rc == 0, lib.lx_gemm_bf16_noalloc_strerror(rc)
        st = (ctypes.c_int * 2)()
        assert lib.lx_gemm_bf16_noalloc_status(st, s.cuda_stream) == 0 and st[0] == 0, list(st)
    ref = x.float() @ w.float().t()
    assert ((got.float() - ref).norm() / ref.norm()).item() < 6e-3
    assert _call(lib, x[:, :0], w[:, :0], got, None, 0) == -2006            # K = 0 is refused, not launched


def test_noalloc_rejects_oversize():
    native, lib = _lib()
    x = torch.zeros(300, 64, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(128, 64, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(300, 128, device="cuda", dtype=torch.bfloat16)
    rc = _call(lib, x, w, out, None, 0)
    assert rc == -2003 and b"256" in lib.lx_gemm_bf16_noalloc_strerror(rc)
    # 256 tokens x 32768 features x split 16 would need 256 tiles * 16 * 128 KiB of partials: far beyond 8 MiB
    x = torch.zeros(256, 4096, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(32768, 4096, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(256, 32768, device="cuda", dtype=torch.bfloat16)
    rc = _call(lib, x, w, out, None, 16)
    assert rc == -2005, lib.lx_gemm_bf16_noalloc_strerror(rc)
    assert lib.lx_gemm_bf16_noalloc_scratch_bytes() == (8 << 20) + 4096 + 16
