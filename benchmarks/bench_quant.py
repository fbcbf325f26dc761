"""Weight-only 4-bit GEMM against the bf16 tcgen05 GEMM on the projection shapes of a 7B model (python benchmarks/bench_quant.py).

Every timing is a CUDA graph of 20 calls rotating through more than 126 MB of weights (larger than L2), best of 5 replays,
CUDA events on the launching stream."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

from lorax_b200.ops import native
from lorax_b200.utils import quant_formats as qf

def timeit(fn, reps=20):
    for _ in range(3): fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps): fn(i)
    g.replay(); torch.cuda.synchronize()
    best = 1e9
    for _ in range(5):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); g.replay(); e.record(); torch.cuda.synchronize()
        best = min(best, s.elapsed_time(e) * 1e3 / reps)
    return best
for (N, K) in ((6144, 4096), (28672, 4096), (4096, 14336)):
    nrot = max(2, int(300e6 / (N * K / 2)) + 1)
    nrot_b = max(2, int(300e6 / (N * K * 2)) + 1)
    wq = []
    base = qf.quantize_rtn(torch.randn(N, K) * 0.02, 4, 128).to("cuda")
    for i in range(nrot):
        wq.append(qf.GroupQuantWeight(base.codes.clone(), base.sz.clone(), 4, 128, (N, K)))
    wb = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(nrot_b)]
    for T in (1, 8, 16, 32):
        x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        lib = native.load()
        def f4(i=0):
            w = wq[i % nrot]
            lib.lx_wq4_gemm_ex(x.data_ptr(), x.stride(0), w.codes.data_ptr(), w.sz.data_ptr(), None, out.data_ptr(), out.stride(0), T, N, K, 128, 1, torch.cuda.current_stream().cuda_stream)
        def fb(i=0):
            native.gemm(x, wb[i % nrot_b], out=out)
        t4, tb = timeit(f4), timeit(fb)
        print(f"N={N} K={K} T={T}: int4 direct {t4:.1f} us ({N*K/2/t4/1e3:.0f} GB/s of codes)  bf16 tcgen05 {tb:.1f} us ({N*K*2/tb/1e3:.0f} GB/s)", flush=True)
    def fd(i=0):
        native.wq_dequant(wq[i % nrot], out=wb[0])
    td = timeit(fd)
    print(f"N={N} K={K}: expansion {td:.1f} us ({N*K*2.5/td/1e3:.0f} GB/s read+write)", flush=True)
    del wq, wb
