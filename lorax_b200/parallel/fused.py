"""In-kernel NVLink collectives for tensor parallelism.

`enable(tp, model)` allocates one symmetric buffer per rank (CUDA VMM allocation exported to every peer through
`torch.distributed._symmetric_memory`, which is only used for the rendezvous and the peer pointers) and attaches a
:class:`FusedCollectives` to the process group.  The data movement itself happens inside this library's kernels
(`csrc/kernels/gemm_allreduce.cu`): peer stores and system-scope atomics over NVLink, no NCCL call on the hot path.

* `gemm_allreduce`  row-parallel O / down projection: GEMM -> reduce-scatter -> all-gather in one kernel, with the
  rank's partial LoRA delta riding along as an addend (replaces GEMM + NCCL all-reduce + LoRA collectives, call
  sites C2 / C3 / C5 of the reference: `utils/layers.py:279-300, 329-374`).
* `embed`           vocabulary-parallel embedding by peer reads: every rank fetches the rows it needs from the owner's shard,
  the [T, H] all-reduce of call site C1 (`layers/tensor_parallel.py:153-190`) disappears.
* `all_reduce`      two-shot all-reduce kernel (`csrc/kernels/allreduce_sym.cu`): every rank reduces its slice with
  16-byte peer loads and stores the result to all ranks; the row-parallel GEMM writes its partial straight into the
  symmetric input area, so there is no staging copy.
* `argmax_tp`       greedy sampling over vocabulary-parallel logits exchanging 16 bytes per row instead of
  all-gathering the logits (C6, `layers/tensor_parallel.py:50-79`).

Every device-side wait is bounded; `check()` reads the status word.
"""

from __future__ import annotations

import ctypes
import json
import os
from typing import Optional

import torch

from ..ops import native


class FusedCollectives:
    MAX_TOKENS = 256          # kernel limit

    def __init__(self, tp, n_max: int, max_rows: int = 512):
        import os
        # plain peer mappings only: this library never issues multimem instructions, and memory that is not bound to an
        # NVLink multicast object cannot fault peers if a rank dies
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        try:
            symm.set_backend("CUDA")
        except Exception:
            pass
        lib = native.load()
        P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.lx_ar_layout.argtypes = [I, I, I, ctypes.POINTER(L)]
        lib.lx_ar_layout.restype = L
        lib.lx_gemm_allreduce.argtypes = [P, L, P, L, P, P, L, I, I, I, P, I, I, ctypes.POINTER(L), I, P, I, P]
        lib.lx_gemm_allreduce.restype = I
        lib.lx_argmax_tp.argtypes = [P, L, I, I, I, P, P, P, I, I, ctypes.POINTER(L), I, P, P]
        lib.lx_argmax_tp.restype = I
        lib.lx_embed_peer.argtypes = [P, P, P, I, I, I, I, I, ctypes.c_float, P]
        lib.lx_embed_peer.restype = I
        self.embed_ptrs = None
        lib.lx_allreduce_sym.argtypes = [P, I, I, L, L, L, L, P, P, P]
        lib.lx_allreduce_sym.restype = I
        lib.lx_allreduce_sym_counter_bytes.restype = I
        self.ar_ptrs = None
        self.lib = lib
        self.tp = tp
        self.rank, self.world = tp.rank, tp.world_size
        self.n_max, self.max_rows = n_max, max_rows
        self.layout = (L * 8)()
        nbytes = lib.lx_ar_layout(self.world, n_max, max_rows, self.layout)
        self.buf = symm.empty(nbytes, dtype=torch.uint8, device=tp.device)
        self.buf.zero_()
        torch.cuda.synchronize(tp.device)
        self.handle = symm.rendezvous(self.buf, tp.group)
        ptrs = list(self.handle.buffer_ptrs)
        self.peer_ptrs = (ctypes.c_ulonglong * self.world)(*ptrs)
        out_off = self.layout[1]
        self.out = self.buf[out_off: out_off + self.MAX_TOKENS * n_max * 2].view(torch.bfloat16).view(self.MAX_TOKENS, n_max)
        self.ws = native.workspace(tp.device)
        # Batches above this size go through GEMM + NCCL all-reduce instead: measured on 2 x B200, the fused kernel is
        # at parity up to ~32 tokens and slower beyond (see profiles/fused_gemm_allreduce_tp2.txt).
        self.max_fused_tokens = int(os.environ.get("LORAX_FUSED_MAX_TOKENS", "32"))
        tp.barrier()
        self.calls = 0

    def gemm_allreduce(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                       addend: Optional[torch.Tensor] = None) -> torch.Tensor:
        """-> view [T, N] of the symmetric output buffer, valid until the next fused call."""
        T, K = x.shape
        N = w.shape[0]
        assert T <= self.MAX_TOKENS and N <= self.n_max
        rc = self.lib.lx_gemm_allreduce(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), bias.data_ptr() if bias is not None else None,
                                        addend.data_ptr() if addend is not None else None, addend.stride(0) if addend is not None else 0,
                                        T, N, K, ctypes.cast(self.peer_ptrs, ctypes.c_void_p), self.rank, self.world, self.layout, self.n_max,
                                        self.ws.status.data_ptr(), self.ws.num_sms, torch.cuda.current_stream().cuda_stream)
        native._check(rc, "lx_gemm_allreduce")
        self.calls += 1
        return self.out[:T, :N]

    def argmax_tp(self, logits: torch.Tensor, vocab_start: int, ids: torch.Tensor, logprobs: torch.Tensor):
        T, V = logits.shape
        rc = self.lib.lx_argmax_tp(logits.data_ptr(), logits.stride(0), T, V, vocab_start, ids.data_ptr(), logprobs.data_ptr(),
                                   ctypes.cast(self.peer_ptrs, ctypes.c_void_p), self.rank, self.world, self.layout, self.max_rows,
                                   self.ws.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        native._check(rc, "lx_argmax_tp")

    def share_embedding(self, table: torch.Tensor, vocab: int) -> torch.Tensor:
        """Move this rank's embedding shard [rows, H] into peer-mapped memory and exchange the pointers.  Returns the new
        home of the shard (the caller drops the old tensor)."""
        import torch.distributed._symmetric_memory as symm
        shared = symm.empty(table.shape, dtype=table.dtype, device=table.device)
        shared.copy_(table)
        torch.cuda.synchronize(table.device)
        self.embed_handle = symm.rendezvous(shared, self.tp.group)
        self.embed_ptrs = (ctypes.c_ulonglong * self.world)(*list(self.embed_handle.buffer_ptrs))
        self.embed_rows, self.embed_vocab, self.embed_h = table.shape[0], vocab, table.shape[1]
        self.tp.barrier()
        return shared

    def embed(self, ids: torch.Tensor, mult: float = 1.0) -> torch.Tensor:
        """Embedding rows read from their owner's memory: [T] ids -> [T, H], no all-reduce."""
        T = ids.shape[0]
        out = torch.empty(T, self.embed_h, dtype=torch.bfloat16, device=ids.device)
        rc = self.lib.lx_embed_peer(ids.data_ptr(), ctypes.cast(self.embed_ptrs, ctypes.c_void_p), out.data_ptr(), T, self.embed_h,
                                    self.embed_rows, self.world, self.embed_vocab, mult, torch.cuda.current_stream().cuda_stream)
        native._check(rc, "lx_embed_peer")
        native.launch_count += 1
        return out

    def setup_all_reduce(self, max_tokens: int, hidden: int):
        """Symmetric buffer of the two-shot all-reduce kernel: [input | output | counters]."""
        import torch.distributed._symmetric_memory as symm
        area = (max_tokens * hidden * 2 + 255) // 256 * 256
        cnt = self.lib.lx_allreduce_sym_counter_bytes()
        self.ar_buf = symm.empty(2 * area + cnt, dtype=torch.uint8, device=self.tp.device)
        self.ar_buf.zero_()
        torch.cuda.synchronize(self.tp.device)
        self.ar_handle = symm.rendezvous(self.ar_buf, self.tp.group)
        self.ar_ptrs = (ctypes.c_ulonglong * self.world)(*list(self.ar_handle.buffer_ptrs))
        self.ar_area, self.ar_capacity = area, max_tokens * hidden
        self.ar_state = torch.zeros(2, dtype=torch.int32, device=self.tp.device)
        self.ar_in = self.ar_buf[:area].view(torch.bfloat16)
        self.ar_out = self.ar_buf[area: 2 * area].view(torch.bfloat16)
        self.ar_calls = 0
        self.tp.barrier()

    def all_reduce_input(self, T: int, N: int) -> Optional[torch.Tensor]:
        """Where the producer of an all-reduce operand should write it ([T, N] bf16 inside the symmetric buffer), or None
        when the operand does not fit (the caller then takes NCCL)."""
        if self.ar_ptrs is None or T * N > self.ar_capacity or (T * N) % 8:
            return None
        return self.ar_in[: T * N].view(T, N)

    def all_reduce(self, x: torch.Tensor):
        """Sum over the ranks with the in-kernel two-shot all-reduce.  Returns a [T, N] view of the output area, valid until
        the next call, or None when the tensor is not eligible (NCCL is used then).  An operand that already sits in
        `all_reduce_input` is reduced in place, anything else is copied there first."""
        if self.ar_ptrs is None or x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_contiguous():
            return None
        T, N = x.shape
        src = self.all_reduce_input(T, N)
        if src is None:
            return None
        if x.data_ptr() != src.data_ptr():
            src.copy_(x)
        rc = self.lib.lx_allreduce_sym(ctypes.cast(self.ar_ptrs, ctypes.c_void_p), self.rank, self.world, 0, self.ar_area, 2 * self.ar_area,
                                       T * N, self.ar_state.data_ptr(), self.ws.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        native._check(rc, "lx_allreduce_sym")
        native.launch_count += 1
        self.ar_calls += 1
        return self.ar_out[: T * N].view(T, N)

    def all_reduce_self_test(self) -> bool:
        """Two reductions of known values (a small and a large one, odd sizes) against the exact sums.  The outcome is combined
        over the ranks with NCCL, so either every rank uses the kernel or none does."""
        import torch.distributed as dist
        ok = True
        for T in (3, 517):
            N = 4096 if self.ar_capacity >= 517 * 4096 else max(8, (self.ar_capacity // 517) // 8 * 8)
            x = torch.arange(T * N, device=self.tp.device, dtype=torch.float32).remainder(7).add(self.rank + 1).view(T, N).to(torch.bfloat16)
            got = self.all_reduce(x)
            if got is None:
                ok = False
                break
            want = torch.arange(T * N, device=self.tp.device, dtype=torch.float32).remainder(7).view(T, N) * self.world + \
                self.world * (self.world + 1) / 2
            torch.cuda.synchronize(self.tp.device)
            ok = ok and bool(torch.equal(got.float(), want))
        try:
            self.ws.check_status()
        except Exception:
            ok = False
        flag = torch.tensor([1.0 if ok else 0.0], device=self.tp.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.tp.group)
        return bool(flag.item() > 0)

    def check(self):
        self.ws.check_status()


def enable(tp, model, max_rows: int = 512) -> FusedCollectives:
    if tp.world_size == 1:
        raise ValueError("fused collectives need a tensor-parallel group")
    fc = FusedCollectives(tp, n_max=model.hidden, max_rows=max_rows)
    if os.environ.get("LORAX_SYM_ALLREDUCE", "1") != "0" and not model.config.parallel_residual:
        # (with parallel residuals two all-reduce results are alive at once; the kernel keeps one output area)
        fc.setup_all_reduce(int(os.environ.get("LORAX_SYM_ALLREDUCE_TOKENS", "4352")), model.hidden)
        if not fc.all_reduce_self_test():
            fc.ar_ptrs = None                   # every rank agrees (the outcome is itself reduced): NCCL carries the all-reduces
            print(json.dumps({"level": "WARN", "message": "two-shot all-reduce kernel failed its self test; using NCCL"}), flush=True)
    if model.embed is not None and model.embed.is_cuda and model.embed.dtype == torch.bfloat16 and model.pos_embed is None:
        model.embed = fc.share_embedding(model.embed, model.vocab_local * tp.world_size)
    tp.fused = fc
    return fc
