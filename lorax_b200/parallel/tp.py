"""Tensor-parallel process group: one process per GPU, `torch.distributed` (NCCL on GPUs, Gloo on CPU).

Collective placement follows the reference (`server/lorax_server/utils/layers.py:329-409`,
`layers/tensor_parallel.py:50-79`): all-reduce after the row-parallel O / down projections and after the
vocab-parallel embedding, all-gather of the vocab-parallel logits.  LoRA needs no collective of its own
here: column-parallel groups keep A replicated and shard B with the base weight, row-parallel groups shard
A with the input features and add their partial `(x_shard A_shard^T) B^T` to the partial GEMM output before
the all-reduce, which sums both (the reference issues an extra all-gather / all-reduce per adapter rank
group, `utils/layers.py:257-300`).

`TensorParallel.all_reduce` dispatches to the in-kernel NVLink path (:mod:`lorax_b200.parallel.fused`) when
that has been set up, and to NCCL otherwise (baseline mode).
"""

from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist


class TensorParallel:
    def __init__(self, rank: int, world_size: int, group=None, device=None):
        self.rank = rank
        self.world_size = world_size
        self.group = group
        self.device = device
        self.fused = None            # set by parallel.fused.enable() on NVLink machines
        self.nccl_calls = 0

    @classmethod
    def single(cls) -> "TensorParallel":
        return cls(0, 1)

    @classmethod
    def init_from_env(cls, backend: Optional[str] = None, timeout_s: int = 60) -> "TensorParallel":
        """Rendezvous through RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (`utils/dist.py:48-83` of the reference
        uses the same env contract and the same 60 s timeout)."""
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world == 1:
            dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
            if dev.type == "cuda":
                torch.cuda.set_device(dev)
            return cls(0, 1, None, dev)
        use_cuda = torch.cuda.is_available()
        backend = backend or ("nccl" if use_cuda else "gloo")
        if use_cuda:
            local = int(os.environ.get("LOCAL_RANK", rank % torch.cuda.device_count()))
            dev = torch.device("cuda", local)
            torch.cuda.set_device(dev)
        else:
            dev = torch.device("cpu")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if not dist.is_initialized():
            kw = {}
            if backend == "nccl":
                kw["device_id"] = dev
            dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s), **kw)
        return cls(rank, world, dist.group.WORLD, dev)

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return x
        if self.fused is not None and x.is_cuda:
            y = self.fused.all_reduce(x)
            if y is not None:
                return y
        self.nccl_calls += 1
        dist.all_reduce(x, group=self.group)
        return x

    def all_gather_cols(self, x: torch.Tensor) -> torch.Tensor:
        """[T, n] per rank -> [T, n * world] with rank r's block at columns [r*n, (r+1)*n)."""
        if self.world_size == 1:
            return x
        self.nccl_calls += 1
        T, n = x.shape
        if x.is_cuda:
            out = torch.empty(self.world_size * T, n, dtype=x.dtype, device=x.device)
            dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
            return out.view(self.world_size, T, n).permute(1, 0, 2).reshape(T, self.world_size * n)
        parts = [torch.empty_like(x) for _ in range(self.world_size)]     # Gloo has no all_gather_into_tensor
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)

    def all_gather_stack(self, x: torch.Tensor) -> torch.Tensor:
        """x per rank -> [world, *x.shape] (small tensors: sampling candidates)."""
        if self.world_size == 1:
            return x[None]
        self.nccl_calls += 1
        x = x.contiguous()
        if x.is_cuda:
            out = torch.empty((self.world_size,) + tuple(x.shape), dtype=x.dtype, device=x.device)
            dist.all_gather_into_tensor(out, x, group=self.group)
            return out
        parts = [torch.empty_like(x) for _ in range(self.world_size)]
        dist.all_gather(parts, x, group=self.group)
        return torch.stack(parts)

    def barrier(self):
        if self.world_size > 1:
            dist.barrier(group=self.group)

    def broadcast_object(self, obj, src: int = 0):
        if self.world_size == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]

    def max_scalar(self, v: float) -> float:
        if self.world_size == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=self.device if self.device is not None and self.device.type == "cuda" else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())

    def broadcast_scalar(self, v: float, src: int = 0) -> float:
        """Rank `src`'s value on every rank, through a host-side (Gloo) group so that no GPU work is queued or waited for:
        used for decisions every rank must take alike from a host clock (request arrivals).  Collective on first use."""
        if self.world_size == 1:
            return v
        if getattr(self, "_host_group", None) is None:
            self._host_group = dist.new_group(backend="gloo")
        t = torch.tensor([v], dtype=torch.float64)
        dist.broadcast(t, src=src, group=self._host_group)
        return float(t[0])

    def destroy(self):
        if self.world_size > 1 and dist.is_initialized():
            dist.destroy_process_group()
