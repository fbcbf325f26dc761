"""Paged KV cache storage and a block allocator for in-process serving.

Storage: one tensor per layer, `[num_blocks, kv_heads_local, 2, PAGE, head_dim]` -- for every (block, head)
the K plane is followed by the V plane, so the attention kernels fetch a page of one head as one contiguous
run.  Memory is zero-initialised: attention multiplies masked probabilities (exact zeros) with whatever
the cache holds, and 0 * NaN would poison the row.

Block bookkeeping mirrors the router-side allocator of the reference (`router/src/block_allocator.rs:146-216`):
block 0 is reserved for health checks, a request needs ceil(tokens / PAGE) blocks, a sliding-window model never
needs more than ceil(window / PAGE) + 1 blocks per request because old pages are recycled cyclically.
"""

from __future__ import annotations

from typing import List, Optional

import torch

PAGE_SIZE = 32


def kv_dtype_of(model, cfg) -> torch.dtype:
    """The page dtype of a model's cache: e4m3 when the engine config asks for an fp8 cache (value / scale with one K and one
    V scale per layer, `model.kv_scales`; the reference's fp8 KV cache, server/lorax_server/utils/paged_attention.py:23-47),
    else the model's own dtype."""
    want = getattr(cfg, "kv_cache_dtype", None)
    if want in ("fp8", "fp8_e4m3", "float8_e4m3fn"):
        if getattr(model, "kv_scales", None) is None:
            model.kv_scales = [(1.0, 1.0)] * model.config.num_hidden_layers
        return torch.float8_e4m3fn
    if want not in (None, "", "auto"):
        raise ValueError(f"unsupported kv_cache_dtype {want!r} (fp8 or unset)")
    return model.dtype


class KVCache:
    def __init__(self, num_layers: int, num_blocks: int, kv_heads: int, head_dim: int, dtype, device, page: int = PAGE_SIZE):
        self.page = page
        self.num_blocks = num_blocks
        self.layers: List[torch.Tensor] = [
            torch.zeros(num_blocks, kv_heads, 2, page, head_dim, dtype=dtype, device=device) for _ in range(num_layers)
        ]

    @staticmethod
    def bytes_per_block(num_layers: int, kv_heads: int, head_dim: int, dtype, page: int = PAGE_SIZE) -> int:
        return num_layers * kv_heads * 2 * page * head_dim * torch.empty(0, dtype=dtype).element_size()

    @property
    def max_tokens(self) -> int:
        return (self.num_blocks - 1) * self.page


class BlockAllocator:
    def __init__(self, num_blocks: int, page: int = PAGE_SIZE, window: Optional[int] = None):
        self.page = page
        self.window = window
        self.free: List[int] = list(range(num_blocks - 1, 0, -1))     # block 0 reserved
        self.num_blocks = num_blocks

    def blocks_needed(self, tokens: int) -> int:
        if self.window:
            tokens = min(tokens, self.window + self.page)
        return (tokens + self.page - 1) // self.page

    def allocate(self, tokens: int) -> Optional[List[int]]:
        n = self.blocks_needed(tokens)
        if n > len(self.free):
            return None
        out = self.free[-n:][::-1]
        del self.free[-n:]
        return out

    def release(self, blocks: List[int]):
        self.free.extend(reversed(blocks))

    @property
    def free_blocks(self) -> int:
        return len(self.free)


def plan_kv_blocks(model, cfg, max_batch: int, page: int = PAGE_SIZE, reserve_bytes: int = 1 << 30) -> int:
    """How many KV blocks fit, measured instead of guessed: run one prefill of `max_batch_prefill_tokens` tokens (prompts of
    `max_input_length`) against a throw-away cache, read the peak of the allocator, and give the cache what is left of the free
    memory after that peak, the decode state and a reserve for CUDA-graph pools (the reference's warm-up does the same with a
    maximum batch, `server/lorax_server/models/flash_causal_lm.py:1293-1401`).  Under tensor parallelism every rank calls this at
    the same time (the prefill contains collectives) and the ranks agree on the minimum."""
    from .runner import ModelRunner, PrefillItem
    c, dev = model.config, model.device
    kv_dtype = kv_dtype_of(model, cfg)
    per_block = KVCache.bytes_per_block(c.num_hidden_layers, model.nkv, model.d, kv_dtype, page)
    if dev.type != "cuda":
        return 1024
    tokens = max(int(cfg.max_batch_prefill_tokens), 16)
    seq = max(1, min(int(cfg.max_input_length), tokens))
    lens = [seq] * (tokens // seq) + ([tokens % seq] if tokens % seq else [])
    window = c.sliding_window
    blocks_per = [min((n + page - 1) // page, (window + page - 1) // page + 1) if window else (n + page - 1) // page for n in lens]
    tmp = KVCache(c.num_hidden_layers, sum(blocks_per) + 2, model.nkv, model.d, kv_dtype, dev, page)
    runner = ModelRunner(model, tmp, max_batch=max_batch, max_seq_tokens=cfg.max_total_tokens, max_prefill_tokens=tokens, use_graphs=False)
    torch.cuda.synchronize(dev)
    torch.cuda.reset_peak_memory_stats(dev)
    base = torch.cuda.memory_allocated(dev)
    items, nxt = [], 1
    for n, nb in zip(lens, blocks_per):
        items.append(PrefillItem([1] * n, 0, list(range(nxt, nxt + nb))))
        nxt += nb
    runner.prefill(items)
    torch.cuda.synchronize(dev)
    peak = torch.cuda.max_memory_allocated(dev) - base
    del runner, tmp, items
    torch.cuda.empty_cache()
    free, _ = torch.cuda.mem_get_info(dev)
    budget = int(free * cfg.memory_wiggle_room) - int(peak * 1.1) - reserve_bytes
    blocks = max(int(budget // per_block), 64)
    tp = model.tp
    if tp.world_size > 1:
        import torch.distributed as dist
        t = torch.tensor([blocks], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=tp.group)
        blocks = int(t.item())
    return blocks
