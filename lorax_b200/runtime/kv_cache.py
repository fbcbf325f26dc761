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
