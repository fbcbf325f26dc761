"""Shard-side adapter store and exchange engine.

Three tiers:
  disk / hub   PEFT directories (read once)
  host DRAM    packed, TP-pre-sharded, pre-scaled blobs in pinned memory (`HostTier`, LRU by bytes)
  HBM          one bf16 arena sized by `adapter_memory_fraction`; resident adapters occupy contiguous ranges

Loading an adapter into HBM is one `cudaMemcpyAsync` from the pinned blob on a dedicated copy stream,
followed by the update of the two-int slot table entry on the same stream and an event; the compute stream
waits on that event before the first step that schedules the adapter.  Eviction only frees the arena range
and clears the slot entry -- the pinned copy stays, so a re-load never touches the disk.  The reference has
no host tier: "offload" drops the tensors and a re-load re-reads the safetensors file synchronously on the
compute stream (`server/lorax_server/models/model.py:336-450`, `utils/weights.py:555-567`).

The slot table (slot_base / slot_rank, device resident) is what the LoRA kernels index with the per-token
slot id, so a decode CUDA graph does not depend on which adapters or ranks are in the batch.
"""

from __future__ import annotations

import threading
import time
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .lora import LM_HEAD, BlobLayout, LoraConfig, ModuleMap, check_architecture, pad_rank

TMAP_GROUPS = ("qkv", "o", "gate_up", "down", LM_HEAD)     # index of a group inside a slot's tensor-map row
TMAP_BYTES = 128


@dataclass
class LoraTiles:
    """Tile table of one step: int32 [n, 4] rows (slot, first row, rows, 0) on the model's device."""
    table: torch.Tensor
    num_tiles: int
    max_rows: int
    live: int = 0               # live entries when the table is padded with dead ones to a fixed size (0: all of them)


class ArenaAllocator:
    """First-fit allocator with coalescing over a 1-D element range (offsets aligned to `align` elements)."""

    def __init__(self, capacity: int, align: int = 64):
        self.capacity = capacity
        self.align = align
        self.free: List[Tuple[int, int]] = [(0, capacity)]     # (offset, size), sorted by offset
        self.used: Dict[int, int] = {}

    def alloc(self, size: int) -> Optional[int]:
        size = (size + self.align - 1) // self.align * self.align
        for i, (off, sz) in enumerate(self.free):
            if sz >= size:
                if sz == size:
                    self.free.pop(i)
                else:
                    self.free[i] = (off + size, sz - size)
                self.used[off] = size
                return off
        return None

    def release(self, off: int):
        size = self.used.pop(off)
        self.free.append((off, size))
        self.free.sort()
        merged: List[Tuple[int, int]] = []
        for o, s in self.free:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + s)
            else:
                merged.append((o, s))
        self.free = merged

    @property
    def free_elems(self) -> int:
        return sum(s for _, s in self.free)

    @property
    def largest_free(self) -> int:
        return max((s for _, s in self.free), default=0)


@dataclass
class HostBlob:
    key: str
    blob: torch.Tensor       # pinned when CUDA is present
    rank: int                # padded rank
    nbytes: int


class HostTier:
    """Pinned host cache of packed blobs, LRU-bounded by bytes.  Entries that are resident in HBM are never
    dropped (their pinned copy is the reload source after an eviction)."""

    def __init__(self, capacity_bytes: int):
        self.capacity = capacity_bytes
        self.entries: "OrderedDict[str, HostBlob]" = OrderedDict()
        self.bytes = 0
        self.lock = threading.Lock()

    def get(self, key: str) -> Optional[HostBlob]:
        with self.lock:
            hb = self.entries.get(key)
            if hb is not None:
                self.entries.move_to_end(key)
            return hb

    def put(self, hb: HostBlob, pinned_keys=()):
        with self.lock:
            if hb.key in self.entries:
                self.bytes -= self.entries.pop(hb.key).nbytes
            self.entries[hb.key] = hb
            self.bytes += hb.nbytes
            for k in list(self.entries.keys()):
                if self.bytes <= self.capacity:
                    break
                if k == hb.key or k in pinned_keys:
                    continue
                self.bytes -= self.entries.pop(k).nbytes

    def __contains__(self, key):
        return key in self.entries


@dataclass
class Resident:
    adapter_index: int
    key: str
    slot: int
    offset: int
    rank: int
    event: Optional[object]
    loaded_at: float


class AdapterManager:
    def __init__(self, model, arena_bytes: int, host_bytes: int = 16 << 30, max_slots: int = 4096, with_lm_head: bool = False):
        self.model = model
        self.device = model.device
        self.dtype = model.dtype
        self.layout = BlobLayout(model, with_lm_head=with_lm_head)
        esize = torch.empty(0, dtype=self.dtype).element_size()
        self.capacity = max(arena_bytes // esize, 0)
        self.arena = torch.zeros(max(self.capacity, 64), dtype=self.dtype, device=self.device)
        self.alloc = ArenaAllocator(self.capacity)
        self.max_slots = max_slots
        self.slot_base = torch.full((max_slots,), -1, dtype=torch.int64, device=self.device)
        self.slot_rank = torch.zeros(max_slots, dtype=torch.int32, device=self.device)
        self.free_slots = list(range(max_slots - 1, -1, -1))
        self.host = HostTier(host_bytes)
        self.resident: Dict[int, Resident] = {}        # adapter_index -> Resident
        self.key_of_index: Dict[int, str] = {}
        self.max_rank = 0
        self.is_cuda = self.device.type == "cuda"
        self.copy_stream = torch.cuda.Stream(device=self.device) if self.is_cuda else None
        self._pending_events: List[object] = []
        self.stats = dict(h2d_bytes=0, loads=0, evictions=0, host_hits=0, host_misses=0)
        # staging for slot-table updates (pinned so the H2D is async)
        self._stage_base = torch.zeros(1, dtype=torch.int64).pin_memory() if self.is_cuda else None
        self._stage_rank = torch.zeros(1, dtype=torch.int32).pin_memory() if self.is_cuda else None
        # per-slot TMA descriptors, read by the tensor-core LoRA kernels: for every projection group the A_cat family
        # {K, nparts * r, layers} at index g and the B_cat family {r, N, layers} at index len(TMAP_GROUPS) + g
        self.groups_per_slot = 2 * len(TMAP_GROUPS)
        self.slot_tmaps = (torch.zeros(max_slots * self.groups_per_slot * TMAP_BYTES, dtype=torch.uint8, device=self.device)
                           if self.is_cuda else None)
        model.adapters = self

    def _encode_slot_tmaps(self, off: int, rp: int) -> torch.Tensor:
        """Host-side encoding of the slot's tensor maps {K, R, layers} for every projection group."""
        from ..ops import native
        host = torch.zeros(self.groups_per_slot * TMAP_BYTES, dtype=torch.uint8).pin_memory()
        esize = self.arena.element_size()
        for gi_idx, gname in enumerate(TMAP_GROUPS):
            gi = self.layout.groups.get(gname)
            if gi is None:
                continue
            nparts = len(gi.parts)
            base = self.arena.data_ptr() + (off + rp * self.layout.unit_off(gname, 0, "A")) * esize
            layers = 1 if gname == LM_HEAD else self.layout.num_layers
            native.lora_encode_tmap(host[gi_idx * TMAP_BYTES:], base, gi.K, nparts * rp, rp * self.layout.layer_units, layers)
            base_b = self.arena.data_ptr() + (off + rp * self.layout.unit_off(gname, 0, "B")) * esize
            native.lora_encode_tmap_b(host[(len(TMAP_GROUPS) + gi_idx) * TMAP_BYTES:], base_b, rp, gi.N, rp * self.layout.layer_units, layers)
        return host

    # ------------------------------------------------------------------ host tier
    def register(self, key: str, cfg: LoraConfig, mm: ModuleMap) -> HostBlob:
        """Pack an adapter into its pinned host blob (the 'download' step). Returns the host entry."""
        hb = self.host.get(key)
        if hb is not None:
            self.stats["host_hits"] += 1
            return hb
        self.stats["host_misses"] += 1
        check_architecture(cfg, mm, self.model.config)
        blob, rp = self.layout.pack(cfg, mm, dtype=self.dtype, pin=self.is_cuda)
        hb = HostBlob(key, blob, rp, blob.numel() * blob.element_size())
        self.host.put(hb, pinned_keys={r.key for r in self.resident.values()})
        return hb

    def register_blob(self, key: str, blob: torch.Tensor, rank_padded: int) -> HostBlob:
        if self.is_cuda and not blob.is_pinned():
            blob = blob.pin_memory()
        hb = HostBlob(key, blob, rank_padded, blob.numel() * blob.element_size())
        self.host.put(hb, pinned_keys={r.key for r in self.resident.values()})
        return hb

    def memory_fraction(self, key: str) -> float:
        """Cost of the adapter as a fraction of the HBM arena (the router budgets with this number)."""
        hb = self.host.get(key)
        if hb is None or self.capacity == 0:
            return 0.0
        return hb.blob.numel() / self.capacity

    # ------------------------------------------------------------------ HBM tier
    def load(self, adapter_index: int, key: str) -> bool:
        """Make the adapter resident under `adapter_index`; asynchronous on the copy stream."""
        if adapter_index in self.resident:
            return True
        hb = self.host.get(key)
        if hb is None:
            raise KeyError(f"adapter {key!r} has not been downloaded/registered")
        n = hb.blob.numel()
        off = self.alloc.alloc(n)
        if off is None:
            return False
        if not self.free_slots:
            self.alloc.release(off)
            return False
        slot = self.free_slots.pop()
        ev = None
        if self.is_cuda:
            tm_host = self._encode_slot_tmaps(off, hb.rank)
            g = self.groups_per_slot * TMAP_BYTES
            with torch.cuda.stream(self.copy_stream):
                self.arena[off: off + n].copy_(hb.blob, non_blocking=True)
                self.slot_tmaps[slot * g:(slot + 1) * g].copy_(tm_host, non_blocking=True)
                self._stage_base[0] = off
                self._stage_rank[0] = hb.rank
                self.slot_base[slot: slot + 1].copy_(self._stage_base, non_blocking=True)
                self.slot_rank[slot: slot + 1].copy_(self._stage_rank, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
            # the staging words are reused by the next load: wait until this one has been consumed
            ev.synchronize() if len(self._pending_events) > 64 else None
            self._pending_events.append(ev)
            self._stage_base = torch.zeros(1, dtype=torch.int64).pin_memory()
            self._stage_rank = torch.zeros(1, dtype=torch.int32).pin_memory()
        else:
            self.arena[off: off + n].copy_(hb.blob)
            self.slot_base[slot] = off
            self.slot_rank[slot] = hb.rank
        self.resident[adapter_index] = Resident(adapter_index, key, slot, off, hb.rank, ev, time.monotonic())
        self.key_of_index[adapter_index] = key
        self.max_rank = max(self.max_rank, hb.rank)
        self.stats["h2d_bytes"] += hb.nbytes
        self.stats["loads"] += 1
        return True

    def offload(self, adapter_index: int) -> bool:
        r = self.resident.pop(adapter_index, None)
        if r is None:
            return False
        if self.is_cuda:
            # in-flight steps may still read the range: order the release after the compute stream
            torch.cuda.current_stream(self.device).synchronize()
        self.slot_base[r.slot] = -1
        self.slot_rank[r.slot] = 0
        self.alloc.release(r.offset)
        self.free_slots.append(r.slot)
        self.max_rank = max((x.rank for x in self.resident.values()), default=0)
        self.stats["evictions"] += 1
        return True

    def fence(self):
        """Make the compute stream wait for every copy issued so far (call before a step that may use them)."""
        if not self.is_cuda:
            return
        cur = torch.cuda.current_stream(self.device)
        for ev in self._pending_events:
            cur.wait_event(ev)
        self._pending_events.clear()

    def slot_of(self, adapter_index: int) -> int:
        r = self.resident.get(adapter_index)
        return -1 if r is None else r.slot

    def is_loaded(self, adapter_index: int) -> bool:
        return adapter_index in self.resident

    # ------------------------------------------------------------------ compute
    def shrink(self, ops, x: torch.Tensor, tok_slot: Optional[torch.Tensor], group: str, layer: int,
               tiles: Optional[LoraTiles] = None):
        """v = x A_cat(slot(t))^T for the projection group (one launch) -> the descriptor `ops.gemm(..., lora=)` takes to
        add the delta in its epilogue, or None when no row of the step has an adapter.

        With a tile table (rows grouped by adapter) the shrink runs on the tensor cores; without one, the per-token
        kernel is used (rows in any order)."""
        from ..ops.native import LoraEpilogue
        if self.max_rank == 0 or tok_slot is None:
            return None
        gi = self.layout.groups.get(group)
        if gi is None:
            return None
        nparts = len(gi.parts)
        n0, n1 = gi.bounds
        offA, offB = self.layout.unit_off(group, layer, "A"), self.layout.unit_off(group, layer, "B")
        if tiles is not None:
            if tiles.num_tiles == 0:
                return None
            if self.is_cuda:
                v = ops.lora_shrink_tiles(x, tiles.table, tiles.num_tiles, tiles.max_rows, self.slot_tmaps, self.groups_per_slot,
                                          TMAP_GROUPS.index(group), self.slot_rank, nparts, 0 if group == LM_HEAD else layer, self.max_rank,
                                          live_tiles=tiles.live)
            else:
                v = ops.lora_shrink_tiles(x, tiles.table, tiles.num_tiles, tiles.max_rows, self.arena, self.slot_base, self.slot_rank,
                                          offA, nparts, self.max_rank)
        else:
            v = ops.lora_shrink(x, tok_slot, self.arena, self.slot_base, self.slot_rank, offA, nparts, self.max_rank)
        return LoraEpilogue(v, tok_slot, self.arena, self.slot_base, self.slot_rank, offB, n0, n1)

    def fused(self, group: str, layer: int, tiles: Optional[LoraTiles]):
        """Descriptor of the projection group's LoRA for the GEMM that carries shrink and expand in its own launch
        (`ops.gemm_lora_fused`); None when the step has no tile table or nothing is resident."""
        from ..ops.native import LoraFused
        if not self.is_cuda or self.max_rank == 0 or tiles is None or tiles.num_tiles == 0:
            return None
        gi = self.layout.groups.get(group)
        if gi is None:
            return None
        n0, n1 = gi.bounds
        g = TMAP_GROUPS.index(group)
        return LoraFused(tiles.table, tiles.num_tiles, tiles.live, self.slot_tmaps, self.groups_per_slot, g, len(TMAP_GROUPS) + g,
                         self.slot_rank, self.slot_base, len(gi.parts), n0, n1, 0 if group == LM_HEAD else layer, self.max_rank,
                         self.arena, self.layout.unit_off(group, layer, "A"), self.layout.unit_off(group, layer, "B"))

    def expand(self, ops, epi, y: torch.Tensor, tiles: Optional[LoraTiles] = None):
        """y += v B_cat(slot(t))^T: the second half of the LoRA delta as its own launch (`epi` comes from `shrink`)."""
        if epi is None:
            return
        if tiles is not None:
            ops.lora_expand_tiles(epi.v[: y.shape[0]], tiles.table, tiles.num_tiles, tiles.max_rows, epi.arena, epi.slot_base, epi.slot_rank,
                                  epi.unit_off, y, epi.n0, epi.n1)
        else:
            ops.lora_expand(epi.v, epi.tok_slot, epi.arena, epi.slot_base, epi.slot_rank, epi.unit_off, y, epi.n0, epi.n1)

    def apply(self, ops, x: torch.Tensor, y: torch.Tensor, tok_slot: Optional[torch.Tensor], group: str, layer: int,
              tiles: Optional[LoraTiles] = None):
        """y += LoRA_{slot(t)}(x) for the projection group: one shrink and one expand launch."""
        self.expand(ops, self.shrink(ops, x, tok_slot, group, layer, tiles=tiles), y, tiles=tiles)
