"""Model runner: turns scheduler decisions into device work.

Design points that differ from the reference runtime (`server/lorax_server/models/flash_causal_lm.py`):

* Decode state is device resident and row-stable.  Every running request owns a row of a few static tensors
  (input id, position, context length, KV slot, block-table row, adapter slot).  A step needs no host to device
  traffic unless a request joins or leaves: a tiny kernel advances positions / slots from the block tables
  (`advance_decode`).  The reference rebuilds index tensors on the host and syncs three `.tolist()` per step
  (`flash_causal_lm.py:1617-1626, 1813-1816`).
* The whole decode step (embedding .. lm_head .. greedy argmax .. advance) is one CUDA graph per padded batch
  size.  Adapter identity and rank are data (slot ids), not graph structure, so one graph serves any adapter
  mix; the reference needs a graph per (batch, rank) and falls back to eager on mixed ranks
  (`utils/graph.py:478-498`).
* Results come back through pinned host buffers with an event, so the host can run one step behind the GPU.
"""

from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..adapters.manager import LoraTiles
from ..models.decoder import DecoderModel, StepInputs
from ..ops import reference
from .kv_cache import KVCache

GRAPH_BUCKETS = [1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 160, 192, 224, 256, 320, 384, 448, 512]


@dataclass
class PrefillItem:
    """One sequence (or chunk of one) in a prefill step."""
    token_ids: Sequence[int]        # tokens of this chunk
    cache_len: int                  # tokens already in the KV cache (prefix hit or earlier chunks)
    blocks: Sequence[int]           # block table of the sequence
    adapter_index: int = 0
    want_logits: bool = True        # False for a non-final chunk
    all_logprobs: bool = False      # prefill token log-probs requested (decoder_input_details)
    # vision-language prompts: rows `embed_index` (positions within token_ids) take `embeds` [len(embed_index), hidden] instead
    # of the embedding of their (placeholder) token id
    embed_index: Optional[Sequence[int]] = None
    embeds: Optional[torch.Tensor] = None


class DecodeState:
    def __init__(self, max_batch: int, max_blocks: int, device):
        i32 = dict(dtype=torch.int32, device=device)
        self.max_batch, self.max_blocks = max_batch, max_blocks
        self.input_ids = torch.zeros(max_batch, **i32)
        self.positions = torch.zeros(max_batch, **i32)
        self.ctx_lens = torch.zeros(max_batch, **i32)
        self.slots = torch.full((max_batch,), -1, **i32)
        self.block_tables = torch.zeros(max_batch, max_blocks, **i32)
        self.tok_slot = torch.full((max_batch,), -1, **i32)
        self.next_ids = torch.zeros(max_batch, **i32)
        self.logprobs = torch.zeros(max_batch, dtype=torch.float32, device=device)
        # LoRA tile table of the decode batch (rows are kept sorted by adapter slot): [max_batch, 4], unused = slot -1
        self.lora_tiles = torch.full((max_batch, 4), -1, **i32)
        self.row_slot: Dict[int, int] = {}      # row -> adapter slot (host mirror)
        self.num_lora_tiles = 0
        self.tile_list: List[Tuple[int, int, int, int]] = []      # host copy of the live part of lora_tiles
        self.free_rows = list(range(max_batch - 1, -1, -1))
        self.live: Dict[int, int] = {}          # row -> request id
        self.high_water = 0

    def take_row(self, request_id: int) -> int:
        self.free_rows.sort(reverse=True)
        r = self.free_rows.pop()
        self.live[r] = request_id
        self.high_water = max(self.live) + 1
        return r

    def drop_row(self, row: int):
        self.live.pop(row, None)
        self.row_slot.pop(row, None)
        self.free_rows.append(row)
        self.high_water = (max(self.live) + 1) if self.live else 0


class ModelRunner:
    def __init__(self, model: DecoderModel, kv: KVCache, max_batch: int = 256, max_seq_tokens: int = 4096,
                 max_prefill_tokens: int = 4096, use_graphs: bool = True):
        self.model = model
        self.kv = kv
        self.device = model.device
        self.is_cuda = self.device.type == "cuda"
        self.page = kv.page
        self.max_blocks = (max_seq_tokens + self.page - 1) // self.page + 1
        self.max_batch = max_batch
        self.max_prefill_tokens = max_prefill_tokens
        self.state = DecodeState(max_batch, self.max_blocks, self.device)
        self.use_graphs = use_graphs and self.is_cuda
        self.graphs: Dict[Tuple[int, bool], object] = {}
        self.graph_pool = None
        self.graph_out: Dict[Tuple[int, bool], torch.Tensor] = {}
        self.buckets = [b for b in GRAPH_BUCKETS if b <= max_batch]
        if self.buckets[-1] != max_batch:
            self.buckets.append(max_batch)
        # pinned result ring (two steps in flight at most)
        self.n_ring = 8
        pin = dict(pin_memory=True) if self.is_cuda else {}
        self.ring_ids = [torch.zeros(max_batch, dtype=torch.int32, **pin) for _ in range(self.n_ring)]
        self.ring_lp = [torch.zeros(max_batch, dtype=torch.float32, **pin) for _ in range(self.n_ring)]
        # the ring events carry device timestamps: a token's time is the completion of its step on the GPU, on the
        # host's clock through an anchor pair (event, perf_counter) taken at a synchronised moment
        self.ring_ev = [torch.cuda.Event(enable_timing=True) if self.is_cuda else None for _ in range(self.n_ring)]
        self.anchor_ev = None
        self.anchor_host = time.perf_counter()
        if self.is_cuda:
            torch.cuda.synchronize(self.device)
            self.anchor_ev = torch.cuda.Event(enable_timing=True)
            self.anchor_ev.record()
            self.anchor_ev.synchronize()
            self.anchor_host = time.perf_counter()
        # the kernels' status word rides in every ring entry: a device-side wait that ran out is seen when the step's result is read
        self.ring_status = [torch.zeros(2, dtype=torch.int32, **pin) for _ in range(self.n_ring)]
        self.status_word = None
        if self.is_cuda:
            from ..ops import native
            self.status_word = native.workspace(self.device).status
        self.device_failed = None          # message of the first device-side failure (the shard reports unhealthy from then on)
        self.ring_pos = 0
        self.steps = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.graph_kernels: Dict[Tuple[int, bool], int] = {}
        self.tiles_valid = False
        self.replayed_launches = 0

    def kernel_launches(self) -> int:
        """Kernels of this library launched so far: eager launches plus the kernels inside every graph replay."""
        eager = 0
        if self.is_cuda:
            from ..ops import native
            eager = native.launch_count
        return eager + self.replayed_launches

    # ------------------------------------------------------------------ helpers
    def _to_dev(self, values, dtype=torch.int32) -> torch.Tensor:
        t = torch.tensor(values, dtype=dtype)
        if self.is_cuda:
            t = t.pin_memory().to(self.device, non_blocking=True)
        self.h2d_bytes += t.numel() * t.element_size()
        return t

    def _slot_of(self, adapter_index: int) -> int:
        ad = self.model.adapters
        if ad is None or adapter_index == 0:
            return -1
        return ad.slot_of(adapter_index)

    def _table_row(self, blocks: Sequence[int]) -> List[int]:
        n = len(blocks)
        if n >= self.max_blocks:
            return list(blocks[: self.max_blocks])
        window = self.model.config.sliding_window
        if window and n * self.page < self.max_blocks * self.page and n > 0 and n * self.page >= window + self.page:
            # sliding window: pages are recycled cyclically, so the table repeats
            return [blocks[i % n] for i in range(self.max_blocks)]
        return list(blocks) + [0] * (self.max_blocks - n)

    # ------------------------------------------------------------------ prefill
    def _prefill_inputs(self, items: Sequence[PrefillItem], row_offset: int = 0, lead_tiles: Sequence[Tuple[int, int, int, int]] = ()):
        """Assembly of a ragged prefill.  The host packs what it alone knows (token ids, per-sequence lengths, block tables, the
        rows that want logits, the LoRA tile table) into one pinned buffer and one H2D transfer; the per-token positions, cache
        slots and adapter slots are computed from the per-sequence arrays on the device (`ops.prefill_metadata`).  Returns the
        StepInputs and whether any prefill row has an adapter.  In the LoRA tile table the prefill rows are numbered from
        `row_offset` and `lead_tiles` (tiles of rows that precede them in a mixed step) come first."""
        import numpy as np
        page = self.page
        id_parts: List = []
        cu = [0]
        cache_lens, tables, head_idx, head_slot, q_lens, seq_slot = [], [], [], [], [], []
        tl: List[Tuple[int, int, int, int]] = list(lead_tiles)
        any_lora = False
        over_rows: List[int] = []
        over_vals: List[torch.Tensor] = []
        for it in items:
            n = len(it.token_ids)
            if it.embeds is not None and len(it.embed_index or ()):
                over_rows += [cu[-1] + int(i) for i in it.embed_index]
                over_vals.append(it.embeds)
            slot_id = self._slot_of(it.adapter_index)
            any_lora |= slot_id >= 0
            id_parts.append(np.asarray(it.token_ids, dtype=np.int32))
            base = cu[-1]
            cu.append(base + n)
            cache_lens.append(it.cache_len)
            tables.append(self._table_row(it.blocks))
            q_lens.append(n)
            seq_slot.append(slot_id)
            if slot_id >= 0:
                # rows of one adapter in tiles of at most 32 (a run that continues the previous sequence's adapter starts a new tile)
                tl += [(slot_id, base + a + row_offset, min(32, n - a), 0) for a in range(0, n, 32)]
            if it.want_logits:
                if it.all_logprobs:
                    head_idx += list(range(base, base + n))
                    head_slot += [slot_id] * n
                else:
                    head_idx.append(base + n - 1)
                    head_slot.append(slot_id)
        T = cu[-1]
        if T > self.max_prefill_tokens:
            raise ValueError(f"prefill of {T} tokens exceeds max_prefill_tokens={self.max_prefill_tokens}")
        ts, tq = reference.prefill_tiles(q_lens)
        if not any_lora:
            tl = list(lead_tiles)
        i32 = lambda v: np.asarray(v, dtype=np.int32).reshape(-1)
        segs = [np.concatenate(id_parts) if id_parts else i32([]), i32(cu), i32(cache_lens), i32(seq_slot), i32(ts), i32(tq), i32(head_idx),
                i32(head_slot), i32(tl), i32(tables)]
        flat = torch.from_numpy(np.concatenate(segs))
        if self.is_cuda:
            flat = flat.pin_memory().to(self.device, non_blocking=True)
        self.h2d_bytes += flat.numel() * 4
        views, o = [], 0
        for sgm in segs:
            views.append(flat[o:o + sgm.shape[0]])
            o += sgm.shape[0]
        d_ids, d_cu, d_cl, d_seqslot, d_ts, d_tq, d_head, d_headslot, d_tiles, d_bt = views
        bt = d_bt.view(len(items), self.max_blocks)
        d_pos, d_slots, d_tokslot = self.model.ops.prefill_metadata(d_cu, d_cl, d_seqslot, bt, page, T)
        if any_lora and self.model.adapters is not None:
            self.model.adapters.fence()
        tiles = LoraTiles(d_tiles.view(-1, 4), len(tl), 32) if tl else None
        inp = StepInputs(input_ids=d_ids, positions=d_pos, slots=d_slots, is_prefill=True, block_tables=bt, cu_q=d_cu,
                         cache_lens=d_cl, tile_seq=d_ts, tile_q0=d_tq, lm_head_indices=d_head if len(head_idx) else d_ids[:0],
                         tok_slot=d_tokslot if any_lora else None, head_tok_slot=d_headslot if any_lora else None,
                         lora_tiles=tiles)
        if over_rows:
            inp.embed_rows = torch.tensor(over_rows, dtype=torch.long, device=self.model.device)
            inp.embed_values = torch.cat(over_vals, 0).to(self.model.dtype).to(self.model.device)
        return inp, any_lora

    def prefill(self, items: Sequence[PrefillItem]):
        """Run one ragged prefill step.  Returns (next_ids, logprobs, logits) for the rows that wanted logits:
        device tensors; `logits` is None unless some item asked for sampling on the host."""
        inp, _ = self._prefill_inputs(items)
        logits = self.model.forward(inp, self.kv.layers)
        if logits.shape[0] == 0:
            return None, None, logits
        next_ids, lps = self.model.ops.argmax_logprob(logits, softcap=self.model.config.final_logit_softcapping or 0.0)
        return next_ids, lps, self._cap(logits)

    def _cap(self, logits):
        """Logits as a sampler must see them: gemma2 squashes the head's output with cap * tanh(x / cap).  The greedy
        arg-max applies the cap inside its own kernel; rows handed to a sampler or scored as log-probs get it here."""
        cap = self.model.config.final_logit_softcapping or 0.0
        if logits is None or cap <= 0:
            return logits
        return torch.tanh(logits.float() / cap).mul_(cap).to(logits.dtype)

    def can_mix(self) -> bool:
        """A prefill can ride along with the decode rows when those are grouped by adapter (or no adapter is in use)."""
        ad = self.model.adapters
        lora = ad is not None and ad.max_rank > 0
        return self.state.high_water > 0 and (self.tiles_valid or not lora)

    def mixed_step(self, items: Sequence[PrefillItem]):
        """One forward pass over the decode rows [0, high_water) AND the tokens of a ragged prefill: the weights, the
        adapters and every elementwise kernel are paid once for both.  Returns (ring index, decode rows, first ids,
        first log-probs); the decode results land in the pinned ring entry, the prefill's first tokens stay on the
        device for `install`."""
        st = self.state
        nd = st.high_water
        ad = self.model.adapters
        lora = ad is not None and ad.max_rank > 0
        # decode tiles as of the last resort(), clipped to the rows that still exist (rows above them have finished)
        lead = [(sl, r0, min(nr, nd - r0), 0) for (sl, r0, nr, _) in st.tile_list if r0 < nd] if lora else []
        pin, any_lora = self._prefill_inputs(items, row_offset=nd, lead_tiles=lead)
        if lora:
            ad.fence()
        dev = self.device
        cat = torch.cat
        tok_slot = head_slot = tiles = None
        if lora:
            none = torch.full((pin.input_ids.shape[0],), -1, dtype=torch.int32, device=dev)
            p_tok = pin.tok_slot if pin.tok_slot is not None else none
            p_head = pin.head_tok_slot if pin.head_tok_slot is not None else none[: pin.lm_head_indices.shape[0]]
            tok_slot = cat([st.tok_slot[:nd], p_tok])
            head_slot = cat([st.tok_slot[:nd], p_head])
            tiles = pin.lora_tiles
        nsplit = 1
        if self.is_cuda and nd * self.model.nkv < 96:
            nsplit = max(1, min(8, 192 // max(nd * self.model.nkv, 1)))
        head = cat([torch.arange(nd, dtype=torch.int32, device=dev), pin.lm_head_indices + nd])
        inp = StepInputs(input_ids=cat([st.input_ids[:nd], pin.input_ids]), positions=cat([st.positions[:nd], pin.positions]),
                         slots=cat([st.slots[:nd], pin.slots]), is_prefill=True, block_tables=pin.block_tables, cu_q=pin.cu_q,
                         cache_lens=pin.cache_lens, tile_seq=pin.tile_seq, tile_q0=pin.tile_q0, lm_head_indices=head,
                         tok_slot=tok_slot, head_tok_slot=head_slot, lora_tiles=tiles, attn_nsplit=nsplit, n_decode=nd,
                         dec_block_tables=st.block_tables[:nd], ctx_lens=st.ctx_lens[:nd], embed_rows=pin.embed_rows,
                         embed_values=pin.embed_values)
        logits = self.model.forward(inp, self.kv.layers)
        ids, lps = self.model.ops.argmax_logprob(logits, softcap=self.model.config.final_logit_softcapping or 0.0)
        st.next_ids[:nd].copy_(ids[:nd])
        st.logprobs[:nd].copy_(lps[:nd])
        self._advance(nd)
        k = self.stash(st.next_ids[:nd], st.logprobs[:nd])
        self.steps += 1
        return k, nd, ids[nd:], lps[nd:]

    # ------------------------------------------------------------------ decode rows
    def install(self, rows: Sequence[int], first_tokens, positions: Sequence[int], blocks: Sequence[Sequence[int]],
                adapter_indices: Sequence[int]):
        """Write freshly prefilled sequences into their decode rows (one packed H2D + six scatters).  `first_tokens` is a
        host list or the device tensor the prefill's argmax left behind (the host then never waits for the prefill)."""
        if not rows:
            return
        dev_first = first_tokens if isinstance(first_tokens, torch.Tensor) else None
        if dev_first is not None:
            first_tokens = [0] * len(rows)
        page = self.page
        st = self.state
        tabs = [self._table_row(b) for b in blocks]
        slots = [tabs[i][positions[i] // page] * page + positions[i] % page for i in range(len(rows))]
        ctx = [p + 1 for p in positions]
        tslot = [self._slot_of(a) for a in adapter_indices]
        n = len(rows)
        flat = list(rows) + list(first_tokens) + list(positions) + ctx + slots + tslot + [x for t in tabs for x in t]
        dev = self._to_dev(flat)
        r = dev[:n].long()
        st.input_ids.index_copy_(0, r, dev[n:2 * n] if dev_first is None else dev_first.to(torch.int32))
        st.positions.index_copy_(0, r, dev[2 * n:3 * n])
        st.ctx_lens.index_copy_(0, r, dev[3 * n:4 * n])
        st.slots.index_copy_(0, r, dev[4 * n:5 * n])
        st.tok_slot.index_copy_(0, r, dev[5 * n:6 * n])
        st.block_tables.index_copy_(0, r, dev[6 * n:].view(n, self.max_blocks))
        for row, sl in zip(rows, tslot):
            st.row_slot[row] = sl
        self.tiles_valid = False        # rows are no longer grouped by adapter until resort() runs

    def resort(self) -> Dict[int, int]:
        """Compact the live rows to [0, n) ordered by adapter slot, so that rows of one adapter are adjacent and the
        LoRA kernels can work on (slot, first row, rows) tiles.  Device state is permuted with a handful of gathers;
        the returned dict maps old row -> new row for the caller's bookkeeping."""
        st = self.state
        old_rows = sorted(st.live.keys(), key=lambda r: (st.row_slot.get(r, -1), r))
        n = len(old_rows)
        mapping = {old: new for new, old in enumerate(old_rows)}
        if n and any(o != nw for o, nw in mapping.items()):
            perm = self._to_dev(old_rows).long()
            for t in (st.input_ids, st.positions, st.ctx_lens, st.slots, st.tok_slot, st.block_tables):
                t[:n] = t.index_select(0, perm)
        hw = st.high_water
        if hw > n:
            st.ctx_lens[n:hw] = 0
            st.slots[n:hw] = -1
            st.tok_slot[n:hw] = -1
        st.live = {mapping[o]: rid for o, rid in st.live.items()}
        st.row_slot = {mapping[o]: sl for o, sl in st.row_slot.items() if o in mapping}
        st.free_rows = list(range(st.max_batch - 1, n - 1, -1))
        st.high_water = n
        # tile table: decode tiles hold at most 32 rows
        tl = reference.build_lora_tiles([st.row_slot.get(r, -1) for r in range(n)], 32)
        st.num_lora_tiles = len(tl)
        st.tile_list = tl
        flat = [x for t in tl for x in t] + [-1, 0, 0, 0] * (st.max_batch - len(tl))
        st.lora_tiles.copy_(self._to_dev(flat).view(-1, 4))
        self.tiles_valid = True
        return mapping

    def reposition(self, rows: Sequence[int], tokens: Sequence[int], positions: Sequence[int], blocks: Sequence[Sequence[int]]):
        """Point decode rows at new (input token, position) pairs without touching their order, adapters or block tables:
        used after a speculative step accepted several tokens of a row at once."""
        if not rows:
            return
        page = self.page
        tabs = [self._table_row(b) for b in blocks]
        slots = [tabs[i][positions[i] // page] * page + positions[i] % page for i in range(len(rows))]
        n = len(rows)
        dev = self._to_dev(list(rows) + list(tokens) + list(positions) + [p + 1 for p in positions] + slots)
        r = dev[:n].long()
        st = self.state
        st.input_ids.index_copy_(0, r, dev[n:2 * n])
        st.positions.index_copy_(0, r, dev[2 * n:3 * n])
        st.ctx_lens.index_copy_(0, r, dev[3 * n:4 * n])
        st.slots.index_copy_(0, r, dev[4 * n:5 * n])

    def retire(self, rows: Sequence[int]):
        """Mark rows as padding: they stop advancing and attention skips them."""
        if not rows:
            return
        r = self._to_dev(list(rows)).long()
        self.state.ctx_lens.index_fill_(0, r, 0)
        self.state.slots.index_fill_(0, r, -1)
        self.state.tok_slot.index_fill_(0, r, -1)

    def rebind_adapter_slots(self, rows: Sequence[int], adapter_indices: Sequence[int]):
        if rows:
            r = self._to_dev(list(rows)).long()
            self.state.tok_slot.index_copy_(0, r, self._to_dev([self._slot_of(a) for a in adapter_indices]))

    # ------------------------------------------------------------------ decode
    def _bucket(self, n: int) -> int:
        for b in self.buckets:
            if b >= n:
                return b
        return self.buckets[-1]

    def _decode_body(self, b: int, lora: bool, need_logits: bool = False):
        st = self.state
        nsplit = 1
        if self.is_cuda and b * self.model.nkv < 96:
            nsplit = max(1, min(8, 192 // max(b * self.model.nkv, 1)))
        # the table always has max_batch rows; a graph launches one CTA per possible tile of the bucket (unused: slot -1)
        tiles = LoraTiles(st.lora_tiles, b, 32, live=st.num_lora_tiles) if (lora and self.tiles_valid) else None
        fused = self.model.tp.fused if self.model.tp.world_size > 1 else None
        fused_head = (fused is not None and not need_logits and b <= fused.max_rows
                      and not (self.model.config.final_logit_softcapping or 0.0))
        inp = StepInputs(input_ids=st.input_ids[:b], positions=st.positions[:b], slots=st.slots[:b], is_prefill=False,
                         block_tables=st.block_tables[:b], ctx_lens=st.ctx_lens[:b], tok_slot=st.tok_slot[:b] if lora else None,
                         head_tok_slot=st.tok_slot[:b] if lora else None, attn_nsplit=nsplit, lora_tiles=tiles, local_logits=fused_head)
        logits = self.model.forward(inp, self.kv.layers)
        if fused_head:
            # vocabulary-parallel greedy head: 16 bytes per row and rank cross NVLink instead of the logits
            fused.argmax_tp(logits, self.model.vocab_start, st.next_ids[:b], st.logprobs[:b])
        else:
            self.model.ops.argmax_logprob(logits, st.next_ids[:b], st.logprobs[:b], softcap=self.model.config.final_logit_softcapping or 0.0)
        return logits

    def _advance(self, b: int):
        st = self.state
        self.model.ops.advance_decode(st.input_ids[:b], st.next_ids[:b], st.positions[:b], st.ctx_lens[:b], st.slots[:b],
                                      st.block_tables[:b], self.page)

    def _ks_class(self, lora: bool) -> int:
        """The LoRA shrink's K split is baked into a captured graph; it depends on how many tiles are live."""
        if not (lora and self.tiles_valid):
            return 0
        return min(8, (2 * 148) // max(1, self.state.num_lora_tiles))

    def capture(self, b: int, lora: bool, need_logits: bool = False):
        key = (b, lora, self.tiles_valid, need_logits, self._ks_class(lora))
        if key in self.graphs:
            return
        # warm up outside capture (lazy cudaFuncSetAttribute calls, workspace allocation)
        saved = [t.clone() for t in (self.state.input_ids, self.state.positions, self.state.ctx_lens, self.state.slots)]
        self._decode_body(b, lora, need_logits)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        from ..ops import native
        before = native.launch_count
        with torch.cuda.graph(g, pool=self.graph_pool, capture_error_mode="thread_local"):      # other threads (NCCL watchdog, RPC handlers) may touch CUDA meanwhile
            logits = self._decode_body(b, lora, need_logits)
            self._advance(b)
        self.graph_kernels[key] = native.launch_count - before
        native.launch_count = before          # captured, not executed
        if self.graph_pool is None:
            self.graph_pool = g.pool()
        for t, s in zip((self.state.input_ids, self.state.positions, self.state.ctx_lens, self.state.slots), saved):
            t.copy_(s)
        self.graphs[key] = g
        self.graph_out[key] = logits

    def decode(self, lora: Optional[bool] = None, need_logits: bool = False, sampler=None, sampler_takes_shards: bool = False):
        """One decode step over rows [0, high_water).  Returns (ring index, bucket, logits or None); the sampled
        ids / log-probs land in the pinned ring entry once its event has completed.  `sampler(logits, state)` runs on the
        device right after the step and may overwrite `next_ids`, `logprobs` and the next `input_ids` of some rows (the
        step itself has already advanced the state with the arg-max)."""
        st = self.state
        # a sampler that draws from vocabulary shards (candidates exchanged, not logits) runs on the graph whose head stays local
        shards = (sampler is not None and sampler_takes_shards and not need_logits and self.model.tp.world_size > 1
                  and self.model.tp.fused is not None and not (self.model.config.final_logit_softcapping or 0.0))
        need_logits = need_logits or (sampler is not None and not shards)
        n = st.high_water
        if n == 0:
            return None
        b = self._bucket(n)
        ad = self.model.adapters
        if lora is None:
            lora = ad is not None and ad.max_rank > 0
        if lora:
            ad.fence()
        logits = None
        if self.use_graphs:
            variant = need_logits and self.model.tp.world_size > 1      # only TP has two head variants
            key = (b, lora, self.tiles_valid, variant, self._ks_class(lora))
            self.capture(b, lora, variant)
            self.graphs[key].replay()
            self.replayed_launches += self.graph_kernels[key]
            logits = self.graph_out[key] if (need_logits or shards) else None
        else:
            logits = self._decode_body(b, lora, need_logits)
            self._advance(b)
        logits = self._cap(logits)
        if sampler is not None:
            sampler(logits, st)
        k = self.ring_pos
        self.ring_pos = (k + 1) % self.n_ring
        self.ring_ids[k][:b].copy_(st.next_ids[:b], non_blocking=True)
        self.ring_lp[k][:b].copy_(st.logprobs[:b], non_blocking=True)
        self.d2h_bytes += b * 8
        if self.is_cuda:
            self.ring_status[k].copy_(self.status_word, non_blocking=True)
            self.d2h_bytes += 8
            self.ring_ev[k].record()
        self.steps += 1
        return k, b, logits

    def stash(self, ids: torch.Tensor, lps: torch.Tensor) -> int:
        """Queue an asynchronous copy of `ids` / `lps` (device) into a pinned ring entry; `wait(k)` returns them."""
        k = self.ring_pos
        self.ring_pos = (k + 1) % self.n_ring
        n = ids.shape[0]
        self.ring_ids[k][:n].copy_(ids, non_blocking=True)
        self.ring_lp[k][:n].copy_(lps, non_blocking=True)
        self.d2h_bytes += n * 8
        if self.is_cuda:
            self.ring_status[k].copy_(self.status_word, non_blocking=True)
            self.d2h_bytes += 8
            self.ring_ev[k].record()
        return k

    def wait(self, k: int):
        """Results of ring entry `k`.  Raises when a kernel of the step (or an earlier one) gave up on a bounded wait: a peer GPU
        that stopped answering, a pipeline that never filled.  The status word is cleared so that the next batch starts clean."""
        if self.is_cuda:
            self.ring_ev[k].synchronize()
            code, detail = int(self.ring_status[k][0]), int(self.ring_status[k][1])
            if code != 0:
                from ..ops import native
                self.status_word.zero_()
                for st in self.ring_status:
                    st.zero_()
                self.device_failed = f"device status {code} ({native.STATUS_NAMES.get(code, '?')}), detail {detail}"
                raise native.NativeError(self.device_failed)
        return self.ring_ids[k], self.ring_lp[k]

    def ring_time(self, k: int) -> float:
        """When ring entry `k` (already waited for) completed on the device, in seconds on the host's perf_counter clock."""
        if not self.is_cuda:
            return time.perf_counter()
        return self.anchor_host + self.anchor_ev.elapsed_time(self.ring_ev[k]) * 1e-3
