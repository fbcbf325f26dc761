"""In-process serving engine: continuous heterogeneous batching over one model shard group.

It plays the roles that the reference splits between the router's batching task
(`router/src/infer.rs:1051-1248`), the adapter scheduler (`router/src/scheduler.rs:283-546`) and the shard's
`generate_token` loop, for users who embed the library (and for `bench.py`).  The C++ router drives the same
:class:`ModelRunner` through the gRPC servicer when the full server stack is used.

Scheduling rules kept from the reference: new prefills interrupt decoding only when enough requests wait
(`waiting_served_ratio`) or the oldest has waited `max_waiting_tokens` decode steps; a prefill step is bounded
by `max_batch_prefill_tokens`; the running batch by `max_batch_total_tokens` (KV blocks); requests of adapters
that are not resident wait for the exchange engine; adapters idle while others wait are evicted first.
The host runs one decode step behind the GPU (results arrive through a pinned ring), and rows that end by
length are retired without waiting for their last token.
"""

from __future__ import annotations

import collections
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence, Tuple

import torch

from ..config import EngineConfig
from ..models.decoder import DecoderModel
from ..sampling.chooser import (FINISH_EOS, FINISH_LENGTH, FINISH_STOP, HeterogeneousNextTokenChooser, NextTokenParams,
                                StoppingCriteria)
from ..sampling.device import RowSampler, has_penalties, needs_device_step, tp_eligible
from ..sampling.device import supported as device_sampling_supported
from .kv_cache import BlockAllocator, KVCache
from .runner import ModelRunner, PrefillItem


@dataclass
class GenRequest:
    request_id: int
    prompt_ids: List[int]
    max_new_tokens: int = 20
    adapter_index: int = 0               # 0 = base model
    params: NextTokenParams = field(default_factory=NextTokenParams)
    eos_token_ids: frozenset = frozenset()
    ignore_eos_token: bool = False
    stop_sequences: List[str] = field(default_factory=list)
    arrival_time: float = 0.0


@dataclass
class TokenEvent:
    request_id: int
    token_id: int
    logprob: float
    index: int                           # 0-based index of the generated token
    finished: bool
    finish_reason: Optional[int] = None
    time: float = 0.0                    # host clock when the host read the token
    device_time: float = 0.0             # when the step that produced it completed on the device (same clock)


@dataclass
class _Seq:
    req: GenRequest
    blocks: List[int]
    row: int = -1
    output_ids: List[int] = field(default_factory=list)
    launched: int = 0                    # tokens whose computation has been launched (incl. the prefill token)
    finished: bool = False
    retired: bool = False
    first_token_time: float = 0.0
    last_token_time: float = 0.0
    stopping: Optional[StoppingCriteria] = None


class Engine:
    def __init__(self, model: DecoderModel, cfg: Optional[EngineConfig] = None, num_blocks: Optional[int] = None,
                 max_batch: int = 256, decode_text: Optional[Callable[[int], str]] = None, use_graphs: Optional[bool] = None):
        self.model = model
        self.cfg = cfg or EngineConfig()
        c = model.config
        page = self.cfg.block_size
        self._max_batch = max_batch
        if num_blocks is None:
            num_blocks = self._auto_blocks(page)
        from .kv_cache import kv_dtype_of
        self.kv = KVCache(c.num_hidden_layers, num_blocks, model.nkv, model.d, kv_dtype_of(model, self.cfg), model.device, page)
        self.alloc = BlockAllocator(num_blocks, page, c.sliding_window)
        self.runner = ModelRunner(model, self.kv, max_batch=max_batch, max_seq_tokens=self.cfg.max_total_tokens,
                                  max_prefill_tokens=self.cfg.max_batch_prefill_tokens,
                                  use_graphs=self.cfg.compile if use_graphs is None else use_graphs)
        self.waiting: Deque[GenRequest] = collections.deque()
        self.running: Dict[int, _Seq] = {}
        self.draining: Dict[int, _Seq] = {}
        self._row_sampler = RowSampler(model.device)
        self._hist: Dict[int, torch.Tensor] = {}     # request id -> token-count histogram on the device (requests with penalties)
        self.inflight: Deque[tuple] = collections.deque()   # ("decode", ring idx, bucket, row->req) | ("first", ring idx, n, [req])
        self.steps_since_prefill = 0
        self.decode_text = decode_text
        self.stats = dict(prefill_steps=0, decode_steps=0, prefill_tokens=0, generated_tokens=0)
        self.finished: Dict[int, _Seq] = {}
        self.on_adapter_needed: Optional[Callable[[int], bool]] = None     # exchange hook: make adapter resident
        # built-in exchange policy: adapters registered here are brought into HBM on demand; when the arena is full the
        # least recently used adapter that no running request needs goes back to the pinned host tier
        self.adapter_keys: Dict[int, str] = {}
        self.adapter_lru: "collections.OrderedDict[int, None]" = collections.OrderedDict()
        self._picking: set = set()
        self.mixed_steps = os.environ.get("LORAX_MIXED_STEPS", "1") != "0"   # prefills ride along with the decode batch

    def _auto_blocks(self, page: int) -> int:
        m, c = self.model, self.model.config
        per_block = KVCache.bytes_per_block(c.num_hidden_layers, m.nkv, m.d, m.dtype, page)
        if m.device.type == "cuda":
            from .kv_cache import plan_kv_blocks
            return plan_kv_blocks(m, self.cfg, self._max_batch, page, reserve_bytes=2 << 30)
        return 512

    # ------------------------------------------------------------------ API
    def add_request(self, req: GenRequest):
        if not req.params.plain and not device_sampling_supported(req.params):
            raise ValueError("the in-process engine samples on the device (penalties, temperature, top-k, top-p, typical-p, seed); "
                             "watermarking, grammars and alternative tokens are served by the shard runtime behind the router")
        if not req.arrival_time:
            req.arrival_time = time.perf_counter()
        if len(req.prompt_ids) + req.max_new_tokens > self.cfg.max_total_tokens:
            raise ValueError("inputs tokens + max_new_tokens must be <= %d" % self.cfg.max_total_tokens)
        self.waiting.append(req)

    @property
    def idle(self) -> bool:
        return not (self.waiting or self.running or self.draining or self.inflight)

    # ------------------------------------------------------------------ scheduling
    def register_adapter(self, adapter_index: int, key: str):
        """Tell the engine which registered adapter (host-tier key) a request's `adapter_index` means, so that it can be
        loaded on demand and offloaded when others need the room."""
        self.adapter_keys[adapter_index] = key

    def _adapter_ready(self, adapter_index: int) -> bool:
        ad = self.model.adapters
        if adapter_index == 0 or ad is None:
            return True
        if ad.is_loaded(adapter_index):
            self.adapter_lru[adapter_index] = None
            self.adapter_lru.move_to_end(adapter_index)
            return True
        if self.on_adapter_needed is not None:
            return bool(self.on_adapter_needed(adapter_index))
        key = self.adapter_keys.get(adapter_index)
        if key is None:
            return False
        in_use = ({s.req.adapter_index for s in self.running.values()} | {s.req.adapter_index for s in self.draining.values()}
                  | self._picking)
        while not ad.load(adapter_index, key):
            victim = next((i for i in self.adapter_lru if i not in in_use and ad.is_loaded(i)), None)
            if victim is None:
                return False                    # everything resident is in use: the request waits
            ad.offload(victim)
            del self.adapter_lru[victim]
            self.stats["adapter_evictions"] = self.stats.get("adapter_evictions", 0) + 1
        self.stats["adapter_loads"] = self.stats.get("adapter_loads", 0) + 1
        self.adapter_lru[adapter_index] = None
        return True

    def _prefetch_adapters(self, lookahead: int = 64, max_loads: int = 2):
        """Bring the adapters of requests that are still queued into HBM ahead of their turn: the copy runs on the exchange
        stream while the batch decodes, so the request does not wait for it when it reaches the head of the queue (the
        reference loads an adapter when its queue becomes active, `router/src/queue.rs:338-451`).  Adapters that neither the
        running batch nor the look-ahead window needs make room, least recently used first."""
        ad = self.model.adapters
        if ad is None or not self.adapter_keys or not self.waiting or self.on_adapter_needed is not None:
            return
        wanted: List[int] = []
        for i, req in enumerate(self.waiting):
            if i >= lookahead:
                break
            a = req.adapter_index
            if a and a not in wanted and a in self.adapter_keys:
                wanted.append(a)
        if all(ad.is_loaded(a) for a in wanted):
            return
        keep = ({s.req.adapter_index for s in self.running.values()} | {s.req.adapter_index for s in self.draining.values()}
                | set(wanted))
        loads = 0
        for a in wanted:
            if loads >= max_loads:
                break
            if ad.is_loaded(a):
                continue
            ok = ad.load(a, self.adapter_keys[a])
            while not ok:
                victim = next((i for i in self.adapter_lru if i not in keep and ad.is_loaded(i)), None)
                if victim is None:
                    return                      # everything resident is needed sooner
                ad.offload(victim)
                del self.adapter_lru[victim]
                self.stats["adapter_evictions"] = self.stats.get("adapter_evictions", 0) + 1
                ok = ad.load(a, self.adapter_keys[a])
            self.adapter_lru[a] = None
            self.stats["adapter_loads"] = self.stats.get("adapter_loads", 0) + 1
            self.stats["adapter_prefetches"] = self.stats.get("adapter_prefetches", 0) + 1
            loads += 1

    def _select_prefill(self) -> List[Tuple[GenRequest, List[int]]]:
        if not self.waiting:
            return []
        free_rows = len(self.runner.state.free_rows)
        if free_rows == 0:
            return []
        n_run = len(self.running)
        if n_run > 0 and self.steps_since_prefill < self.cfg.max_waiting_tokens:
            min_size = int(n_run * self.cfg.waiting_served_ratio)
            # a shrinking batch makes room: admit when the gap to the target batch is worth a prefill step
            if len(self.waiting) < min(min_size, free_rows):
                return []
            # enough requests wait to fill every free row: gather a few rows first, one prefill pass then serves several prompts
            if (free_rows < min(self.cfg.prefill_min_rows, len(self.waiting), self.runner.max_batch)
                    and self.steps_since_prefill < self.cfg.prefill_max_wait_steps):
                return []
        picked: List[Tuple[GenRequest, List[int]]] = []
        self._picking = set()           # adapters of requests admitted in this pass: not eviction candidates
        budget = self.cfg.max_batch_prefill_tokens
        skipped: List[GenRequest] = []
        while self.waiting and len(picked) < free_rows:
            req = self.waiting[0]
            n = len(req.prompt_ids)
            if n > budget:
                if not picked and n > self.cfg.max_batch_prefill_tokens:
                    self.waiting.popleft()
                    raise ValueError(f"prompt of {n} tokens exceeds max_batch_prefill_tokens")
                break
            if not self._adapter_ready(req.adapter_index):
                skipped.append(self.waiting.popleft())
                continue
            blocks = self.alloc.allocate(n + req.max_new_tokens + 1)
            if blocks is None:
                break
            self.waiting.popleft()
            picked.append((req, blocks))
            self._picking.add(req.adapter_index)
            budget -= n
        for r in reversed(skipped):
            self.waiting.appendleft(r)
        return picked

    def _finish(self, seq: _Seq, reason: int):
        seq.finished = True
        if not seq.retired and seq.row >= 0:
            self.runner.retire([seq.row])
        seq.retired = True
        if seq.row >= 0:
            self.runner.state.drop_row(seq.row)
        self.alloc.release(seq.blocks)
        self.running.pop(seq.req.request_id, None)
        self.draining.pop(seq.req.request_id, None)
        self.finished[seq.req.request_id] = seq

    def _emit(self, seq: _Seq, token: int, lp: float, now: float, events: List[TokenEvent], dev_now: float = 0.0):
        if seq.finished:
            return
        idx = len(seq.output_ids)
        seq.output_ids.append(token)
        if idx == 0:
            seq.first_token_time = now
        seq.last_token_time = now
        text = self.decode_text(token) if (self.decode_text and seq.stopping.stop_sequences) else ""
        stop, reason = seq.stopping(token, text)
        events.append(TokenEvent(seq.req.request_id, token, lp, idx, stop, reason, now, dev_now or now))
        self.stats["generated_tokens"] += 1
        if stop:
            self._finish(seq, reason)

    # ------------------------------------------------------------------ one iteration
    def _admit(self, picked, next_ids, lps):
        """Give freshly prefilled requests their decode rows.  The first tokens stay on the device: they are scattered
        into the rows there and reach the host through the pinned ring like every later token, so the host never waits
        for a prefill to finish."""
        rows, sel, poss, blks, ads, rids = [], [], [], [], [], []
        for i, (req, blocks) in enumerate(picked):
            seq = _Seq(req, blocks, stopping=StoppingCriteria(req.max_new_tokens, req.eos_token_ids, list(req.stop_sequences),
                                                              req.ignore_eos_token))
            seq.launched = 1
            rids.append(req.request_id)
            if req.max_new_tokens > 1:
                seq.row = self.runner.state.take_row(req.request_id)
                self.running[req.request_id] = seq
                rows.append(seq.row); sel.append(i); poss.append(len(req.prompt_ids)); blks.append(blocks)
                ads.append(req.adapter_index)
            else:                       # only the prefill token is wanted: no decode row
                seq.retired = True
                self.draining[req.request_id] = seq
        if rows:
            first = next_ids if len(sel) == len(picked) else next_ids[torch.tensor(sel, device=next_ids.device)]
            self.runner.install(rows, first, poss, blks, ads)
        mapping = self.runner.resort()
        for s_ in list(self.running.values()) + list(self.draining.values()):
            if s_.row in mapping:
                s_.row = mapping[s_.row]
        self.inflight.append(("first", self.runner.stash(next_ids, lps), len(picked), rids))
        self.stats["prefill_steps"] += 1
        self.stats["prefill_tokens"] += sum(len(r.prompt_ids) for r, _ in picked)
        self.steps_since_prefill = 0

    def _after_decode_launch(self, k: int, b: int, snapshot: Dict[int, int]):
        self.inflight.append(("decode", k, b, snapshot))
        self.stats["decode_steps"] += 1
        self.steps_since_prefill += 1
        # rows that reach max_new_tokens with this step need no further steps: retire them now
        done_rows = []
        for rid in list(snapshot.values()):
            s = self.running.get(rid)
            if s is None:
                continue
            s.launched += 1
            if s.launched >= s.req.max_new_tokens and not s.retired:
                s.retired = True
                done_rows.append(s.row)
                self.draining[rid] = self.running.pop(rid)
        self.runner.retire(done_rows)

    # ------------------------------------------------------------------ one iteration
    def _sample_first(self, picked, next_ids, lps, logits):
        """Requests that sample draw their first token on the device from the prefill logits (one row per request)."""
        idx = [i for i, (r, _) in enumerate(picked) if needs_device_step(r.params)]
        if not idx:
            return
        V = logits.shape[1]
        for i in idx:                                        # the prompt opens the history of a request with penalties
            r = picked[i][0]
            if has_penalties(r.params):
                prompt = torch.tensor(r.prompt_ids, dtype=torch.int64, device=logits.device).clamp_(0, V - 1)
                self._hist[r.request_id] = torch.bincount(prompt, minlength=V).to(torch.float32)
        sampler = RowSampler(logits.device)
        sampler.bind(idx, [picked[i][0].params for i in idx], [picked[i][0].request_id for i in idx], self._hist)
        ids, lp = sampler(logits, [0] * len(idx))
        sampler.release()
        next_ids.index_copy_(0, sampler.rows, ids.to(next_ids.dtype))
        lps.index_copy_(0, sampler.rows, lp.to(lps.dtype))

    def _decode_sampler(self, snapshot: Dict[int, int]):
        """The device-side hook of a decode step, or None when every running request is greedy."""
        rows = sorted(r for r, rid in snapshot.items() if needs_device_step(self.running[rid].req.params))
        if not rows:
            self._row_sampler.release()
            return None
        seqs = [self.running[snapshot[r]] for r in rows]
        self._row_sampler.bind(rows, [s.req.params for s in seqs], [snapshot[r] for r in rows], self._hist)
        steps = [s.launched for s in seqs]                   # index of the token this step generates for the row
        rs = self._row_sampler

        model = self.model
        tp = model.tp

        def hook(logits, st):
            if tp.world_size > 1 and logits.shape[1] != model.vocab:
                # the head stayed vocabulary-parallel: draw from the shards, exchanging candidates instead of logits
                ids, lp = rs.call_tp(logits, steps, model.vocab_start, model.vocab, tp.all_gather_stack)
            else:
                ids, lp = rs(logits, steps)
            ids32 = ids.to(st.next_ids.dtype)
            st.next_ids.index_copy_(0, rs.rows, ids32)
            st.logprobs.index_copy_(0, rs.rows, lp.to(st.logprobs.dtype))
            st.input_ids.index_copy_(0, rs.rows, ids32)      # the step advanced the state with the arg-max
        hook.takes_shards = tp.world_size > 1 and all(tp_eligible(s.req.params) for s in seqs)
        return hook

    def step(self) -> List[TokenEvent]:
        events: List[TokenEvent] = []
        queued_before = len(self.inflight)
        self._prefetch_adapters()
        picked = self._select_prefill()
        launched = False
        if picked:
            items = [PrefillItem(r.prompt_ids, 0, b, r.adapter_index) for r, b in picked]
            snapshot = {s.row: rid for rid, s in self.running.items() if not s.retired}
            sampling = any(needs_device_step(r.params) for r, _ in picked) or any(needs_device_step(s.req.params) for s in self.running.values())
            if self.mixed_steps and snapshot and self.runner.can_mix() and not sampling:
                # one pass over the weights for the running decode rows and the new prompts together
                k, b, next_ids, lps = self.runner.mixed_step(items)
                self._after_decode_launch(k, b, snapshot)
                self._admit(picked, next_ids, lps)
                launched = True
            else:
                next_ids, lps, logits = self.runner.prefill(items)
                self._sample_first(picked, next_ids, lps, logits)
                self._admit(picked, next_ids, lps)

        if not launched and self.running:
            snapshot = {s.row: rid for rid, s in self.running.items() if not s.retired}
            hook = self._decode_sampler(snapshot) if snapshot else None
            out = self.runner.decode(sampler=hook, sampler_takes_shards=bool(getattr(hook, "takes_shards", False))) if snapshot else None
            if out is not None:
                self._after_decode_launch(out[0], out[1], snapshot)
                launched = True

        # results are read one step behind the GPU: what this step queued stays queued (everything, once idle)
        keep = (len(self.inflight) - queued_before) if launched else 0
        while len(self.inflight) > keep:
            kind, k, b, who = self.inflight.popleft()
            ids_p, lps_p = self.runner.wait(k)
            now = time.perf_counter()
            dev_now = self.runner.ring_time(k)
            ids_h, lps_h = ids_p[:b].tolist(), lps_p[:b].tolist()
            if kind == "first":
                for i, rid in enumerate(who):
                    seq = self.running.get(rid) or self.draining.get(rid)
                    if seq is not None and not seq.finished:
                        self._emit(seq, ids_h[i], lps_h[i], now, events, dev_now)
                continue
            for row, rid in who.items():
                seq = self.running.get(rid) or self.draining.get(rid)
                if seq is None or seq.finished:
                    continue
                self._emit(seq, ids_h[row], lps_h[row], now, events, dev_now)
        if self._hist:                                         # histories of requests that no longer decode
            for rid in [k for k in self._hist if k not in self.running]:
                del self._hist[rid]
            if not self._hist:
                self._row_sampler.release()
        return events

    def run(self, max_steps: Optional[int] = None) -> List[TokenEvent]:
        out: List[TokenEvent] = []
        n = 0
        while not self.idle and (max_steps is None or n < max_steps):
            out += self.step()
            n += 1
        return out

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 20, adapter_indices: Optional[Sequence[int]] = None,
                 params: Optional[Sequence[NextTokenParams]] = None, eos_token_ids: frozenset = frozenset()) -> List[List[int]]:
        base = max(list(self.finished.keys()) + [0]) + 1
        for i, p in enumerate(prompts):
            self.add_request(GenRequest(base + i, list(p), max_new_tokens, adapter_indices[i] if adapter_indices else 0,
                                        params[i] if params else NextTokenParams(), eos_token_ids))
        self.run()
        return [self.finished[base + i].output_ids for i in range(len(prompts))]
