"""Per-row sampling on the device, with no host synchronisation.

The continuous-batching engine reads results one step behind the GPU, so a sampler that pulls logits to the host would stall
the pipeline.  Here the rows that sample are penalised (repetition, frequency, presence), warped (temperature, top-k, top-p,
typical-p) and drawn on the device inside the step; the drawn ids overwrite the greedy ids before the asynchronous copy to the
host is queued.  The penalties need every request's history, which the host only learns a step late, so the history lives on the
device too: one histogram of token counts per request (prompt and generated tokens), bumped at the drawn id inside the step.

The draw is the exponential-noise arg-max the reference uses to avoid a synchronising `multinomial`
(`server/lorax_server/utils/tokens.py:533-544`): argmax_i p_i / e_i with e_i ~ Exp(1).  The noise comes from a counter-based
hash of (request seed, index of the generated token, vocabulary index), so a request's output depends on its seed only, not on
which other requests share the batch or which decode row it sits in.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .chooser import NextTokenParams


def _s64(c: int) -> int:
    """A 64-bit constant as the signed value torch's int64 arithmetic wraps to."""
    return c - (1 << 64) if c >= (1 << 63) else c


_K_SEED, _K_STEP, _K_IDX = _s64(0x9E3779B97F4A7C15), _s64(0xBF58476D1CE4E5B9), _s64(0x94D049BB133111EB)
_M1, _M2 = _s64(0xFF51AFD7ED558CCD), _s64(0xC4CEB9FE1A85EC53)


def _lsr(x: torch.Tensor, s: int) -> torch.Tensor:
    """Logical shift right of int64 (torch's >> is arithmetic)."""
    return (x >> s) & ((1 << (64 - s)) - 1)


def uniform_noise(seeds: torch.Tensor, steps: torch.Tensor, vocab: int, offset: int = 0) -> torch.Tensor:
    """[R, vocab] floats in (0, 1): a 64-bit mix (the finaliser of MurmurHash3) of seed, step and column.  `offset` is the
    vocabulary index of column 0 (a tensor-parallel rank draws the noise of its own shard: the same numbers as the full row)."""
    idx = torch.arange(offset, offset + vocab, dtype=torch.int64, device=seeds.device)[None, :]
    x = seeds[:, None] * _K_SEED + steps[:, None] * _K_STEP + idx * _K_IDX
    x = (x ^ _lsr(x, 33)) * _M1
    x = (x ^ _lsr(x, 33)) * _M2
    x = x ^ _lsr(x, 33)
    return (_lsr(x, 40).to(torch.float32) + 0.5) * (1.0 / (1 << 24))


def warp(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor, typical_p: torch.Tensor) -> torch.Tensor:
    """Vectorised warpers in the reference's order (temperature, top-k, top-p, typical-p; `utils/logits_process.py:110-430`).
    top_k == 0, top_p == 1 and typical_p == 1 switch the respective filter off for a row.  Returns fp32 scores with -inf on
    the filtered entries."""
    x = logits.float() / temperature[:, None].clamp_min(1e-6)
    V = x.shape[1]
    neg = float("-inf")
    # top-k: keep the k best of every row
    k = torch.where(top_k > 0, top_k.clamp(max=V), torch.full_like(top_k, V))
    srt, _ = x.sort(dim=-1, descending=True)
    kth = srt.gather(1, (k - 1).clamp_min(0)[:, None])
    x = torch.where(x < kth, torch.full_like(x, neg), x)
    # top-p: smallest prefix of the sorted distribution whose mass reaches p (the best token always stays)
    srt, order = x.sort(dim=-1, descending=True)
    probs = torch.softmax(srt, -1)
    before = probs.cumsum(-1) - probs
    drop = before >= top_p[:, None]
    drop[:, 0] = False
    x = x.masked_fill(torch.zeros_like(drop).scatter(1, order, drop), neg)
    # typical-p: keep the tokens whose surprise is closest to the entropy until their mass reaches p
    if bool((typical_p < 1.0).any()):
        logp = torch.log_softmax(x, -1)
        p = logp.exp()
        ent = -(torch.where(p > 0, p * logp, torch.zeros_like(p))).sum(-1, keepdim=True)
        dist = torch.where(torch.isfinite(logp), (-logp - ent).abs(), torch.full_like(logp, float("inf")))
        dsrt, dorder = dist.sort(dim=-1)
        mass = p.gather(1, dorder)
        before = mass.cumsum(-1) - mass
        drop = (before >= typical_p[:, None]) & (typical_p[:, None] < 1.0)
        drop[:, 0] = False
        x = x.masked_fill(torch.zeros_like(drop).scatter(1, dorder, drop), neg)
    return x


def penalise(logits: torch.Tensor, counts: torch.Tensor, repetition: torch.Tensor, frequency: torch.Tensor,
             presence: torch.Tensor) -> torch.Tensor:
    """The history penalties in the reference's order (`utils/logits_process.py:181-300`): scores of tokens already seen are
    divided by the repetition penalty (multiplied when negative), then lowered by frequency * count + presence.  `counts` is
    [R, V]: how often each token occurs in the row's prompt and output so far."""
    x = logits.float()
    seen = counts > 0
    r = repetition[:, None]
    x = torch.where(seen, torch.where(x < 0, x * r, x / r), x)
    return x - counts * frequency[:, None] - seen.to(x.dtype) * presence[:, None]


def draw(scores: torch.Tensor, seeds: torch.Tensor, steps: torch.Tensor, sample: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """One token per row from softmax(scores): ids [R] int64 and their log-probabilities under the warped distribution.
    Rows where `sample` is False take the arg-max (greedy requests that only carry penalties)."""
    logp = torch.log_softmax(scores, -1)
    e = -torch.log(uniform_noise(seeds, steps, scores.shape[1]))
    noisy = logp - torch.log(e)
    if sample is not None:
        noisy = torch.where(sample[:, None], noisy, logp)
    ids = noisy.argmax(-1)
    return ids, logp.gather(1, ids[:, None])[:, 0]


def has_penalties(p: NextTokenParams) -> bool:
    return p.repetition_penalty != 1.0 or p.frequency_penalty != 0.0 or p.presence_penalty != 0.0


def needs_device_step(p: NextTokenParams) -> bool:
    """Whether a request's token cannot be the plain arg-max of the logits."""
    return p.do_sample or has_penalties(p)


def supported(p: NextTokenParams) -> bool:
    """What the device sampler covers; watermarking, grammars and alternative tokens need the host-side chooser of the served
    path."""
    return not p.watermark and p.schema is None and p.return_k_alternatives == 0


TP_CANDIDATES = 128     # candidates a tensor-parallel rank contributes per row: bounds the top-k that is exact without the logits


def tp_eligible(p: NextTokenParams) -> bool:
    """Whether a row can be sampled from vocabulary shards by exchanging candidates instead of logits: its filter must be
    decided by the best TP_CANDIDATES tokens of every shard (top-k up to that, with or without top-p inside it), or there is no
    filter at all (temperature only, or a greedy row that only carries penalties)."""
    if not p.do_sample:
        return True
    if p.typical_p < 1.0:
        return False
    if p.top_k and p.top_k > 0:
        return p.top_k <= TP_CANDIDATES
    return p.top_p >= 1.0


class RowSampler:
    """Parameter tensors for a set of rows, rebuilt only when the set changes."""

    def __init__(self, device):
        self.device = device
        self.key = None
        self.rows = self.temperature = self.top_k = self.top_p = self.typical_p = self.seeds = self.sample = None
        self.counts = self.rep = self.freq = self.pres = None
        self._owners: List[Tuple[int, object]] = []      # (index in the bound set, key of the histogram in the store)
        self._store = None

    def release(self):
        """Hand the histograms back to the store they came from (as views of the stacked tensor: nothing is copied)."""
        if self.counts is not None and self._store is not None:
            for i, k in self._owners:
                if k in self._store:
                    self._store[k] = self.counts[i]
        self.counts, self._owners, self._store, self.key = None, [], None, None

    def bind(self, rows: Sequence[int], params: Sequence[NextTokenParams], keys: Optional[Sequence[object]] = None,
             store: Optional[dict] = None):
        """`store[keys[i]]` is the token-count histogram [V] (fp32, on the device) of request i; only requests with penalties
        need one.  While bound, the histograms live stacked in `self.counts` and are bumped by every call."""
        key = (tuple(rows), tuple(id(p) for p in params), tuple(keys) if keys is not None else None)
        if key == self.key:
            return
        self.release()
        self.key = key
        dev = self.device
        f32 = lambda vals: torch.tensor(list(vals), dtype=torch.float32, device=dev)
        self.rows = torch.tensor(list(rows), dtype=torch.int64, device=dev)
        # greedy requests that only carry penalties pass the warpers untouched
        self.temperature = f32(p.temperature if p.do_sample else 1.0 for p in params)
        self.top_k = torch.tensor([p.top_k if p.do_sample else 0 for p in params], dtype=torch.int64, device=dev)
        self.top_p = f32(p.top_p if p.do_sample else 1.0 for p in params)
        self.typical_p = f32(p.typical_p if p.do_sample else 1.0 for p in params)
        self.seeds = torch.tensor([p.seed or 0 for p in params], dtype=torch.int64, device=dev)
        self.sample = torch.tensor([bool(p.do_sample) for p in params], dtype=torch.bool, device=dev)
        owners = [(i, keys[i]) for i, p in enumerate(params) if has_penalties(p)] if (keys is not None and store is not None) else []
        if owners:
            first = store[owners[0][1]]
            blank = torch.zeros_like(first)
            own = dict(owners)
            self.counts = torch.stack([store[own[i]] if i in own else blank for i in range(len(params))])
            self.rep, self.freq, self.pres = (f32(getattr(p, n) for p in params) for n in
                                              ("repetition_penalty", "frequency_penalty", "presence_penalty"))
            self._owners, self._store = owners, store
            for i, k in owners:
                store[k] = self.counts[i]

    def __call__(self, logits: torch.Tensor, steps: Sequence[int]) -> Tuple[torch.Tensor, torch.Tensor]:
        """logits: all rows of the step; returns (ids, logprobs) for the bound rows."""
        sel = logits.index_select(0, self.rows)
        st = torch.tensor(list(steps), dtype=torch.int64, device=self.device)
        if self.counts is not None:
            sel = penalise(sel[:, : self.counts.shape[1]], self.counts, self.rep, self.freq, self.pres)
        ids, lp = draw(warp(sel, self.temperature, self.top_k, self.top_p, self.typical_p), self.seeds, st, self.sample)
        if self.counts is not None:
            self.counts.scatter_add_(1, ids[:, None], torch.ones_like(ids, dtype=self.counts.dtype)[:, None])
        return ids, lp

    # ------------------------------------------------------------------ vocabulary-parallel sampling
    # The reference gathers the full logits on every rank before it samples (`layers/tensor_parallel.py:50-79`).  Here a rank
    # keeps its vocabulary shard: the ranks exchange their best TP_CANDIDATES scores and the (max, sum of exponentials) of their
    # shard per row, which fixes the cut-off of top-k / top-p and the normaliser exactly; every rank then draws inside its own
    # shard with the noise of its own columns (the noise is a function of seed, step and vocabulary index, so the shards see
    # the numbers the full row would) and the best (noisy score, log-probability, id) triple of all ranks wins.  A few hundred
    # bytes per row cross the links instead of the vocabulary.
    def tp_candidates(self, local_logits: torch.Tensor, v0: int, vocab: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """-> (x [R, Vl]: penalised, temperature-scaled scores of this shard with padding columns at -inf,
               payload [R, K + 2]: the K best of them, their maximum, and sum exp(x - maximum))."""
        sel = local_logits.index_select(0, self.rows).float()
        Vl = sel.shape[1]
        if self.counts is not None:
            sel = penalise(sel, self.counts[:, v0:v0 + Vl] if self.counts.shape[1] >= v0 + Vl else
                           torch.nn.functional.pad(self.counts[:, v0:], (0, v0 + Vl - self.counts.shape[1])), self.rep, self.freq, self.pres)
        x = sel / self.temperature[:, None].clamp_min(1e-6)
        if v0 + Vl > vocab:
            x[:, max(vocab - v0, 0):] = float("-inf")
        k = min(TP_CANDIDATES, Vl)
        top = x.topk(k, dim=-1).values
        if k < TP_CANDIDATES:
            top = torch.nn.functional.pad(top, (0, TP_CANDIDATES - k), value=float("-inf"))
        m = top[:, :1]
        ssum = torch.exp(x - m).sum(-1, keepdim=True)
        return x, torch.cat([top, m, ssum], 1)

    def tp_cutoff(self, payloads: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """payloads [ranks, R, K + 2] -> (tau [R]: scores below it are filtered, logz [R]: log of the sum of exp(score) over the
        tokens that stay)."""
        K = TP_CANDIDATES
        ms, ss = payloads[:, :, K], payloads[:, :, K + 1]
        M = ms.max(0).values
        logz_all = M + torch.log((ss * torch.exp(ms - M[None])).sum(0))
        cand = payloads[:, :, :K].permute(1, 0, 2).reshape(payloads.shape[1], -1).sort(dim=-1, descending=True).values      # [R, ranks * K]
        neg = float("-inf")
        has_k = self.top_k > 0
        kth = cand.gather(1, (self.top_k.clamp(min=1, max=cand.shape[1]) - 1)[:, None])[:, 0]
        kept = cand >= torch.where(has_k, kth, torch.full_like(kth, neg))[:, None]
        c = torch.where(kept, cand, torch.full_like(cand, neg))
        # top-p inside the top-k set (rows without top-k have top_p == 1: nothing to do)
        probs = torch.softmax(c, -1)
        before = probs.cumsum(-1) - probs
        drop = (before >= self.top_p[:, None]) & has_k[:, None]
        drop[:, 0] = False
        c = c.masked_fill(drop, neg)
        last = torch.where(torch.isfinite(c), c, torch.full_like(c, float("inf"))).min(-1).values
        tau = torch.where(has_k, last, torch.full_like(last, neg))
        logz = torch.where(has_k, torch.logsumexp(c, -1), logz_all)
        return tau, logz

    def tp_local_best(self, x: torch.Tensor, tau: torch.Tensor, logz: torch.Tensor, steps: Sequence[int], v0: int) -> torch.Tensor:
        """-> [R, 3]: the best noisy score of this shard, the log-probability of that token, its vocabulary index."""
        st = torch.tensor(list(steps), dtype=torch.int64, device=self.device)
        logp = torch.where(x >= tau[:, None], x - logz[:, None], torch.full_like(x, float("-inf")))
        e = -torch.log(uniform_noise(self.seeds, st, x.shape[1], offset=v0))
        noisy = torch.where(self.sample[:, None], logp - torch.log(e), logp)
        best, idx = noisy.max(-1)
        return torch.stack([best, logp.gather(1, idx[:, None])[:, 0], (idx + v0).to(torch.float32)], 1)

    def tp_finish(self, bests: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """bests [ranks, R, 3] -> (ids, logprobs); the histograms of the penalties are bumped at the drawn ids."""
        win = bests[:, :, 0].argmax(0)                                        # the lowest rank wins a tie, as arg-max over the row would
        pick = bests.gather(0, win[None, :, None].expand(1, -1, 3))[0]
        ids = pick[:, 2].to(torch.int64)
        if self.counts is not None:
            self.counts.scatter_add_(1, ids[:, None].clamp(max=self.counts.shape[1] - 1), torch.ones_like(ids, dtype=self.counts.dtype)[:, None])
        return ids, pick[:, 1]

    def call_tp(self, local_logits: torch.Tensor, steps: Sequence[int], v0: int, vocab: int, all_gather) -> Tuple[torch.Tensor, torch.Tensor]:
        """`all_gather(t)` returns the ranks' tensors stacked along a new first dimension."""
        x, payload = self.tp_candidates(local_logits, v0, vocab)
        tau, logz = self.tp_cutoff(all_gather(payload))
        return self.tp_finish(all_gather(self.tp_local_best(x, tau, logz, steps, v0)))
