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


def uniform_noise(seeds: torch.Tensor, steps: torch.Tensor, vocab: int) -> torch.Tensor:
    """[R, vocab] floats in (0, 1): a 64-bit mix (the finaliser of MurmurHash3) of seed, step and column."""
    idx = torch.arange(vocab, dtype=torch.int64, device=seeds.device)[None, :]
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
