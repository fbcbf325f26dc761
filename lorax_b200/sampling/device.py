"""Per-row sampling on the device, with no host synchronisation.

The continuous-batching engine reads results one step behind the GPU, so a sampler that pulls logits to the host would stall
the pipeline.  Here the rows that sample are warped (temperature, top-k, top-p, typical-p) and drawn on the device inside the
step; the drawn ids overwrite the greedy ids before the asynchronous copy to the host is queued.

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


def draw(scores: torch.Tensor, seeds: torch.Tensor, steps: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """One token per row from softmax(scores): ids [R] int64 and their log-probabilities under the warped distribution."""
    logp = torch.log_softmax(scores, -1)
    e = -torch.log(uniform_noise(seeds, steps, scores.shape[1]))
    ids = (logp - torch.log(e)).argmax(-1)
    return ids, logp.gather(1, ids[:, None])[:, 0]


def supported(p: NextTokenParams) -> bool:
    """What the device sampler covers; penalties over the history, watermarking, grammars and alternative tokens need the
    host-side chooser of the served path."""
    return (p.repetition_penalty == 1.0 and p.frequency_penalty == 0.0 and p.presence_penalty == 0.0 and not p.watermark
            and p.schema is None and p.return_k_alternatives == 0)


class RowSampler:
    """Parameter tensors for a set of rows, rebuilt only when the set changes."""

    def __init__(self, device):
        self.device = device
        self.key = None
        self.rows = self.temperature = self.top_k = self.top_p = self.typical_p = self.seeds = None

    def bind(self, rows: Sequence[int], params: Sequence[NextTokenParams]):
        key = (tuple(rows), tuple(id(p) for p in params))
        if key == self.key:
            return
        self.key = key
        dev = self.device
        self.rows = torch.tensor(list(rows), dtype=torch.int64, device=dev)
        self.temperature = torch.tensor([p.temperature for p in params], dtype=torch.float32, device=dev)
        self.top_k = torch.tensor([p.top_k for p in params], dtype=torch.int64, device=dev)
        self.top_p = torch.tensor([p.top_p for p in params], dtype=torch.float32, device=dev)
        self.typical_p = torch.tensor([p.typical_p for p in params], dtype=torch.float32, device=dev)
        self.seeds = torch.tensor([p.seed for p in params], dtype=torch.int64, device=dev)

    def __call__(self, logits: torch.Tensor, steps: Sequence[int]) -> Tuple[torch.Tensor, torch.Tensor]:
        """logits: all rows of the step; returns (ids, logprobs) for the bound rows."""
        sel = logits.index_select(0, self.rows)
        st = torch.tensor(list(steps), dtype=torch.int64, device=self.device)
        return draw(warp(sel, self.temperature, self.top_k, self.top_p, self.typical_p), self.seeds, st)
