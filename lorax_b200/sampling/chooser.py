"""Next-token selection for a heterogeneous batch: every request carries its own sampling parameters and the
whole batch is processed with vectorised tensor ops (no per-request Python in the logits path).

Behavioural counterpart of `server/lorax_server/utils/tokens.py:230-615` and `utils/logits_process.py:110-430`
in the reference: repetition / frequency / presence penalties, temperature, top-k, top-p, typical-p, optional
watermark and grammar (FSM) masks, sampling with per-request seeded generators through the exponential-noise
argmax trick (`tokens.py:539-544`), log-probabilities of the chosen token, top-k alternatives, and the
speculative verify/accept loop with n-gram (prompt-lookup) proposals.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class NextTokenParams:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    typical_p: float = 1.0
    do_sample: bool = False
    seed: int = 0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    watermark: bool = False
    return_k_alternatives: int = 0
    schema: Optional[str] = None

    @property
    def greedy(self) -> bool:
        return not self.do_sample

    @property
    def plain(self) -> bool:
        """True when the argmax of the raw logits is the answer (the fused greedy kernel can be used)."""
        return (not self.do_sample and self.repetition_penalty == 1.0 and self.frequency_penalty == 0.0
                and self.presence_penalty == 0.0 and not self.watermark and self.schema is None
                and self.return_k_alternatives == 0)


class Watermark:
    """Green-list watermark (Kirchenbauer et al.), gamma / delta as in `utils/watermark.py:26-84`."""

    def __init__(self, gamma: float = 0.5, delta: float = 2.0, hash_key: int = 15485863):
        self.gamma, self.delta, self.hash_key = gamma, delta, hash_key

    def greenlist(self, last_token: int, vocab: int, device) -> torch.Tensor:
        g = torch.Generator(device="cpu").manual_seed(self.hash_key * int(last_token))
        n = int(vocab * self.gamma)
        return torch.randperm(vocab, generator=g)[:n].to(device)

    def __call__(self, last_token: int, scores: torch.Tensor) -> torch.Tensor:
        ids = self.greenlist(last_token, scores.shape[-1], scores.device)
        scores = scores.clone()
        scores[..., ids] += self.delta
        return scores


class HeterogeneousNextTokenChooser:
    def __init__(self, params: Sequence[NextTokenParams], device, vocab_size: int, watermark: Optional[Watermark] = None,
                 grammars: Optional[List[Optional[object]]] = None):
        self.params = list(params)
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.watermark = watermark or Watermark()
        self.grammars = grammars or [None] * len(self.params)
        self.generators: Dict[int, torch.Generator] = {}
        self._build()

    def _build(self):
        p, dev = self.params, self.device
        f = lambda name, dt=torch.float32: torch.tensor([getattr(x, name) for x in p], dtype=dt, device=dev)
        self.temperature = f("temperature").clamp_min(1e-6)
        self.top_k = f("top_k", torch.int64)
        self.top_p = f("top_p")
        self.typical_p = f("typical_p")
        self.rep = f("repetition_penalty")
        self.freq = f("frequency_penalty")
        self.pres = f("presence_penalty")
        self.do_sample = torch.tensor([x.do_sample for x in p], dtype=torch.bool, device=dev)
        self.any_sample = any(x.do_sample for x in p)
        self.any_rep = any(x.repetition_penalty != 1.0 for x in p)
        self.any_freq = any(x.frequency_penalty != 0.0 or x.presence_penalty != 0.0 for x in p)
        self.any_temp = any(x.do_sample and x.temperature != 1.0 for x in p)
        self.any_topk = any(x.do_sample and x.top_k > 0 for x in p)
        self.any_topp = any(x.do_sample and x.top_p < 1.0 for x in p)
        self.any_typical = any(x.do_sample and x.typical_p < 1.0 for x in p)
        self.any_watermark = any(x.watermark for x in p)
        self.any_grammar = any(g is not None for g in self.grammars)
        self.max_alternatives = max((x.return_k_alternatives for x in p), default=0)
        self.all_plain = all(x.plain for x in p) and not self.any_grammar
        for i, x in enumerate(p):
            if x.do_sample and i not in self.generators:
                self.generators[i] = torch.Generator(device=dev).manual_seed(int(x.seed) & 0x7FFFFFFFFFFFFFFF)

    # ------------------------------------------------------------------ batch surgery
    def filter(self, keep: Sequence[int]) -> "HeterogeneousNextTokenChooser":
        new = HeterogeneousNextTokenChooser.__new__(HeterogeneousNextTokenChooser)
        new.params = [self.params[i] for i in keep]
        new.device, new.vocab_size, new.watermark = self.device, self.vocab_size, self.watermark
        new.grammars = [self.grammars[i] for i in keep]
        new.generators = {j: self.generators[i] for j, i in enumerate(keep) if i in self.generators}
        new._build()
        return new

    @classmethod
    def concatenate(cls, choosers: Sequence["HeterogeneousNextTokenChooser"]) -> "HeterogeneousNextTokenChooser":
        first = choosers[0]
        new = cls.__new__(cls)
        new.params, new.grammars, new.generators = [], [], {}
        for c in choosers:
            base = len(new.params)
            new.params += c.params
            new.grammars += c.grammars
            for i, g in c.generators.items():
                new.generators[base + i] = g
        new.device, new.vocab_size, new.watermark = first.device, first.vocab_size, first.watermark
        new._build()
        return new

    # ------------------------------------------------------------------ logits pipeline
    def warp(self, history: Optional[torch.Tensor], history_mask: Optional[torch.Tensor], scores: torch.Tensor,
             last_tokens: Optional[Sequence[int]] = None) -> torch.Tensor:
        """scores: [B, V] float32 -> processed scores.  history: [B, L] token ids seen so far (prompt + generated),
        history_mask: [B, L] bool."""
        B, V = scores.shape
        if (self.any_rep or self.any_freq) and history is not None:
            h = history.long().clamp(0, V - 1)
            m = history_mask if history_mask is not None else torch.ones_like(h, dtype=torch.bool)
            if self.any_rep:
                # padded history slots carry token id 0 with mask False: accumulate instead of overwriting, so that they can
                # never clear the mark of a real token 0 in the same row
                seen = torch.zeros(B, V, dtype=torch.int32, device=scores.device).scatter_add_(1, h, m.to(torch.int32)) > 0
                pen = self.rep[:, None]
                scores = torch.where(seen, torch.where(scores < 0, scores * pen, scores / pen), scores)
            if self.any_freq:
                counts = torch.zeros(B, V, dtype=scores.dtype, device=scores.device)
                counts.scatter_add_(1, h, m.to(scores.dtype))
                scores = scores - counts * self.freq[:, None] - (counts > 0).to(scores.dtype) * self.pres[:, None]
        if self.any_watermark and last_tokens is not None:
            for i, x in enumerate(self.params):
                if x.watermark:
                    scores[i] = self.watermark(int(last_tokens[i]), scores[i])
        if self.any_grammar:
            for i, g in enumerate(self.grammars):
                if g is not None:
                    allowed = g.allowed_tokens()
                    if allowed is not None:
                        mask = torch.full((V,), float("-inf"), device=scores.device)
                        mask[torch.as_tensor(allowed, device=scores.device, dtype=torch.long)] = 0
                        scores[i] = scores[i] + mask
        if not self.any_sample:
            return scores
        ds = self.do_sample[:, None]
        if self.any_temp:
            scores = torch.where(ds, scores / self.temperature[:, None], scores)
        if self.any_topk:
            k = torch.where(self.top_k > 0, self.top_k, torch.full_like(self.top_k, V)).clamp(max=V)
            kmax = int(k.max().item())
            topv = scores.topk(kmax, dim=-1).values
            thresh = topv.gather(1, (k - 1).clamp(0, kmax - 1)[:, None])
            scores = torch.where(ds & (scores < thresh), torch.full_like(scores, float("-inf")), scores)
        if self.any_topp:
            sorted_s, idx = scores.sort(dim=-1, descending=False)
            cum = sorted_s.softmax(-1).cumsum(-1)
            remove = cum <= (1 - self.top_p[:, None])
            remove[:, -1] = False
            remove = remove.scatter(1, idx, remove)
            scores = torch.where(ds & remove, torch.full_like(scores, float("-inf")), scores)
        if self.any_typical:
            logp = scores.log_softmax(-1)
            p = logp.exp()
            ent = -(torch.where(p > 0, p * logp, torch.zeros_like(p))).sum(-1, keepdim=True)
            shifted = (-logp - ent).abs()
            sorted_sh, idx = shifted.sort(dim=-1, descending=False)
            cum = scores.gather(-1, idx).softmax(-1).cumsum(-1)
            last = (cum < self.typical_p[:, None]).sum(-1).clamp(max=V - 1)
            remove = sorted_sh > sorted_sh.gather(1, last[:, None])
            remove = remove.scatter(1, idx, remove)
            scores = torch.where(ds & (self.typical_p[:, None] < 1.0) & remove, torch.full_like(scores, float("-inf")), scores)
        return scores

    def _sample(self, scores: torch.Tensor, rows: Optional[Sequence[int]] = None) -> torch.Tensor:
        greedy = scores.argmax(-1)
        if not self.any_sample:
            return greedy
        probs = scores.softmax(-1)
        out = greedy.clone()
        B = scores.shape[0]
        for r in range(B):
            i = rows[r] if rows is not None else r
            if self.params[i].do_sample:
                q = torch.empty_like(probs[r]).exponential_(1, generator=self.generators[i])
                out[r] = (probs[r] / q).argmax()
        return out

    def __call__(self, history, history_mask, logits: torch.Tensor, last_tokens=None):
        """-> (next_ids [B] int64, logprobs [B] float32, alternatives or None)."""
        scores = self.warp(history, history_mask, logits.float(), last_tokens)
        next_ids = self._sample(scores)
        logp = scores.log_softmax(-1)
        lp = logp.gather(1, next_ids[:, None])[:, 0]
        alts = None
        if self.max_alternatives > 0:
            v, i = logp.topk(self.max_alternatives, dim=-1)
            alts = (i, v)
        if self.any_grammar:
            for r, g in enumerate(self.grammars):
                if g is not None:
                    g.advance(int(next_ids[r]))
        return next_ids, lp, alts

    # ------------------------------------------------------------------ speculation
    def verify(self, history, history_mask, logits: torch.Tensor, spec_ids: torch.Tensor, last_tokens=None):
        """Speculative decoding check.  logits: [B, S+1, V] for the real next position followed by S proposals;
        spec_ids [B, S].  Returns (tokens [B, S+1] chosen by the model at each position, accepted [B] = number of
        emitted tokens in 1..S+1): proposal j is accepted while it equals the model's own choice at position j
        (`utils/tokens.py:405-447` of the reference)."""
        B, S1, V = logits.shape
        chosen = torch.empty(B, S1, dtype=torch.int64, device=logits.device)
        lps = torch.empty(B, S1, dtype=torch.float32, device=logits.device)
        hist, mask = history, history_mask
        for j in range(S1):
            scores = self.warp(hist, mask, logits[:, j].float(), last_tokens)
            ids = self._sample(scores)
            chosen[:, j] = ids
            lps[:, j] = scores.log_softmax(-1).gather(1, ids[:, None])[:, 0]
            if hist is not None and j < S1 - 1:
                hist = torch.cat([hist, spec_ids[:, j:j + 1].to(hist.dtype)], 1)
                if mask is not None:
                    mask = torch.cat([mask, torch.ones(B, 1, dtype=torch.bool, device=mask.device)], 1)
        match = (chosen[:, :-1] == spec_ids.to(chosen.dtype)) if S1 > 1 else torch.zeros(B, 0, dtype=torch.bool, device=logits.device)
        accepted = 1 + match.long().cumprod(1).sum(1) if S1 > 1 else torch.ones(B, dtype=torch.int64, device=logits.device)
        return chosen, lps, accepted


def ngram_speculate(history: torch.Tensor, lengths: Sequence[int], last_ids: Sequence[int], n_spec: int) -> torch.Tensor:
    """Prompt-lookup proposals: find the most recent earlier occurrence of the last token and propose the tokens
    that followed it (`utils/tokens.py:594-615`); falls back to repeating the last token."""
    B = history.shape[0]
    out = torch.empty(B, n_spec, dtype=torch.int64)
    h = history.cpu()
    for b in range(B):
        L = int(lengths[b])
        seq = h[b, :L]
        last = int(last_ids[b])
        pos = (seq[:-1] == last).nonzero()
        if pos.numel() > 0:
            start = int(pos[-1]) + 1
            cand = seq[start:start + n_spec].tolist()
        else:
            cand = []
        cand += [last] * (n_spec - len(cand))
        out[b] = torch.tensor(cand)
    return out.to(history.device)


# ------------------------------------------------------------------------------------------------ stopping
FINISH_LENGTH, FINISH_EOS, FINISH_STOP = 0, 1, 2


@dataclass
class StoppingCriteria:
    max_new_tokens: int = 20
    eos_token_ids: frozenset = frozenset()
    stop_sequences: List[str] = field(default_factory=list)
    ignore_eos_token: bool = False
    current_tokens: int = 0
    current_output: str = ""

    def __call__(self, token_id: int, token_text: str = "") -> Tuple[bool, Optional[int]]:
        self.current_tokens += 1
        if self.current_tokens >= self.max_new_tokens:
            return True, FINISH_LENGTH
        if not self.ignore_eos_token and token_id in self.eos_token_ids:
            return True, FINISH_EOS
        if self.stop_sequences:
            self.current_output += token_text
            for s in self.stop_sequences:
                if s and self.current_output.endswith(s):
                    return True, FINISH_STOP
            keep = max(len(s) for s in self.stop_sequences)
            self.current_output = self.current_output[-(keep + 64):]
        return False, None
