"""Shard runtime: what the 13 RPCs of `LoraxService` operate on.

One instance per GPU process.  It owns the model shard, the paged KV cache, the adapter manager with its
host / HBM tiers, the tokenizer, and the cached batches.  Block tables come from the router (Request.blocks);
the runtime maps every running request to a row of the device-resident decode state.

Counterpart of `server/lorax_server/models/flash_causal_lm.py` (`FlashCausalLMBatch.from_pb / filter /
concatenate`, `generate_token`) and `models/model.py` (`decode_token`, `load_adapter`, `offload_adapter`).
"""

from __future__ import annotations

import collections
import json
import os
import threading
import time
from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..adapters.lora import LoraConfig, load_peft_adapter
from ..adapters.manager import AdapterManager
from ..adapters.medusa import MedusaHeads, is_medusa_dir, load_medusa_adapter
from ..adapters.merges import merge_adapters
from ..config import EngineConfig, ModelConfig
from ..models.decoder import DecoderModel
from ..parallel.tp import TensorParallel
from ..runtime.kv_cache import KVCache
from ..runtime.runner import ModelRunner, PrefillItem
from ..sampling.chooser import (FINISH_EOS, FINISH_LENGTH, FINISH_STOP, HeterogeneousNextTokenChooser, NextTokenParams, ngram_speculate,
                                StoppingCriteria)
from ..sampling.grammar import compile_schema
from ..utils.sources import resolve_adapter, resolve_model
from ..utils.weights import Weights, checkpoint_quantization, safetensors_nbytes, weight_files
from .proto import load_pb


class Detokenizer:
    """Incremental detokenisation with a sliding window of ids, so that multi-token characters and
    leading-space conventions come out right (same scheme as `models/model.py:195-219` of the reference)."""

    def __init__(self, tokenizer, prompt_ids: Sequence[int]):
        self.tok = tokenizer
        self.ids = list(prompt_ids[-8:])
        self.prefix = 0
        self.read = len(self.ids)

    def push(self, token_id: int) -> str:
        self.ids.append(token_id)
        if self.tok is None:
            return ""
        prefix_text = self.tok.decode(self.ids[self.prefix:self.read], skip_special_tokens=False)
        new_text = self.tok.decode(self.ids[self.prefix:], skip_special_tokens=False)
        if len(new_text) > len(prefix_text) and not new_text.endswith("�"):
            out = new_text[len(prefix_text):]
            self.prefix = self.read
            self.read = len(self.ids)
            return out
        return ""


@dataclass
class SeqState:
    request_id: int
    batch_id: int
    prompt_ids: List[int]
    blocks: List[int]
    adapter_index: int
    params: NextTokenParams
    stopping: StoppingCriteria
    detok: Detokenizer
    row: int = -1
    output_ids: List[int] = field(default_factory=list)
    output_text: str = ""
    grammar: Optional[object] = None
    seed: int = 0
    spec_next: Optional[List[int]] = None        # Medusa guesses for the tokens after the last emitted one
    medusa_index: int = 0                        # whose heads guess for this request (0 = the default heads)


class ShardRuntime:
    def __init__(self, model: DecoderModel, tokenizer=None, cfg: Optional[EngineConfig] = None, model_id: str = "",
                 num_blocks: Optional[int] = None, max_batch: int = 256, adapter_arena_bytes: Optional[int] = None):
        self.pb = load_pb()
        self.model = model
        self.tokenizer = tokenizer
        self.cfg = cfg or EngineConfig()
        self.model_id = model_id
        self.tp = model.tp
        c = model.config
        dev = model.device
        if adapter_arena_bytes is None:
            if dev.type == "cuda":
                total = torch.cuda.get_device_properties(dev).total_memory
                adapter_arena_bytes = int(total * self.cfg.adapter_memory_fraction)
            else:
                adapter_arena_bytes = 256 << 20
        self.adapters = AdapterManager(model, arena_bytes=adapter_arena_bytes,
                                       host_bytes=int(self.cfg.host_adapter_cache_gb * (1 << 30)))
        page = self.cfg.block_size
        if num_blocks is None:
            if dev.type == "cuda":
                from ..runtime.kv_cache import plan_kv_blocks
                num_blocks = plan_kv_blocks(model, self.cfg, max_batch, page)      # a maximum prefill runs first: its peak is measured
            else:
                num_blocks = 1024
        from ..runtime.kv_cache import kv_dtype_of
        self.kv = KVCache(c.num_hidden_layers, num_blocks, model.nkv, model.d, kv_dtype_of(model, self.cfg), dev, page)
        self.runner = ModelRunner(model, self.kv, max_batch=max_batch, max_seq_tokens=self.cfg.max_total_tokens,
                                  max_prefill_tokens=max(self.cfg.max_batch_prefill_tokens, 16), use_graphs=self.cfg.compile)
        self.seqs: Dict[int, SeqState] = {}
        self.batches: Dict[int, List[int]] = {}
        eos = c.eos_token_id
        self.eos_ids = frozenset(eos if isinstance(eos, (list, tuple)) else ([eos] if eos is not None else []))
        self.special_ids = set(self.eos_ids)
        self.downloaded: Dict[str, Tuple[LoraConfig, object]] = {}
        self.lock = threading.Lock()
        self.spec_stats = {"steps": 0, "tokens": 0}          # speculative decoding: row-steps and tokens they produced
        # Medusa heads: pinned host copies by adapter key, device copies by adapter index (0 = the default adapter, applied to
        # every request whose own adapter has no heads)
        self.medusa_host: Dict[str, tuple] = {}
        self.medusa: Dict[int, "MedusaHeads"] = {}
        self.fused_stats = {"one_pass": 0, "two_pass": 0}    # fused Prefill + Decode requests served in one / two forward passes

    # ------------------------------------------------------------------ info / health
    def info(self):
        pb = self.pb
        c = self.model.config
        r = pb.InfoResponse(requires_padding=False, dtype=str(self.model.dtype).replace("torch.", ""),
                            device_type=self.model.device.type, block_size=self.kv.page, speculate=self.cfg.speculative_tokens,
                            supports_generation=True, supports_embeddings=False, supports_classification=False,
                            chunked_prefill=self.cfg.chunked_prefill, requires_block_allocator=True,
                            fused_prefill_decode=True)
        if c.sliding_window:
            r.window_size = c.sliding_window
        for aid, idx in getattr(self, "preloaded", {}).items():
            r.preloaded_adapters.append(pb.PreloadedAdapter(adapter_parameters=pb.AdapterParameters(adapter_ids=[aid]),
                                                            adapter_source=getattr(self, "preloaded_source", 0), adapter_index=idx))
        return r

    def health(self):
        """Unhealthy once a kernel has given up on a bounded wait (a peer GPU that stopped answering): the step that saw it
        failed its batch, and the launcher restarts the shard group (the reference's health check fails the same way when a
        shard's prefill raises, router/src/health.rs:150-178)."""
        if getattr(self.runner, "device_failed", None):
            raise RuntimeError("shard is unhealthy: " + self.runner.device_failed)
        # A one-token prefill into block 0, which no request ever owns: every kernel of a step runs (and, under tensor
        # parallelism, every collective: the router sends Health to all shards at once).
        from ..runtime.runner import PrefillItem
        _, lps, _ = self.runner.prefill([PrefillItem([0], 0, [0])])
        if self.model.device.type == "cuda":
            torch.cuda.synchronize(self.model.device)
            from ..ops import native
            native.workspace(self.model.device).check_status()
        if lps is not None and not bool(torch.isfinite(lps.float()).all()):
            raise RuntimeError("shard is unhealthy: the probe step returned a non-finite log-probability")
        return self.pb.HealthResponse()

    def warmup(self, req):
        """The KV cache was sized at construction, after a maximum prefill had run and its memory peak had been measured
        (`runtime/kv_cache.py:plan_kv_blocks`); report what it can hold."""
        return self.pb.WarmupResponse(max_supported_total_tokens=self.kv.max_tokens)

    # ------------------------------------------------------------------ tokenizer helpers
    def tokenize(self, text: str, add_special: bool = True) -> List[int]:
        if self.tokenizer is None:
            return [int(x) for x in text.split()] if text.replace(" ", "").isdigit() else [ord(ch) % self.model.config.vocab_size for ch in text]
        return self.tokenizer.encode(text, add_special_tokens=add_special).ids

    def router_tokenizer_json(self) -> str:
        """The tokenizer file as a string, for the router to tokenise requests itself; empty when there is no tokenizer file.
        A first line `#images` tells the router that this runtime expands image markdown (`![](uri)`) into feature tokens: prompts
        whose images the router cannot size itself (URLs, unknown formats) keep coming to the shard; the JSON behind `#images` tells
        the router how many tokens an image becomes."""
        if self.tokenizer is None:
            return ""
        plain = type(self).tokenize in (ShardRuntime.tokenize, EncoderRuntime.tokenize)
        return ("" if plain else "#images " + json.dumps(self.image_token_policy()) + "\n") + self.tokenizer.to_str()

    def image_token_policy(self) -> dict:
        """How many tokens an image in a prompt becomes, for the router's own count (`csrc/host/image_chunks.hpp`); `{}`: only this
        runtime can tell."""
        return {}

    def tokenize_detailed(self, body: dict) -> list:
        text = body.get("inputs", "")
        if self.tokenizer is None:
            return [{"id": i, "text": str(i), "start": 0, "stop": 0} for i in self.tokenize(text)]
        enc = self.tokenizer.encode(text, add_special_tokens=body.get("add_special_tokens", True))
        return [{"id": i, "text": t, "start": o[0], "stop": o[1]} for i, t, o in zip(enc.ids, enc.tokens, enc.offsets)]

    def apply_chat_template(self, body: dict) -> str:
        from .chat_template import render_chat
        return render_chat(body.get("messages", []), self.chat_template, tools=body.get("tools"), bos_token=self.bos_token,
                           eos_token=self.eos_token, guideline=body.get("guideline"), tool_prompt=body.get("tool_prompt"))

    chat_template: Optional[str] = None
    bos_token: str = ""
    eos_token: str = ""

    # ------------------------------------------------------------------ adapters
    def _adapter_key(self, params, source: int) -> str:
        ids = list(params.adapter_ids)
        if len(ids) == 1:
            return f"{source}:{ids[0]}"
        return f"{source}:" + ",".join(ids) + f"|{params.merge_strategy}|{params.density}|{params.majority_sign_method}|" + \
            ",".join(f"{w:.6g}" for w in params.weights)

    def download_adapter(self, req):
        pb = self.pb
        params, source = req.adapter_parameters, req.adapter_source
        key = self._adapter_key(params, source)
        if self.adapters.host.get(key) is not None:          # already packed in the pinned host tier
            return pb.DownloadAdapterResponse(downloaded=True, memory_fraction=self.adapters.memory_fraction(key))
        src_name = {0: "hub", 1: "s3", 2: "local", 3: "pbase"}.get(source, "hub")
        loaded = []
        for aid in params.adapter_ids:
            if aid in ("", "__base_model__"):
                continue
            path = resolve_adapter(aid, src_name, api_token=req.api_token if req.HasField("api_token") else None)
            if is_medusa_dir(path):
                if len(params.adapter_ids) > 1:
                    raise ValueError("Medusa adapters cannot be merged with other adapters")
                self.medusa_host[key] = load_medusa_adapter(path)
                if not os.path.exists(os.path.join(path, "adapter_config.json")):           # heads only, no LoRA part
                    total = torch.cuda.get_device_properties(self.model.device).total_memory if self.model.device.type == "cuda" else 1 << 40
                    nbytes = sum(v.numel() * 2 for v in self.medusa_host[key][1].values())
                    return pb.DownloadAdapterResponse(downloaded=True, memory_fraction=nbytes / (total * max(self.cfg.adapter_memory_fraction, 1e-6)))
            loaded.append(load_peft_adapter(path))
        if not loaded:
            return pb.DownloadAdapterResponse(downloaded=False, memory_fraction=0.0)
        if len(loaded) == 1:
            cfg, mm = loaded[0]
        else:
            strategy = {0: "linear", 1: "ties", 2: "dare_linear", 3: "dare_ties"}[params.merge_strategy]
            cfg, mm = merge_adapters(loaded, list(params.weights) or [1.0] * len(loaded), strategy, params.density or 1.0,
                                     "frequency" if params.majority_sign_method == 1 else "total")
        self.adapters.register(key, cfg, mm)
        return pb.DownloadAdapterResponse(downloaded=True, memory_fraction=self.adapters.memory_fraction(key))

    def load_adapter(self, req):
        key = self._adapter_key(req.adapter_parameters, req.adapter_source)
        if self.adapters.host.get(key) is None and key not in self.medusa_host:
            self.download_adapter(self.pb.DownloadAdapterRequest(adapter_parameters=req.adapter_parameters, adapter_source=req.adapter_source))
        if key in self.medusa_host:
            self.load_medusa(req.adapter_index, *self.medusa_host[key])
            if self.adapters.host.get(key) is None:          # heads only; a Medusa + LoRA adapter goes on below
                return self.pb.LoadAdapterResponse(loaded=True)
        ok = self.adapters.load(req.adapter_index, key)
        if not ok:
            raise RuntimeError(f"adapter {key} does not fit in the adapter memory reservation")
        return self.pb.LoadAdapterResponse(loaded=True)

    def offload_adapter(self, req):
        had_heads = self.medusa.pop(req.adapter_index, None) is not None if req.adapter_index != 0 else False
        return self.pb.OffloadAdapterResponse(offloaded=self.adapters.offload(req.adapter_index) or had_heads)

    def load_default_adapter(self, adapter_id: str, source: int = 0):
        """The adapter named on the command line: a LoRA goes to adapter index 1; Medusa heads become the default heads
        (index 0), which also turns speculation on with one token per head."""
        pb = self.pb
        params = pb.AdapterParameters(adapter_ids=[adapter_id])
        self.download_adapter(pb.DownloadAdapterRequest(adapter_parameters=params, adapter_source=source))
        key = self._adapter_key(params, source)
        if key in self.medusa_host:
            self.load_medusa(0, *self.medusa_host[key])
        if self.adapters.host.get(key) is not None:
            idx = 1 + max(list(getattr(self, "preloaded", {}).values()) + [0])
            self.load_adapter(pb.LoadAdapterRequest(adapter_parameters=params, adapter_source=source, adapter_index=idx))
            self.preloaded = dict(getattr(self, "preloaded", {}), **{adapter_id: idx})      # announced to the router like a preloaded one
            self.preloaded_source = source

    def preload_adapters(self, adapter_ids: Sequence[str], source: int = 0, threads: int = 20):
        """Adapters named at start-up (`--preloaded-adapter-ids`): fetched in parallel, loaded under indices 1..n and announced in
        `Info`, so the router maps requests for them to those indices and never has to load them on demand (reference:
        `server.py:342-417`: 20 download threads, then `register_preloaded_adapters`)."""
        from concurrent.futures import ThreadPoolExecutor
        pb = self.pb
        ids = [a for a in adapter_ids if a]
        if not ids:
            return
        first = 1 + max([i for i in getattr(self, "preloaded", {}).values()] + [0])

        def fetch(aid):
            self.download_adapter(pb.DownloadAdapterRequest(adapter_parameters=pb.AdapterParameters(adapter_ids=[aid]), adapter_source=source))
        with ThreadPoolExecutor(max_workers=max(1, min(threads, len(ids)))) as ex:
            list(ex.map(fetch, ids))
        self.preloaded = dict(getattr(self, "preloaded", {}))
        self.preloaded_source = source
        for k, aid in enumerate(ids):
            self.load_adapter(pb.LoadAdapterRequest(adapter_parameters=pb.AdapterParameters(adapter_ids=[aid]), adapter_source=source,
                                                    adapter_index=first + k))
            self.preloaded[aid] = first + k

    def load_medusa(self, adapter_index: int, config, tensors):
        """Put Medusa heads on the device under `adapter_index` (0 = default heads for every request).  As in the reference
        (adapters/medusa.py:52-71) heads loaded at request time need speculation to be on and must not have more heads than
        the configured number of speculative tokens; the first heads loaded as index 0 turn speculation on."""
        heads = MedusaHeads(config, tensors, self.model.device, self.model.dtype)
        if adapter_index == 0 and self.cfg.speculative_tokens == 0:
            self.cfg.speculative_tokens = heads.num_heads
        if self.cfg.speculative_tokens == 0:
            raise ValueError("Medusa adapters can only be loaded at request time when the server was started with speculation on "
                             "(a default Medusa adapter or --speculative-tokens)")
        if heads.num_heads > self.cfg.speculative_tokens and adapter_index != 0:
            raise ValueError(f"cannot load a Medusa adapter with {heads.num_heads} heads: the server speculates "
                             f"{self.cfg.speculative_tokens} tokens")
        self.medusa[adapter_index] = heads
        self.model.keep_hidden = True

    def _medusa_guess(self, seqs: List[SeqState], hidden: torch.Tensor):
        """Fill `spec_next` of every sequence from the hidden state (one row per sequence) that produced its last token."""
        if not self.medusa:
            return
        groups: Dict[int, List[int]] = {}
        for i, s in enumerate(seqs):
            idx = s.medusa_index if s.medusa_index in self.medusa else 0
            if idx in self.medusa:
                groups.setdefault(idx, []).append(i)
            else:
                s.spec_next = None
        inp = SimpleNamespace(head_tok_slot=None, local_logits=False)
        for idx, members in groups.items():
            rows = hidden.index_select(0, torch.tensor(members, device=hidden.device))
            guesses = self.medusa[idx].propose(rows, lambda x: self.model.lm_head_forward(x, inp)).tolist()
            for i, gs in zip(members, guesses):
                seqs[i].spec_next = [int(t) for t in gs]

    # ------------------------------------------------------------------ batches
    def clear_cache(self, req):
        ids = [req.id] if req.HasField("id") else list(self.batches.keys())
        for bid in ids:
            for rid in self.batches.pop(bid, []):
                self._drop(rid)
        if self.seqs:
            self._resort()
        return self.pb.ClearCacheResponse()

    def _drop(self, rid: int):
        s = self.seqs.pop(rid, None)
        if s is not None and s.row >= 0:
            self.runner.retire([s.row])
            self.runner.state.drop_row(s.row)

    def _resort(self):
        mapping = self.runner.resort()
        for s in self.seqs.values():
            if s.row in mapping:
                s.row = mapping[s.row]

    def filter_batch(self, req):
        keep = set(req.request_ids)
        for rid in self.batches.get(req.batch_id, []):
            if rid not in keep:
                self._drop(rid)
        self.batches[req.batch_id] = [r for r in self.batches.get(req.batch_id, []) if r in keep]
        self._resort()
        return self.pb.FilterBatchResponse(batch=self._cached(req.batch_id))

    def _cached(self, bid: int):
        rids = self.batches.get(bid, [])
        mt = sum(len(self.seqs[r].prompt_ids) + self.seqs[r].stopping.max_new_tokens for r in rids)
        cur = sum(len(self.seqs[r].prompt_ids) + len(self.seqs[r].output_ids) for r in rids)
        return self.pb.CachedBatch(id=bid, request_ids=rids, size=len(rids), max_tokens=mt, current_tokens=cur)

    # ------------------------------------------------------------------ token post-processing
    def _params_from_pb(self, p) -> NextTokenParams:
        return NextTokenParams(temperature=p.temperature or 1.0, top_k=p.top_k, top_p=p.top_p or 1.0, typical_p=p.typical_p or 1.0,
                               do_sample=p.do_sample, seed=p.seed, repetition_penalty=p.repetition_penalty or 1.0,
                               frequency_penalty=p.frequency_penalty, presence_penalty=p.presence_penalty, watermark=p.watermark,
                               return_k_alternatives=p.return_k_alternatives, schema=p.schema if p.HasField("schema") else None)

    def _emit(self, s: SeqState, token: int, logprob: float, alts=None):
        """Append a token; returns (Generation or None for other ranks' requests, finished)."""
        pb = self.pb
        s.output_ids.append(token)
        text = s.detok.push(token)
        s.output_text += text
        stop, reason = s.stopping(token, text)
        mine = (s.request_id % self.tp.world_size) == self.tp.rank
        gen = None
        if mine:
            nt = pb.NextTokens(ids=[token], logprobs=[logprob], texts=[text], is_special=[token in self.special_ids])
            if alts is not None:
                ids, lps = alts
                nt.alternative_tokens.append(pb.AlternativeTokens(ids=ids, logprobs=lps, texts=[self._tok_text(i) for i in ids]))
            gen = pb.Generation(request_id=s.request_id, next_tokens=nt, prefill_tokens_length=len(s.prompt_ids))
            if stop:
                out_text = s.output_text
                if reason == FINISH_STOP:
                    for ss in s.stopping.stop_sequences:
                        if ss and out_text.endswith(ss):
                            break
                gt = pb.GeneratedText(text=out_text, generated_tokens=len(s.output_ids), skipped_tokens=0, finish_reason=reason)
                if s.params.do_sample:
                    gt.seed = s.seed
                gen.generated_text.CopyFrom(gt)
        return gen, stop

    def _emit_many(self, s: SeqState, tokens: Sequence[int], logprobs: Sequence[float]):
        """Append the tokens a speculative step accepted (stopping at the first that ends the request) as ONE Generation
        whose NextTokens lists them in order.  Returns (Generation or None, finished, number of tokens kept)."""
        pb = self.pb
        mine = (s.request_id % self.tp.world_size) == self.tp.rank
        ids, lps, texts, special = [], [], [], []
        stop, reason = False, None
        for tok, lp in zip(tokens, logprobs):
            s.output_ids.append(tok)
            text = s.detok.push(tok)
            s.output_text += text
            ids.append(tok); lps.append(lp); texts.append(text); special.append(tok in self.special_ids)
            stop, reason = s.stopping(tok, text)
            if stop:
                break
        gen = None
        if mine:
            gen = pb.Generation(request_id=s.request_id, next_tokens=pb.NextTokens(ids=ids, logprobs=lps, texts=texts, is_special=special),
                                prefill_tokens_length=len(s.prompt_ids))
            if stop:
                gen.generated_text.CopyFrom(pb.GeneratedText(text=s.output_text, generated_tokens=len(s.output_ids), skipped_tokens=0,
                                                             finish_reason=reason))
        return gen, stop, len(ids)

    def _decode_speculative(self, seqs: List[SeqState], n_spec: int):
        """Greedy decoding with prompt-lookup proposals (reference: `utils/tokens.py:594-615` proposes, `:363-460` verifies).
        Every row is run as a short ragged prefill over [last token, proposals...] against its cached context; the model's
        arg-max at each position is compared with the proposal that follows, and the longest agreeing prefix plus one
        token is emitted.  Rejected positions leave stale K/V behind the new context length, where nothing reads them
        before they are overwritten."""
        page = self.kv.page
        items, props = [], []
        for s in seqs:
            h = s.prompt_ids + s.output_ids
            room = len(s.blocks) * page - len(h) - 1                 # slots left after the token that must be written anyway
            want = max(0, min(n_spec, room, s.stopping.max_new_tokens - len(s.output_ids) - 1))
            if want > 0 and s.spec_next:                            # Medusa heads guessed after the previous pass
                cand = list(s.spec_next[:want])
            elif want > 0:
                hist = torch.tensor([h], dtype=torch.long)
                cand = ngram_speculate(hist, [len(h)], [h[-1]], want)[0].tolist()
            else:
                cand = []
            props.append(cand)
            items.append(PrefillItem([h[-1]] + cand, len(h) - 1, list(s.blocks), s.adapter_index, all_logprobs=True))
        next_ids, lps, _ = self.runner.prefill(items)
        ids_h, lps_h = next_ids.tolist(), lps.tolist()
        out, o, last_rows = [], 0, []
        for s, cand in zip(seqs, props):
            n = 1 + len(cand)
            toks, tlps = [int(ids_h[o])], [float(lps_h[o])]
            for j, c in enumerate(cand):
                if c != toks[-1]:
                    break
                toks.append(int(ids_h[o + j + 1]))
                tlps.append(float(lps_h[o + j + 1]))
            out.append((toks, tlps))
            last_rows.append(o + len(toks) - 1)                     # the position whose arg-max is the last token kept
            o += n
        if self.medusa and self.model.last_hidden is not None:
            self._medusa_guess(seqs, self.model.last_hidden.index_select(0, torch.tensor(last_rows, device=self.model.last_hidden.device)))
        return out

    def _tok_text(self, tid: int) -> str:
        return self.tokenizer.decode([tid], skip_special_tokens=False) if self.tokenizer is not None else ""

    def _sample_rows(self, seqs: List[SeqState], logits: torch.Tensor, greedy_ids: List[int], greedy_lps: List[float]):
        """Per-request sampling for the rows whose parameters need more than an argmax; the rest keep the result of
        the fused greedy kernel.  Returns (ids, logprobs, alternatives)."""
        need = [i for i, s in enumerate(seqs) if not (s.params.plain and s.grammar is None)]
        ids, lps, alts = list(greedy_ids), list(greedy_lps), [None] * len(seqs)
        if not need:
            return ids, lps, alts
        sub = [seqs[i] for i in need]
        chooser = HeterogeneousNextTokenChooser([s.params for s in sub], logits.device, logits.shape[-1],
                                                grammars=[s.grammar for s in sub])
        for j, s in enumerate(sub):
            g = getattr(s, "_gen", None)
            if g is not None:
                chooser.generators[j] = g
        L = max(len(s.prompt_ids) + len(s.output_ids) for s in sub)
        hist = torch.zeros(len(sub), L, dtype=torch.long, device=logits.device)
        mask = torch.zeros(len(sub), L, dtype=torch.bool, device=logits.device)
        for j, s in enumerate(sub):
            h = s.prompt_ids + s.output_ids
            hist[j, :len(h)] = torch.tensor(h, device=logits.device)
            mask[j, :len(h)] = True
        rows = torch.tensor(need, device=logits.device)
        nid, nlp, nalts = chooser(hist, mask, logits.index_select(0, rows).float(),
                                  last_tokens=[(s.prompt_ids + s.output_ids)[-1] for s in sub])
        for j, s in enumerate(sub):
            s._gen = chooser.generators.get(j)
        nid_l, nlp_l = nid.tolist(), nlp.tolist()
        for j, i in enumerate(need):
            ids[i], lps[i] = nid_l[j], nlp_l[j]
            k = seqs[i].params.return_k_alternatives
            if nalts is not None and k > 0:
                alts[i] = (nalts[0][j, :k].tolist(), nalts[1][j, :k].tolist())
        return ids, lps, alts

    # ------------------------------------------------------------------ Prefill / Decode
    def prefill(self, req):
        """Prefill of a new batch.  With `decode_batches` set, the running batches take one decode step in the same
        forward pass (one pass over the weights for both) and the response merges everything into one cached batch."""
        prof = getattr(self, "profiler", None)
        if prof is not None:
            prof.step()
        if len(req.decode_batches):
            return self._prefill_and_decode(req)
        seqs, items, chunks = self._new_sequences(req.batch)
        next_ids, lps, logits = self.runner.prefill(items + chunks)
        if not items:                                       # prompt chunks only: nothing to emit yet
            return self.pb.PrefillResponse()
        return self._finish_prefill(req.batch, seqs, items, next_ids, lps, logits)

    def _new_sequences(self, batch):
        """-> (sequences, their prefill items, items of prompt chunks that do not reach the end of their prompt).  A request
        with `chunk_len` set and `cache_len + chunk_len` short of its prompt is such a chunk: its keys and values are written
        and nothing else happens; the router sends the rest of the prompt in later Prefill calls with a larger `cache_len`
        (chunked prefill: reference `server.py:93-123`, `flash_causal_lm.py:171-389`)."""
        items, seqs, chunks = [], [], []
        max_in = self.cfg.max_input_length
        for r in batch.requests:
            ids = list(r.tokenized_inputs.ids) if r.HasField("tokenized_inputs") and len(r.tokenized_inputs.ids) else self.tokenize(r.inputs)
            trunc = r.truncate or max_in
            ids = ids[-trunc:]
            if r.HasField("chunk_len") and r.cache_len + r.chunk_len < len(ids):
                lora_index = r.adapter_index if (r.adapter_index == 0 or self.adapters.is_loaded(r.adapter_index)) else 0
                chunks.append(PrefillItem(ids[r.cache_len: r.cache_len + r.chunk_len], r.cache_len, list(r.blocks), lora_index,
                                          want_logits=False))
                continue
            params = self._params_from_pb(r.parameters)
            stopping = StoppingCriteria(r.stopping_parameters.max_new_tokens or 1, self.eos_ids, list(r.stopping_parameters.stop_sequences),
                                        r.stopping_parameters.ignore_eos_token)
            lora_index = r.adapter_index
            if r.adapter_index != 0 and not self.adapters.is_loaded(r.adapter_index):
                if r.adapter_index not in self.medusa:
                    raise RuntimeError(f"adapter index {r.adapter_index} is not loaded on this shard")
                lora_index = 0                                      # Medusa heads only: the base model's weights
            s = SeqState(r.id, batch.id, ids, list(r.blocks), lora_index, params, stopping, Detokenizer(self.tokenizer, ids), seed=params.seed,
                         medusa_index=r.adapter_index)
            if params.schema:
                s.grammar = compile_schema(params.schema, self.tokenizer, self.eos_ids)
            seqs.append(s)
            items.append(PrefillItem(ids[r.cache_len:] if r.cache_len else ids, r.cache_len, list(r.blocks), lora_index,
                                     all_logprobs=r.prefill_logprobs))
        return seqs, items, chunks

    def _finish_prefill(self, batch, seqs, items, next_ids, lps, logits, merge_with: Optional[List[int]] = None, merged_id: Optional[int] = None,
                        extra_generations=()):
        """Sample / emit the first tokens, give the survivors decode rows and answer with the cached batch.  With
        `merge_with` (request ids that survived a decode step of the same pass) everything lands in batch `merged_id`."""
        pb = self.pb
        # rows of `logits` per request: the last one when prefill log-probs were requested
        row_of, o = [], 0
        for it in items:
            n = len(it.token_ids) if it.all_logprobs else 1
            row_of.append(o + n - 1)
            o += n
        last_rows = torch.tensor(row_of, device=next_ids.device)
        gid = next_ids.index_select(0, last_rows).tolist()
        glp = lps.index_select(0, last_rows).tolist()
        # (a fused prefill + decode pass keeps no logits: it is only taken when every request is plain greedy)
        ids_l, lps_l, alts = self._sample_rows(seqs, logits.index_select(0, last_rows) if logits is not None else None, gid, glp)
        if self.medusa and self.model.last_hidden is not None and self.model.last_hidden.shape[0] == next_ids.shape[0]:
            self._medusa_guess(seqs, self.model.last_hidden.index_select(0, last_rows))
        gens, live, rows, firsts, poss, blks, ads = [], [], [], [], [], [], []
        o = 0
        for s, it, tok, lp, alt in zip(seqs, items, ids_l, lps_l, alts):
            gen, stop = self._emit(s, int(tok), float(lp), alt)
            if gen is not None and it.all_logprobs:
                n = len(it.token_ids)
                plp = torch.log_softmax(logits[o:o + n].float(), -1)
                tgt = torch.tensor(it.token_ids[1:], device=logits.device)
                vals = [float("nan")] + plp[:-1].gather(1, tgt[:, None])[:, 0].tolist() if n > 1 else [float("nan")]
                gen.prefill_tokens.CopyFrom(pb.NextTokens(ids=list(it.token_ids), logprobs=vals,
                                                          texts=[self._tok_text(i) for i in it.token_ids]))
            o += len(it.token_ids) if it.all_logprobs else 1
            if gen is not None:
                gens.append(gen)
            if not stop:
                self.seqs[s.request_id] = s
                s.row = self.runner.state.take_row(s.request_id)
                live.append(s.request_id)
                rows.append(s.row); firsts.append(int(tok)); poss.append(len(s.prompt_ids)); blks.append(s.blocks); ads.append(s.adapter_index)
        resp = pb.PrefillResponse(generations=list(extra_generations) + gens)
        if live:
            self.runner.install(rows, firsts, poss, blks, ads)
            self._resort()
        bid = batch.id if merged_id is None else merged_id
        members = list(merge_with or []) + live
        if members:
            self.batches[bid] = members
            for r in members:
                self.seqs[r].batch_id = bid
            resp.batch.CopyFrom(self._cached(bid))
        return resp

    def _prefill_and_decode(self, req):
        """One decode step of the running batches fused with the prefill of a new one."""
        pb = self.pb
        bids = [b.id for b in req.decode_batches]
        rids = [r for b in bids for r in self.batches.get(b, [])]
        if not rids:
            raise RuntimeError("all batches of the fused Prefill request are missing from the cache")
        old = [self.seqs[r] for r in rids]
        seqs, items, chunks = self._new_sequences(req.batch)
        plain = all(s.params.plain and s.grammar is None for s in old + seqs)
        if not (plain and not chunks and self.cfg.speculative_tokens == 0 and not any(it.all_logprobs for it in items) and self.runner.can_mix()
                and self.runner.state.high_water + sum(len(it.token_ids) for it in items) <= self.runner.max_prefill_tokens):
            # same result in two passes: decode the running batches, then prefill the new one into the merged batch
            self.fused_stats["two_pass"] += 1
            d = self.decode(pb.DecodeRequest(batches=list(req.decode_batches)))
            survivors = list(self.batches.pop(bids[0], [])) if d.HasField("batch") else []
            next_ids, lps, logits = self.runner.prefill(items + chunks)
            if not items:                                   # prompt chunks only: the decode step is the whole answer
                resp = pb.PrefillResponse(generations=d.generations)
                if survivors:
                    self.batches[bids[0]] = survivors
                    resp.batch.CopyFrom(self._cached(bids[0]))
                return resp
            return self._finish_prefill(req.batch, seqs, items, next_ids, lps, logits, merge_with=survivors, merged_id=bids[0],
                                        extra_generations=d.generations)
        self.fused_stats["one_pass"] += 1
        k, nd, first_ids, first_lps = self.runner.mixed_step(items)
        ids_p, lps_p = self.runner.wait(k)
        gens, finished = [], []
        for s in old:
            gen, stop = self._emit(s, int(ids_p[s.row]), float(lps_p[s.row]))
            if gen is not None:
                gens.append(gen)
            if stop:
                finished.append(s.request_id)
        for bid in bids:
            self.batches.pop(bid, None)
        for rid in finished:
            self._drop(rid)
        survivors = [r for r in rids if r not in finished]
        return self._finish_prefill(req.batch, seqs, items, first_ids, first_lps, None, merge_with=survivors, merged_id=bids[0],
                                    extra_generations=gens)

    def decode(self, req):
        pb = self.pb
        bids = [b.id for b in req.batches]
        rids = [r for b in bids for r in self.batches.get(b, [])]
        if not rids:
            raise RuntimeError("all batches of the Decode request are missing from the cache")
        seqs = [self.seqs[r] for r in rids]
        need_logits = any(not (s.params.plain and s.grammar is None) for s in seqs)
        # (large batches decode one token per row: verifying guesses multiplies the rows of the step; reference
        # LORAX_SPECULATION_MAX_BATCH_SIZE, adapters/medusa.py:162-166)
        if self.cfg.speculative_tokens > 0 and not need_logits and len(seqs) <= self.cfg.speculation_max_batch_size:
            return self._decode_spec_step(bids, rids, seqs)
        k, b, logits = self.runner.decode(need_logits=need_logits)
        ids_p, lps_p = self.runner.wait(k)
        rows = [s.row for s in seqs]
        gid = [int(ids_p[r]) for r in rows]
        glp = [float(lps_p[r]) for r in rows]
        alts = [None] * len(seqs)
        if need_logits:
            sel = logits.index_select(0, torch.tensor(rows, device=logits.device))
            gid2, glp2, alts = self._sample_rows(seqs, sel, gid, glp)
            changed = [(r, t) for r, t, t0 in zip(rows, gid2, gid) if t != t0]
            if changed:
                # the graph already advanced the state with the greedy token: overwrite the next input id
                rr = torch.tensor([c[0] for c in changed], device=logits.device)
                self.runner.state.input_ids.index_copy_(0, rr, torch.tensor([c[1] for c in changed], dtype=torch.int32, device=logits.device))
            gid, glp = gid2, glp2
        gens, finished = [], []
        for s, tok, lp, alt in zip(seqs, gid, glp, alts):
            gen, stop = self._emit(s, tok, lp, alt)
            if gen is not None:
                gens.append(gen)
            if stop:
                finished.append(s.request_id)
        new_id = bids[0]
        merged = [r for r in rids if r not in finished]
        for bid in bids:
            self.batches.pop(bid, None)
        for rid in finished:
            self._drop(rid)
        resp = pb.DecodeResponse(generations=gens)
        if merged:
            self.batches[new_id] = merged
            for r in merged:
                self.seqs[r].batch_id = new_id
            resp.batch.CopyFrom(self._cached(new_id))
        return resp

    def _decode_spec_step(self, bids, rids, seqs):
        pb = self.pb
        accepted = self._decode_speculative(seqs, self.cfg.speculative_tokens)
        gens, finished, rows, toks, poss, blks = [], [], [], [], [], []
        for s, (tk, lp) in zip(seqs, accepted):
            gen, stop, kept = self._emit_many(s, tk, lp)
            self.spec_stats["steps"] += 1
            self.spec_stats["tokens"] += kept
            if gen is not None:
                gens.append(gen)
            if stop:
                finished.append(s.request_id)
            else:
                rows.append(s.row); toks.append(s.output_ids[-1]); poss.append(len(s.prompt_ids) + len(s.output_ids) - 1); blks.append(s.blocks)
        # the device-resident decode state follows, so that plain decode steps (sampling rows joining later) stay possible
        self.runner.reposition(rows, toks, poss, blks)
        new_id = bids[0]
        merged = [r for r in rids if r not in finished]
        for bid in bids:
            self.batches.pop(bid, None)
        for rid in finished:
            self._drop(rid)
        resp = pb.DecodeResponse(generations=gens)
        if merged:
            self.batches[new_id] = merged
            for r in merged:
                self.seqs[r].batch_id = new_id
            resp.batch.CopyFrom(self._cached(new_id))
        return resp

    def embed(self, req):
        return self.pb.EmbedResponse(errorMsg="this model does not produce embeddings")

    def classify(self, req):
        return self.pb.ClassifyResponse(errorMsg="this model is not a classifier")


# ---------------------------------------------------------------------------------------------- construction
def _token_text(tok) -> Optional[str]:
    """`bos_token` / `eos_token` of a tokenizer_config.json: a string, or an AddedToken dictionary with `content`."""
    if isinstance(tok, dict):
        tok = tok.get("content")
    return tok if isinstance(tok, str) and tok else None


def llama_post_processor(tokenizer, tokenizer_config: dict):
    """The template a Llama tokenizer gets from transformers at load time, which its tokenizer.json does not carry: BOS in front
    when `add_bos_token` (default true), EOS behind when `add_eos_token` (default false).  The reference router applies the same
    override (`router/src/main.rs:587-655`) for tokenizer classes LlamaTokenizer / LlamaTokenizerFast.  None when a token the
    template needs is not in the vocabulary."""
    from tokenizers import processors
    add_bos = tokenizer_config.get("add_bos_token", True)
    add_eos = tokenizer_config.get("add_eos_token", False)
    bos, eos = _token_text(tokenizer_config.get("bos_token")), _token_text(tokenizer_config.get("eos_token"))
    single, pair, special = [], [], []
    for flag, tok in ((add_bos, bos), (add_eos, eos)):
        if flag and (tok is None or tokenizer.token_to_id(tok) is None):
            return None
    if add_bos:
        special.append((bos, tokenizer.token_to_id(bos)))
        single.append(f"{bos}:0")
        pair.append(f"{bos}:0")
    single.append("$A:0")
    pair.append("$A:0")
    if add_eos:
        special.append((eos, tokenizer.token_to_id(eos)))
        single.append(f"{eos}:0")
        pair.append(f"{eos}:0")
    if add_bos:
        pair.append(f"{bos}:1")
    pair.append("$B:1")
    if add_eos:
        pair.append(f"{eos}:1")
    return processors.TemplateProcessing(single=" ".join(single), pair=" ".join(pair), special_tokens=list(dict(special).items()))


def load_tokenizer(model_dir: str):
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.exists(path):
        return None
    from tokenizers import Tokenizer
    tok = Tokenizer.from_file(path)
    # some files carry the padding / truncation of the run that saved them (sentence-transformers: pad to 128, cut at 512);
    # transformers resets both on every call, and serving wants neither: length limits are the router's validation
    tok.no_padding()
    tok.no_truncation()
    cfg_path = os.path.join(model_dir, "tokenizer_config.json")
    if os.path.exists(cfg_path):
        try:
            with open(cfg_path) as f:
                tcfg = json.load(f)
        except (OSError, ValueError):
            tcfg = {}
        if tcfg.get("tokenizer_class") in ("LlamaTokenizer", "LlamaTokenizerFast"):
            pp = llama_post_processor(tok, tcfg)
            if pp is not None:
                tok.post_processor = pp
    return tok


class Seq2SeqRuntime(ShardRuntime):
    """Shard runtime of an encoder-decoder model (T5 family): Prefill runs the encoder once per request and the first decoder
    step, Decode advances every request of the batch by one decoder position.  The decoding state (cross-attention projections,
    self-attention keys / values) lives with the request, not in the paged KV cache, and adapters are not applied
    (reference: `Seq2SeqLM`, `server/lorax_server/models/seq2seq_lm.py`: padded batches, `past_key_values`, no adapters)."""

    def __init__(self, model, tokenizer=None, cfg: Optional[EngineConfig] = None, model_id: str = ""):
        self.pb = load_pb()
        self.model = model
        self.tokenizer = tokenizer
        self.cfg = cfg or EngineConfig()
        self.model_id = model_id
        self.tp = model.tp
        self.seqs: Dict[int, SeqState] = {}
        self.batches: Dict[int, List[int]] = {}
        self.states: Dict[int, object] = {}
        c = model.config
        self.eos_ids = frozenset([c.eos_token_id])
        self.special_ids = {c.eos_token_id, c.pad_token_id}
        self.lock = threading.Lock()
        self.spec_stats = {"steps": 0, "tokens": 0}
        self.fused_stats = {"one_pass": 0, "two_pass": 0}
        self.medusa_host, self.medusa = {}, {}

    def info(self):
        return self.pb.InfoResponse(requires_padding=True, dtype=str(self.model.dtype).replace("torch.", ""),
                                    device_type=self.model.device.type, block_size=16, speculate=0, supports_generation=True,
                                    supports_embeddings=False, supports_classification=False, chunked_prefill=False,
                                    requires_block_allocator=False, fused_prefill_decode=False)

    def warmup(self, req):
        return self.pb.WarmupResponse(max_supported_total_tokens=max(self.cfg.max_batch_total_tokens or 0, 16 * self.cfg.max_total_tokens))

    def _no_adapters(self, *_a, **_k):
        raise ValueError("adapters are not supported for encoder-decoder models")

    download_adapter = load_adapter = offload_adapter = _no_adapters

    def _drop(self, rid: int):
        self.seqs.pop(rid, None)
        self.states.pop(rid, None)

    def _resort(self):
        pass

    def _step(self, seqs: List[SeqState]):
        """One decoder position for `seqs`; returns the generations and the ids of the finished requests."""
        states = [self.states[s.request_id] for s in seqs]
        logits = self.model.decode_step(states)
        lps_all = torch.log_softmax(logits, -1)
        gid = logits.argmax(-1)
        glp = lps_all.gather(1, gid[:, None])[:, 0]
        ids, lps, alts = self._sample_rows(seqs, logits, gid.tolist(), glp.tolist())
        gens, finished = [], []
        for s, st, tok, lp, alt in zip(seqs, states, ids, lps, alts):
            st.last_token, st.position = int(tok), st.position + 1
            gen, stop = self._emit(s, int(tok), float(lp), alt)
            if gen is not None:
                gens.append(gen)
            if stop:
                finished.append(s.request_id)
        return gens, finished

    def prefill(self, req):
        pb = self.pb
        batch = req.batch
        seqs = []
        for r in batch.requests:
            ids = list(r.tokenized_inputs.ids) if r.HasField("tokenized_inputs") and len(r.tokenized_inputs.ids) else self.tokenize(r.inputs)
            ids = ids[-(r.truncate or self.cfg.max_input_length):]
            params = self._params_from_pb(r.parameters)
            stopping = StoppingCriteria(r.stopping_parameters.max_new_tokens or 1, self.eos_ids, list(r.stopping_parameters.stop_sequences),
                                        r.stopping_parameters.ignore_eos_token)
            s = SeqState(r.id, batch.id, ids, [], 0, params, stopping, Detokenizer(self.tokenizer, []), seed=params.seed)
            if params.schema:
                s.grammar = compile_schema(params.schema, self.tokenizer, self.eos_ids)
            with torch.inference_mode():
                self.states[r.id] = self.model.encode(ids)
            self.seqs[r.id] = s
            seqs.append(s)
        with torch.inference_mode():
            gens, finished = self._step(seqs)
        for rid in finished:
            self._drop(rid)
        live = [s.request_id for s in seqs if s.request_id not in finished]
        resp = pb.PrefillResponse(generations=gens)
        if live:
            self.batches[batch.id] = live
            resp.batch.CopyFrom(self._cached(batch.id))
        return resp

    def decode(self, req):
        pb = self.pb
        bids = [b.id for b in req.batches]
        rids = [r for b in bids for r in self.batches.get(b, [])]
        if not rids:
            raise RuntimeError("all batches of the Decode request are missing from the cache")
        with torch.inference_mode():
            gens, finished = self._step([self.seqs[r] for r in rids])
        for bid in bids:
            self.batches.pop(bid, None)
        for rid in finished:
            self._drop(rid)
        merged = [r for r in rids if r not in finished]
        resp = pb.DecodeResponse(generations=gens)
        if merged:
            self.batches[bids[0]] = merged
            for r in merged:
                self.seqs[r].batch_id = bids[0]
            resp.batch.CopyFrom(self._cached(bids[0]))
        return resp

    def filter_batch(self, req):
        keep = set(req.request_ids)
        for rid in self.batches.get(req.batch_id, []):
            if rid not in keep:
                self._drop(rid)
        self.batches[req.batch_id] = [r for r in self.batches.get(req.batch_id, []) if r in keep]
        return self.pb.FilterBatchResponse(batch=self._cached(req.batch_id))

    def health(self):
        return self.pb.HealthResponse()

    def embed(self, req):
        return self.pb.EmbedResponse(errorMsg="this model does not serve embeddings")

    def classify(self, req):
        return self.pb.ClassifyResponse(errorMsg="this model is not a classifier")


class MllamaRuntime(Seq2SeqRuntime):
    """Shard runtime of Mllama (Llama 3.2 Vision): like the encoder-decoder runtime, a request carries its own state -- here the
    cross-attention keys / values of its images and the self-attention store of the text model (reference: `MllamaCausalLM`,
    `server/lorax_server/models/mllama.py`).  Images arrive as markdown links in the prompt and become one `<|image|>` token each
    (the reference's router does the same with `router/src/config.rs` / `validation.rs:498-638`)."""

    def __init__(self, model, tokenizer=None, cfg: Optional[EngineConfig] = None, model_id: str = ""):
        super().__init__(model, tokenizer, cfg, model_id)
        import collections
        e = model.config.text.eos_token_id
        self.eos_ids = frozenset(e if isinstance(e, (list, tuple)) else [e])
        self.special_ids = set(self.eos_ids) | {model.config.pad_token_id, model.config.image_token_index}
        self._images = collections.OrderedDict()

    def image_token_policy(self) -> dict:
        return {"kind": "one_per_image", "image_token": int(self.model.config.image_token_index)}

    def _image(self, uri: str):
        hit = self._images.get(uri)
        if hit is not None:
            self._images.move_to_end(uri)
            return hit
        from ..models.vlm import load_image
        out = self.model.pixel_values(load_image(uri))
        self._images[uri] = out
        while len(self._images) > 32:
            self._images.popitem(last=False)
        return out

    def tokenize(self, text: str, add_special: bool = True) -> List[int]:
        from ..models.vlm import split_prompt
        parts = split_prompt(text)
        if not any(k == "image" for k, _ in parts):
            return ShardRuntime.tokenize(self, text, add_special)
        ids: List[int] = []
        first = True
        for kind, val in parts:
            if kind == "text":
                ids += ShardRuntime.tokenize(self, val, add_special and first)
            else:
                ids.append(self.model.config.image_token_index)
            first = False
        return ids

    def prefill(self, req):
        from ..models.vlm import split_prompt
        pb = self.pb
        batch = req.batch
        seqs = []
        for r in batch.requests:
            ids = list(r.tokenized_inputs.ids) if r.HasField("tokenized_inputs") and len(r.tokenized_inputs.ids) else self.tokenize(r.inputs)
            uris = [v for k, v in split_prompt(r.inputs) if k == "image"]
            keep = r.truncate or self.cfg.max_input_length
            if len(ids) > keep and uris:
                raise ValueError(f"request {r.id}: a prompt with images cannot be truncated ({len(ids)} tokens, limit {keep})")
            ids = ids[-keep:]
            params = self._params_from_pb(r.parameters)
            stopping = StoppingCriteria(r.stopping_parameters.max_new_tokens or 1, self.eos_ids, list(r.stopping_parameters.stop_sequences),
                                        r.stopping_parameters.ignore_eos_token)
            s = SeqState(r.id, batch.id, ids, [], 0, params, stopping, Detokenizer(self.tokenizer, []), seed=params.seed)
            if params.schema:
                s.grammar = compile_schema(params.schema, self.tokenizer, self.eos_ids)
            with torch.inference_mode():
                self.states[r.id] = self.model.encode(ids, [self._image(u) for u in uris])
            self.seqs[r.id] = s
            seqs.append(s)
        with torch.inference_mode():
            gens, finished = self._step(seqs)
        for rid in finished:
            self._drop(rid)
        live = [s.request_id for s in seqs if s.request_id not in finished]
        resp = pb.PrefillResponse(generations=gens)
        if live:
            self.batches[batch.id] = live
            resp.batch.CopyFrom(self._cached(batch.id))
        return resp


class VlmRuntime(ShardRuntime):
    """Shard runtime of a vision-language model (LLaVA-NeXT): prompts may contain images as markdown, `![](data:image/png;base64,...)`
    or `![](http://...)`.  Tokenisation (which the router delegates to shard 0) replaces every image by as many `<image>` token ids
    as the image yields feature rows; Prefill computes those rows (vision tower, projector, any-resolution packing) and splices
    them into the decoder's input embeddings.  Everything else is the decoder runtime (reference: `VlmCausalLM`,
    `server/lorax_server/models/vlm_causal_lm.py`; image chunking `router/src/validation.rs:498-638`)."""

    def __init__(self, vlm_model, tokenizer=None, cfg: Optional[EngineConfig] = None, model_id: str = "", **kw):
        super().__init__(vlm_model.text, tokenizer, cfg, model_id=model_id, **kw)
        self.vlm = vlm_model
        self._images: "collections.OrderedDict[str, tuple]" = collections.OrderedDict()      # uri -> (tiles, (h, w)), most recent last

    def image_token_policy(self) -> dict:
        c, v = self.vlm.config, self.vlm.config.vision
        return {"kind": "llava_next", "image_token": int(c.image_token_index), "image_size": int(v.image_size), "patch_size": int(v.patch_size),
                "extra_tokens": int(v.extra_tokens), "strategy": c.vision_feature_select_strategy,
                "pinpoints": [[int(h), int(w)] for h, w in c.image_grid_pinpoints]}

    def _image(self, uri: str):
        hit = self._images.get(uri)
        if hit is not None:
            self._images.move_to_end(uri)
            return hit
        from ..models.vlm import load_image
        tiles, size = self.vlm.pixel_values(load_image(uri))
        self._images[uri] = (tiles, size)
        while len(self._images) > 32:
            self._images.popitem(last=False)
        return tiles, size

    def tokenize(self, text: str, add_special: bool = True) -> List[int]:
        from ..models.vlm import split_prompt
        parts = split_prompt(text)
        if not any(k == "image" for k, _ in parts):
            return super().tokenize(text, add_special)
        ids: List[int] = []
        first = True
        for kind, val in parts:
            if kind == "text":
                ids += super().tokenize(val, add_special and first)
            else:
                _, (h, w) = self._image(val)
                ids += [self.vlm.config.image_token_index] * self.vlm.num_image_features(h, w)
            first = False
        return ids

    def tokenize_detailed(self, body: dict) -> list:
        text = body.get("inputs", "")
        if "![](" not in text:
            return super().tokenize_detailed(body)
        return [{"id": i, "text": "<image>" if i == self.vlm.config.image_token_index else self._tok_text(i), "start": 0, "stop": 0}
                for i in self.tokenize(text, body.get("add_special_tokens", True))]

    def _new_sequences(self, batch):
        from ..models.vlm import split_prompt
        seqs, items, chunks = super()._new_sequences(batch)
        tok = self.vlm.config.image_token_index
        ii = ci = 0
        for r in batch.requests:
            ids = list(r.tokenized_inputs.ids) if r.HasField("tokenized_inputs") and len(r.tokenized_inputs.ids) else self.tokenize(r.inputs)
            ids = ids[-(r.truncate or self.cfg.max_input_length):]
            is_chunk = r.HasField("chunk_len") and r.cache_len + r.chunk_len < len(ids)
            item = chunks[ci] if is_chunk else items[ii]
            if is_chunk:
                ci += 1
            else:
                ii += 1
            where = [p for p, t in enumerate(ids) if t == tok]
            if not where:
                continue
            uris = [v for k, v in split_prompt(r.inputs) if k == "image"]
            with torch.inference_mode():
                feats = torch.cat([self.vlm.image_features(*self._image(u)) for u in uris], 0) if uris else None
            if feats is None or feats.shape[0] != len(where):
                raise ValueError(f"request {r.id}: the prompt holds {len(where)} image positions but its images yield "
                                 f"{0 if feats is None else feats.shape[0]} feature rows (was the prompt truncated inside an image?)")
            lo = r.cache_len
            hi = lo + len(item.token_ids)
            sel = [j for j, p in enumerate(where) if lo <= p < hi]
            if sel:
                item.embed_index = [where[j] - lo for j in sel]
                item.embeds = feats[sel[0]: sel[-1] + 1]
        return seqs, items, chunks


class EncoderRuntime:
    """Shard runtime of an embedding / token-classification model (BERT, RoBERTa, DistilBERT): `Embed` and `Classify`
    are served, every generation RPC answers with an error (reference: `FlashBert.embed/classify`,
    `server/lorax_server/models/flash_bert.py:186-218`)."""

    chat_template: Optional[str] = None
    bos_token: str = ""
    eos_token: str = ""

    def __init__(self, model, tokenizer=None, cfg: Optional[EngineConfig] = None, model_id: str = ""):
        self.pb = load_pb()
        self.model = model
        self.tokenizer = tokenizer
        self.cfg = cfg or EngineConfig()
        self.model_id = model_id
        self.lock = threading.Lock()

    def info(self):
        return self.pb.InfoResponse(requires_padding=False, dtype=str(self.model.dtype).replace("torch.", ""),
                                    device_type=self.model.device.type, block_size=self.cfg.block_size, speculate=0,
                                    supports_generation=False, supports_embeddings=True,
                                    supports_classification=self.model.cls_w is not None, chunked_prefill=False,
                                    requires_block_allocator=False)

    def health(self):
        return self.pb.HealthResponse()

    def warmup(self, req):
        return self.pb.WarmupResponse(max_supported_total_tokens=self.cfg.max_batch_prefill_tokens)

    def tokenize(self, text: str, add_special: bool = True) -> List[int]:
        if self.tokenizer is None:
            return [int(x) for x in text.split()] if text.replace(" ", "").isdigit() else [ord(ch) % self.model.config.vocab_size for ch in text]
        return self.tokenizer.encode(text, add_special_tokens=add_special).ids

    router_tokenizer_json = ShardRuntime.router_tokenizer_json

    def tokenize_detailed(self, body: dict) -> list:
        if self.tokenizer is not None:          # character offsets: the router turns token classes into entity spans with them
            enc = self.tokenizer.encode(body.get("inputs", ""), add_special_tokens=body.get("add_special_tokens", True))
            return [{"id": i, "text": t, "start": o[0], "stop": o[1]} for i, t, o in zip(enc.ids, enc.tokens, enc.offsets)]
        return [{"id": i, "text": str(i), "start": 0, "stop": 0} for i in self.tokenize(body.get("inputs", ""))]

    def apply_chat_template(self, body: dict) -> str:
        raise ValueError("an embedding model has no chat template")

    def _ids(self, r) -> List[int]:
        ids = list(r.tokenized_inputs.ids) if r.HasField("tokenized_inputs") and len(r.tokenized_inputs.ids) else self.tokenize(r.inputs)
        if r.truncate:
            ids = ids[: r.truncate]
        return ids

    def embed(self, req):
        try:
            with self.lock:
                vecs = self.model.embed([self._ids(r) for r in req.batch.requests])
            return self.pb.EmbedResponse(embeddings=[self.pb.Embedding(request_id=r.id, values=v) for r, v in zip(req.batch.requests, vecs)])
        except Exception as e:      # surfaced to the router as the RPC's error string, as the reference does
            return self.pb.EmbedResponse(errorMsg=str(e))

    def classify(self, req):
        try:
            with self.lock:
                labels, scores = self.model.classify([self._ids(r) for r in req.batch.requests])
            return self.pb.ClassifyResponse(classify_prediction_lists=[
                self.pb.ClassifyPredictionList(request_id=r.id, predictions=l, scores=sc) for r, l, sc in zip(req.batch.requests, labels, scores)])
        except Exception as e:
            return self.pb.ClassifyResponse(errorMsg=str(e))

    def _no_generation(self, *_a, **_k):
        raise ValueError("this model serves embeddings / classification, not text generation")

    prefill = decode = filter_batch = download_adapter = load_adapter = offload_adapter = _no_generation

    def clear_cache(self, req):
        return self.pb.ClearCacheResponse()


def _checkpoint_kv_scales(w, mc):
    """Per-layer (k scale, v scale) of an fp8 KV cache: `...self_attn.k_scale` / `v_scale` (or the older single `kv_scale`) where
    the checkpoint carries them (the reference reads the same tensors, server/lorax_server/models/flash_causal_lm.py:1240-1270),
    else 1."""
    out = []
    for li in range(mc.num_hidden_layers):
        ks = vs = 1.0
        for pre in ("model.layers", "transformer.h"):
            base = f"{pre}.{li}.self_attn"
            try:
                if w.has_tensor(f"{base}.k_scale"):
                    ks = float(w.get_tensor(f"{base}.k_scale").float().item())
                    vs = float(w.get_tensor(f"{base}.v_scale").float().item())
                elif w.has_tensor(f"{base}.kv_scale"):
                    ks = vs = float(w.get_tensor(f"{base}.kv_scale").float().item())
            except Exception:
                pass
        out.append((ks, vs))
    return out


def build_runtime(model_id: str, cfg: EngineConfig, tp: Optional[TensorParallel] = None, dtype: Optional[torch.dtype] = None,
                  device: Optional[str] = None, source: str = "hub", revision: Optional[str] = None, **kw) -> ShardRuntime:
    tp = tp or TensorParallel.init_from_env()
    model_dir = resolve_model(model_id, source, revision)
    dev = torch.device(device) if device else (tp.device or torch.device("cpu"))
    if dtype is None:
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    with open(os.path.join(model_dir, "config.json")) as f:
        raw_cfg = json.load(f)
    from ..models.encoder import ENCODER_TYPES, EncoderConfig, EncoderModel
    from ..models.seq2seq import SEQ2SEQ_TYPES, Seq2SeqConfig, Seq2SeqModel
    if raw_cfg.get("model_type") in SEQ2SEQ_TYPES:
        if tp.world_size > 1:
            raise ValueError("encoder-decoder models are served on one shard")
        w = Weights(weight_files(model_dir), device="cpu", dtype=dtype)
        s2s = Seq2SeqModel.from_weights(Seq2SeqConfig.from_dict(raw_cfg), w, dev, dtype)
        return Seq2SeqRuntime(s2s, load_tokenizer(model_dir), cfg, model_id=model_id)
    if raw_cfg.get("model_type") == "mllama":
        if tp.world_size > 1:
            raise ValueError("mllama is served on one shard")
        from ..models.mllama import MllamaConfig, MllamaModel
        w = Weights(weight_files(model_dir), device="cpu", dtype=dtype)
        mm = MllamaModel.from_weights(MllamaConfig.from_dict(raw_cfg), w, dev, dtype)
        return MllamaRuntime(mm, load_tokenizer(model_dir), cfg, model_id=model_id)
    from ..models.vlm import VLM_TYPES, LlavaNextConfig, LlavaNextModel
    if raw_cfg.get("model_type") in VLM_TYPES:
        vcfg = LlavaNextConfig.from_dict(raw_cfg)
        w = Weights(weight_files(model_dir), device="cpu", dtype=dtype, rank=tp.rank, world_size=tp.world_size)
        tp.barrier()
        vm = LlavaNextModel.from_weights(vcfg, w, dev, dtype, tp, max_positions=min(vcfg.text.max_position_embeddings,
                                                                                    max(cfg.max_total_tokens + 64, 2048)))
        kw.pop("quantize", None)
        return VlmRuntime(vm, load_tokenizer(model_dir), cfg, model_id=model_id, **kw)
    if raw_cfg.get("model_type") in ENCODER_TYPES:
        w = Weights(weight_files(model_dir), device="cpu", dtype=dtype)
        enc = EncoderModel.from_weights(EncoderConfig.from_dict(raw_cfg), w, dev, dtype)
        return EncoderRuntime(enc, load_tokenizer(model_dir), cfg, model_id=model_id)
    mc = ModelConfig.from_pretrained(model_dir)
    w = Weights(weight_files(model_dir), device="cpu", dtype=dtype, rank=tp.rank, world_size=tp.world_size)
    quantize = kw.pop("quantize", None) or cfg.quantize
    # a GPTQ / AWQ checkpoint: its packed layers are served as they are unless another scheme is asked for
    w.quant = checkpoint_quantization(model_dir, raw_cfg)
    w.keep_packed = quantize in (None, "gptq", "awq")
    merge_id = kw.pop("merge_adapter", None)
    if merge_id:
        # one adapter folded into the base weights while they load; requests then need no adapter id for it
        from ..utils.weights import MergedWeights
        lcfg, mm = load_peft_adapter(resolve_adapter(merge_id, kw.pop("merge_adapter_source", "hub")))
        w = MergedWeights(w, lcfg, mm)
    tp.barrier()
    model = DecoderModel.from_weights(mc, w, dev, dtype, tp, max_positions=min(mc.max_position_embeddings, max(cfg.max_total_tokens + 64, 2048)))
    qc = getattr(mc, "quantization_config", None) or {}
    if quantize is None and isinstance(qc, dict) and qc.get("quant_method") == "fp8":
        quantize = "fp8"
    if quantize == "fp8-kv":
        # block-scaled fp8 weights and an e4m3 KV cache (per-layer k / v scales from the checkpoint where it has them, else 1)
        cfg.kv_cache_dtype = "fp8"
        quantize = "fp8"
    if cfg.kv_cache_dtype == "fp8":
        model.kv_scales = _checkpoint_kv_scales(w, mc)
    if quantize in ("gptq", "awq") and w.quant is None:
        raise ValueError(f"--quantize {quantize} needs a {quantize} checkpoint (no quantization_config / quantize_config.json found)")
    if quantize is not None and not (quantize in ("gptq", "awq") and model.quantized):
        model.quantize(quantize)           # on-load quantisation of whatever is still dense
    if tp.world_size > 1 and dev.type == "cuda" and os.environ.get("LORAX_FUSED_COLLECTIVES", "1") != "0":
        # in-kernel NVLink collectives (fused GEMM + all-reduce for small batches, peer-read embedding, arg-max exchange);
        # every rank takes the same branch, NCCL stays as the path for everything else
        try:
            from ..parallel import fused
            fused.enable(tp, model)
        except Exception as e:          # no peer access / symmetric memory: NCCL only
            print(json.dumps({"level": "WARN", "message": f"fused NVLink collectives unavailable: {e}"}), flush=True)
    tp.barrier()
    tok = load_tokenizer(model_dir)
    rt = ShardRuntime(model, tok, cfg, model_id=model_id, **kw)
    # the launcher's --tokenizer-config-path (router/src/main.rs:196-363 of the reference reads the same override)
    tc_path = os.environ.get("TOKENIZER_CONFIG_PATH") or os.path.join(model_dir, "tokenizer_config.json")
    if os.path.exists(tc_path):
        with open(tc_path) as f:
            tc = json.load(f)
        rt.chat_template = tc.get("chat_template")

        def _tok(v):
            return v.get("content", "") if isinstance(v, dict) else (v or "")
        rt.bos_token, rt.eos_token = _tok(tc.get("bos_token")), _tok(tc.get("eos_token"))
    gc_path = os.path.join(model_dir, "generation_config.json")
    if os.path.exists(gc_path):
        with open(gc_path) as f:
            eos = json.load(f).get("eos_token_id")
        if eos is not None:
            rt.eos_ids = frozenset(eos if isinstance(eos, list) else [eos])
            rt.special_ids |= set(rt.eos_ids)
    return rt
