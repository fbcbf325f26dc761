"""ctypes bindings of ``_lx_host.so``: the C++ router's block allocator, radix trie, adapter queues and the
in-process Infer harness that runs against a fake shard (used by the tests and by tools that want the exact
scheduling behaviour of the router without starting it)."""

from __future__ import annotations

import ctypes
import json
from ctypes import c_char_p, c_double, c_int, c_uint32, c_uint64, c_void_p
from pathlib import Path
from typing import List, Optional, Sequence

_PKG = Path(__file__).resolve().parent.parent
_LIB = _PKG / "_lx_host.so"
_lib = None


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB.exists():
        from lorax_b200.csrc import build
        build.build_host()
    lib = ctypes.CDLL(str(_LIB))
    U32P = ctypes.POINTER(c_uint32)
    sig = {
        "lx_alloc_new": ([c_uint32, c_uint32, c_int, c_int], c_void_p),
        "lx_alloc_delete": ([c_void_p], None),
        "lx_alloc_free_blocks": ([c_void_p], c_uint64),
        "lx_alloc_allocate": ([c_void_p, c_uint32, c_uint32, U32P, c_uint32], c_void_p),
        "lx_allocation_num_blocks": ([c_void_p], c_uint32),
        "lx_allocation_prefix_len": ([c_void_p], c_uint32),
        "lx_allocation_num_slots": ([c_void_p], c_uint32),
        "lx_allocation_blocks": ([c_void_p, U32P], None),
        "lx_allocation_slots": ([c_void_p, U32P], None),
        "lx_alloc_free": ([c_void_p, c_void_p, c_uint32, U32P, c_uint32], None),
        "lx_json_roundtrip": ([c_char_p], c_char_p),
        "lx_queues_script": ([c_int, c_double, c_char_p], c_char_p),
        "lx_infer_fake_run": ([c_char_p, c_int, c_int, c_uint32, c_int], c_char_p),
        "lx_tokenizer_load": ([c_char_p, c_int, c_char_p, c_int], c_void_p),
        "lx_tokenizer_free": ([c_void_p], None),
        "lx_tokenizer_encode": ([c_void_p, c_char_p, ctypes.c_size_t, c_int, U32P, ctypes.c_size_t], ctypes.c_long),
        "lx_tokenizer_error": ([c_void_p], c_char_p),
        "lx_unicode_normalize": ([c_char_p, c_char_p], c_char_p),
        "lx_regex_find_all": ([c_char_p, c_char_p], c_char_p),
        "lx_encoder_batcher_fake_run": ([c_int, c_int], c_char_p),
        "lx_chat_render": ([c_char_p], c_char_p),
        "lx_image_token_count": ([c_char_p, c_char_p], ctypes.c_long),
        "lx_split_image_prompt": ([c_char_p], c_char_p),
    }
    for name, (args, res) in sig.items():
        f = getattr(lib, name)
        f.argtypes, f.restype = args, res
    _lib = lib
    return lib


def _arr(xs: Optional[Sequence[int]]):
    if xs is None:
        return None, 0
    a = (c_uint32 * len(xs))(*xs)
    return a, len(xs)


class Allocation:
    def __init__(self, handle, lib):
        self._h = handle
        n = lib.lx_allocation_num_blocks(handle)
        b = (c_uint32 * n)()
        lib.lx_allocation_blocks(handle, b)
        self.blocks: List[int] = list(b)
        ns = lib.lx_allocation_num_slots(handle)
        s = (c_uint32 * ns)()
        lib.lx_allocation_slots(handle, s)
        self.slots: List[int] = list(s)
        self.prefix_len: int = lib.lx_allocation_prefix_len(handle)


class BlockAllocator:
    """The router's allocator (free list, or radix trie when `prefix_caching`)."""

    def __init__(self, num_blocks: int, block_size: int, window: Optional[int] = None, prefix_caching: bool = False):
        self._lib = load()
        self._a = self._lib.lx_alloc_new(num_blocks, block_size, window or 0, int(prefix_caching))

    def __del__(self):
        if getattr(self, "_a", None):
            self._lib.lx_alloc_delete(self._a)
            self._a = None

    @property
    def free_blocks(self) -> int:
        return self._lib.lx_alloc_free_blocks(self._a)

    def allocate(self, tokens: int, adapter_index: int = 0, prompt: Optional[Sequence[int]] = None) -> Optional[Allocation]:
        a, n = _arr(prompt)
        h = self._lib.lx_alloc_allocate(self._a, adapter_index, tokens, a, n)
        return Allocation(h, self._lib) if h else None

    def free(self, alloc: Allocation, adapter_index: int = 0, all_tokens: Optional[Sequence[int]] = None):
        a, n = _arr(all_tokens)
        self._lib.lx_alloc_free(self._a, alloc._h, adapter_index, a, n)
        alloc._h = None


def json_roundtrip(s: str) -> str:
    return load().lx_json_roundtrip(s.encode()).decode()


def queues_script(ops, max_active: int = 2, cycle_s: float = 2.0):
    return json.loads(load().lx_queues_script(max_active, cycle_s, json.dumps(ops).encode()).decode())


def infer_fake_run(requests, max_active_adapters: int = 8, fail_decode_after: int = -1, num_blocks: int = 4096,
                   prefix_caching: bool = False):
    out = load().lx_infer_fake_run(json.dumps(requests).encode(), max_active_adapters, fail_decode_after, num_blocks, int(prefix_caching))
    return json.loads(out.decode())


class RouterTokenizer:
    """The router's C++ tokenizer (``csrc/host/tokenizer.hpp``) on a pool of worker threads.  Raises ``ValueError`` with the
    reason when the tokenizer file uses a component it does not implement (the router then asks shard 0 instead)."""

    def __init__(self, path: str, workers: int = 2):
        self._lib = load()
        err = ctypes.create_string_buffer(512)
        self._h = self._lib.lx_tokenizer_load(str(path).encode(), workers, err, len(err))
        if not self._h:
            raise ValueError(err.value.decode(errors="replace"))

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        raw = text.encode("utf-8", errors="replace")
        cap = max(16, len(raw) + 16)
        buf = (c_uint32 * cap)()
        n = self._lib.lx_tokenizer_encode(self._h, raw, len(raw), int(add_special_tokens), buf, cap)
        if n < 0:
            raise ValueError(self._lib.lx_tokenizer_error(self._h).decode(errors="replace"))
        if n > cap:                                  # more ids than bytes: only with long special-token templates
            buf = (c_uint32 * n)()
            n = self._lib.lx_tokenizer_encode(self._h, raw, len(raw), int(add_special_tokens), buf, n)
        return list(buf[:n])

    def close(self):
        if self._h:
            self._lib.lx_tokenizer_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def unicode_normalize(text: str, form: str) -> str:
    return load().lx_unicode_normalize(text.encode(), form.encode()).decode()


def regex_find_all(pattern: str, text: str) -> List[List[int]]:
    """Matches of the router's regex engine as [begin, end) code point offsets; ``ValueError`` for a pattern outside its subset."""
    out = load().lx_regex_find_all(pattern.encode(), text.encode()).decode()
    if out.startswith("error: "):
        raise ValueError(out[7:])
    return json.loads(out)


def encoder_batcher_fake_run(threads: int, each: int) -> dict:
    """Concurrent embed / classify inputs through the router's encoder batcher against the fake shard (see capi.cpp)."""
    return json.loads(load().lx_encoder_batcher_fake_run(threads, each).decode())


def chat_render(template: str, messages, bos_token: str = "", eos_token: str = "", **extra) -> dict:
    """The router's chat template interpreter: {"text"}, {"error"} or {"unsupported"} (see capi.cpp)."""
    req = dict(template=template, messages=messages, bos_token=bos_token, eos_token=eos_token, **extra)
    return json.loads(load().lx_chat_render(json.dumps(req).encode()).decode())


def image_token_count(policy: dict, uri: str) -> int:
    """Feature tokens the router counts for an image reference; -1 when it leaves the image to the shard."""
    return load().lx_image_token_count(json.dumps(policy).encode(), uri.encode())


def split_image_prompt(text: str):
    """The router's cut of a prompt at its `![](uri)` references: [("text" | "image", value), ...]."""
    return [("image" if is_img else "text", v) for is_img, v in json.loads(load().lx_split_image_prompt(text.encode()).decode())]
