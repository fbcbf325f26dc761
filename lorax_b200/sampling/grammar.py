"""Structured output: constrain generation to JSON that follows a JSON schema.

The reference compiles the schema to a regex FSM with Outlines and masks logits with the FSM's allowed tokens
(`server/lorax_server/utils/logits_process.py:464-601`).  Outlines is not available here, so this module carries
its own incremental validator: `JsonPrefix` decides whether a string is a prefix of a JSON document that can
still satisfy the schema, and `SchemaGrammar` turns that into per-step token masks (a token is allowed when
appending its text keeps the prefix viable; EOS is allowed exactly when the document is complete).

Supported schema subset: type object / array / string / number / integer / boolean / null, properties, required,
additionalProperties (false), items, enum and const of scalars, anyOf.  Whitespace between tokens is allowed.
"""

from __future__ import annotations

import json
from typing import Dict, List, Optional, Sequence, Tuple


class _Fail(Exception):
    pass


class _Incomplete(Exception):
    pass


class JsonPrefix:
    """Recursive-descent check of a (possibly truncated) JSON text against a schema.

    `status(text)` -> "complete" | "prefix" | "invalid".
    """

    def __init__(self, schema: Optional[dict]):
        self.schema = schema if isinstance(schema, dict) else {}

    def status(self, text: str) -> str:
        self.t = text
        self.n = len(text)
        try:
            i = self._ws(0)
            i = self._value(i, self.schema)
            i = self._ws(i, at_end_ok=True)
            if i < self.n:
                return "invalid"
            return "complete"
        except _Incomplete:
            return "prefix"
        except _Fail:
            return "invalid"

    # ---- helpers: every method returns the index after what it parsed, raises _Incomplete at end of text
    def _ws(self, i, at_end_ok=False):
        while i < self.n and self.t[i] in " \n\t\r":
            i += 1
        return i

    def _need(self, i):
        if i >= self.n:
            raise _Incomplete()

    def _types(self, schema) -> Optional[set]:
        t = schema.get("type")
        if t is None:
            return None
        return set(t) if isinstance(t, list) else {t}

    def _value(self, i, schema) -> int:
        self._need(i)
        if "anyOf" in schema or "oneOf" in schema:
            alts = schema.get("anyOf") or schema.get("oneOf")
            incomplete = False
            for alt in alts:
                try:
                    return self._value(i, alt)
                except _Incomplete:
                    incomplete = True
                except _Fail:
                    continue
            if incomplete:
                raise _Incomplete()
            raise _Fail()
        if "const" in schema:
            return self._literal_choice(i, [schema["const"]])
        if "enum" in schema:
            return self._literal_choice(i, schema["enum"])
        types = self._types(schema)
        c = self.t[i]
        ok = lambda name: types is None or name in types
        if c == "{" and ok("object"):
            return self._object(i, schema)
        if c == "[" and ok("array"):
            return self._array(i, schema)
        if c == '"' and ok("string"):
            return self._string(i)
        if (c == "-" or c.isdigit()) and (ok("number") or ok("integer")):
            return self._number(i, integer=(types is not None and "number" not in types))
        if c in "tf" and ok("boolean"):
            return self._word(i, ["true", "false"])
        if c == "n" and ok("null"):
            return self._word(i, ["null"])
        raise _Fail()

    def _word(self, i, words):
        rest = self.t[i:]
        for w in words:
            if rest.startswith(w):
                return i + len(w)
            if w.startswith(rest):
                raise _Incomplete()
        raise _Fail()

    def _literal_choice(self, i, values):
        rest = self.t[i:]
        incomplete = False
        for v in values:
            s = json.dumps(v)
            if rest.startswith(s):
                return i + len(s)
            if s.startswith(rest):
                incomplete = True
        if incomplete:
            raise _Incomplete()
        raise _Fail()

    def _string(self, i) -> int:
        i += 1
        while True:
            self._need(i)
            c = self.t[i]
            if c == '"':
                return i + 1
            if c == "\\":
                self._need(i + 1)
                e = self.t[i + 1]
                if e == "u":
                    for k in range(4):
                        self._need(i + 2 + k)
                        if self.t[i + 2 + k] not in "0123456789abcdefABCDEF":
                            raise _Fail()
                    i += 6
                    continue
                if e not in '"\\/bfnrt':
                    raise _Fail()
                i += 2
                continue
            if ord(c) < 0x20:
                raise _Fail()
            i += 1

    def _number(self, i, integer=False) -> int:
        j = i
        if self.t[j] == "-":
            j += 1
            self._need(j)
        if not self.t[j].isdigit():
            raise _Fail()
        if self.t[j] == "0":
            j += 1
        else:
            while j < self.n and self.t[j].isdigit():
                j += 1
        if j >= self.n:
            raise _Incomplete()          # more digits may follow
        if not integer and self.t[j] == ".":
            j += 1
            self._need(j)
            if not self.t[j].isdigit():
                raise _Fail()
            while j < self.n and self.t[j].isdigit():
                j += 1
            if j >= self.n:
                raise _Incomplete()
        if not integer and self.t[j] in "eE":
            j += 1
            self._need(j)
            if self.t[j] in "+-":
                j += 1
                self._need(j)
            if not self.t[j].isdigit():
                raise _Fail()
            while j < self.n and self.t[j].isdigit():
                j += 1
            if j >= self.n:
                raise _Incomplete()
        return j

    def _array(self, i, schema) -> int:
        items = schema.get("items", {}) if isinstance(schema.get("items", {}), dict) else {}
        i = self._ws(i + 1)
        self._need(i)
        if self.t[i] == "]":
            return i + 1
        while True:
            i = self._value(i, items)
            i = self._ws(i)
            self._need(i)
            if self.t[i] == ",":
                i = self._ws(i + 1)
                self._need(i)
                continue
            if self.t[i] == "]":
                return i + 1
            raise _Fail()

    def _object(self, i, schema) -> int:
        props: Dict[str, dict] = schema.get("properties", {}) or {}
        required = list(schema.get("required", []) or [])
        closed = schema.get("additionalProperties", None) is False or (bool(props) and "additionalProperties" not in schema)
        seen: List[str] = []
        i = self._ws(i + 1)
        self._need(i)
        if self.t[i] == "}":
            if any(r not in seen for r in required):
                raise _Fail()
            return i + 1
        while True:
            self._need(i)
            if self.t[i] != '"':
                raise _Fail()
            # key: with a closed property set, the key must be (a prefix of) an unseen property name
            if closed:
                cands = [k for k in props if k not in seen]
                rest = self.t[i:]
                match = None
                incomplete = False
                for k in cands:
                    s = json.dumps(k)
                    if rest.startswith(s):
                        match = k
                        break
                    if s.startswith(rest):
                        incomplete = True
                if match is None:
                    if incomplete:
                        raise _Incomplete()
                    raise _Fail()
                key = match
                i += len(json.dumps(key))
            else:
                j = self._string(i)
                key = json.loads(self.t[i:j])
                i = j
            seen.append(key)
            i = self._ws(i)
            self._need(i)
            if self.t[i] != ":":
                raise _Fail()
            i = self._ws(i + 1)
            i = self._value(i, props.get(key, {}))
            i = self._ws(i)
            self._need(i)
            if self.t[i] == ",":
                if closed and all(k in seen for k in props):
                    raise _Fail()
                i = self._ws(i + 1)
                continue
            if self.t[i] == "}":
                if any(r not in seen for r in required):
                    raise _Fail()
                return i + 1
            raise _Fail()


class SchemaGrammar:
    def __init__(self, schema: dict, vocab_texts: Sequence[str], eos_ids: Sequence[int]):
        self.checker = JsonPrefix(schema)
        self.vocab = list(vocab_texts)
        self.eos_ids = [int(e) for e in eos_ids]
        self.text = ""
        self.done = False
        self._cache: Dict[str, List[int]] = {}

    def allowed_tokens(self) -> Optional[List[int]]:
        if self.done:
            return self.eos_ids or None
        key = self.text[-256:] if len(self.text) > 256 else self.text
        cached = self._cache.get(self.text)
        if cached is not None:
            return cached
        out = []
        status_now = self.checker.status(self.text) if self.text else "prefix"
        if status_now == "complete":
            out += self.eos_ids
        for tid, piece in enumerate(self.vocab):
            if not piece:
                continue
            if self.checker.status(self.text + piece) != "invalid":
                out.append(tid)
        if not out:
            out = self.eos_ids or list(range(len(self.vocab)))
        self._cache[self.text] = out
        return out

    def advance(self, token_id: int):
        if token_id in self.eos_ids:
            self.done = True
            return
        if 0 <= token_id < len(self.vocab):
            self.text += self.vocab[token_id]
        if self.checker.status(self.text) == "complete" and self.text.rstrip().endswith(("}", "]")):
            self.done = True


_vocab_cache: Dict[int, List[str]] = {}


def vocab_texts(tokenizer) -> List[str]:
    key = id(tokenizer)
    if key not in _vocab_cache:
        n = tokenizer.get_vocab_size()
        # decode every id in the context of a leading token so that leading-space pieces keep their space
        _vocab_cache[key] = [tokenizer.decode([i], skip_special_tokens=True) for i in range(n)]
    return _vocab_cache[key]


def compile_schema(schema_json: str, tokenizer, eos_ids) -> Optional[SchemaGrammar]:
    if tokenizer is None:
        return None
    schema = json.loads(schema_json) if isinstance(schema_json, str) else schema_json
    return SchemaGrammar(schema, vocab_texts(tokenizer), list(eos_ids))
