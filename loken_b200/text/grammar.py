"""Structured outputs: a request's JSON schema, regular expression or grammar becomes a matcher
that says, before every token, which tokens keep the output inside the language.

The reference wires `llguidance` to its tokenizer the same way
(`src/inference/engine/llm_engine/mod.rs:1705-1760`, `grammar_factory_for`): JSON schema, Lark,
GBNF and regex sources; the mask is applied to the logits before the sampler and the request ends
when the matcher reaches an accepting stop.  Request spellings accepted by `spec_from_request`:
OpenAI `response_format` (`json_object`, `json_schema`), vLLM `guided_json`, `guided_regex`,
`guided_grammar`, `guided_choice` and `structured_outputs`.
"""
from __future__ import annotations

import json
from typing import List, Optional, Tuple

import numpy as np


class GrammarError(ValueError):
    pass


def spec_from_request(body: dict) -> Optional[Tuple[str, object]]:
    """-> (kind, source) with kind in json_schema | regex | lark | choice, or None."""
    so = body.get("structured_outputs") or {}
    rf = body.get("response_format") or {}
    if rf.get("type") == "json_schema":
        js = rf.get("json_schema") or {}
        return "json_schema", js.get("schema", js)
    if rf.get("type") == "json_object":
        return "json_schema", {"type": "object"}
    for key, kind in (("guided_json", "json_schema"), ("json", "json_schema"), ("guided_regex", "regex"),
                      ("regex", "regex"), ("guided_grammar", "lark"), ("grammar", "lark"),
                      ("guided_choice", "choice"), ("choice", "choice")):
        src = body.get(key) if key.startswith("guided_") else so.get(key)
        if src is not None:
            if kind == "json_schema" and isinstance(src, str):
                src = json.loads(src)
            if kind == "json_schema":
                src = _json_options(src, so, body)
            return kind, src
    if so.get("json_object"):
        return "json_schema", _json_options({"type": "object"}, so, body)
    return None


def _json_options(schema, so: dict, body: dict):
    """vLLM's options of a JSON constraint, as the matcher's own schema annotations: `disable_any_whitespace`
    (no whitespace between tokens of the JSON), `whitespace_pattern` / `guided_whitespace_pattern` (a regular
    expression for what may stand there) and `disable_additional_properties` (every object of the schema that
    does not say otherwise is closed)."""
    if not isinstance(schema, dict):
        return schema
    ws = so.get("whitespace_pattern") or body.get("guided_whitespace_pattern")
    if not (so.get("disable_any_whitespace") or so.get("disable_additional_properties") or ws):
        return schema
    schema = json.loads(json.dumps(schema))              # the request's own object is left as sent
    xg = dict(schema.get("x-guidance") or {})
    if so.get("disable_any_whitespace"):
        xg["whitespace_flexible"] = False
    if ws:
        xg["whitespace_pattern"] = str(ws)
    if xg:
        schema["x-guidance"] = xg
    if so.get("disable_additional_properties"):
        def close(node):
            if isinstance(node, dict):
                if (node.get("type") == "object" or "properties" in node) and "additionalProperties" not in node:
                    node["additionalProperties"] = False
                for v in node.values():
                    close(v)
            elif isinstance(node, list):
                for v in node:
                    close(v)
        close(schema)
    return schema


class _VocabAdapter:
    """What llguidance needs to know about a tokenizer: token bytes, end / begin ids, encode."""

    def __init__(self, tk):
        self.tk = tk
        n = tk.vocab_size
        self.eos_token_id = tk.eos_id if tk.eos_id is not None else 0
        self.bos_token_id = tk.bos_id
        toks: List[bytes] = []
        special = []
        for i in range(n):
            plain = tk.decode_bytes([i], skip_special=True)
            if plain:
                toks.append(plain)
            else:
                raw = tk.decode_bytes([i], skip_special=False)
                toks.append(raw if raw else f"<|unused_{i}|>".encode())
                special.append(i)
        self.tokens = toks
        self.special_token_ids = special

    def __call__(self, s):
        if isinstance(s, bytes):
            s = s.decode("utf-8", "replace")
        return self.tk.encode(s, add_special=False)


_ll_cache = {}


def ll_tokenizer(tk):
    import llguidance

    key = id(tk)
    if key not in _ll_cache:
        _ll_cache[key] = llguidance.LLTokenizer(llguidance.TokenizerWrapper(_VocabAdapter(tk)))
    return _ll_cache[key]


class GrammarSession:
    """One request's matcher."""

    def __init__(self, tokenizer, kind: str, source):
        import llguidance

        self.vocab = tokenizer.vocab_size
        self.words = (self.vocab + 31) // 32
        try:
            if kind == "json_schema":
                g = llguidance.LLMatcher.grammar_from_json_schema(json.dumps(source))
            elif kind == "regex":
                g = llguidance.LLMatcher.grammar_from_regex(str(source))
            elif kind == "choice":
                import re

                g = llguidance.LLMatcher.grammar_from_regex("|".join(re.escape(str(c)) for c in source))
            elif kind == "lark":
                src = str(source)
                if "::=" in src:
                    src = llguidance.gbnf_to_lark(src)
                g = llguidance.LLMatcher.grammar_from_lark(src)
            else:
                raise GrammarError(f"unknown grammar kind {kind}")
            self.m = llguidance.LLMatcher(ll_tokenizer(tokenizer), g)
        except GrammarError:
            raise
        except Exception as e:
            raise GrammarError(f"cannot compile the {kind} constraint: {e}")
        err = self.m.get_error()
        if err:
            raise GrammarError(f"cannot compile the {kind} constraint: {err}")

    def mask(self) -> np.ndarray:
        """int32 [words]: bit t set = token t keeps the output valid."""
        import llguidance.numpy as lln

        bm = lln.allocate_token_bitmask(1, self.vocab)
        lln.fill_next_token_bitmask(self.m, bm, 0)
        return bm[0]

    def accept(self, token: int) -> bool:
        return bool(self.m.consume_token(int(token)))

    def done(self) -> bool:
        return bool(self.m.is_stopped())

    def rollback(self, n: int):
        """Forgets the last `n` accepted tokens (rows of a speculative step that were only looked at)."""
        if n > 0 and not self.m.rollback(int(n)):
            raise GrammarError(f"the matcher cannot go back {n} tokens: {self.m.get_error()}")

    def rows_for_drafts(self, drafts) -> tuple:
        """Masks for the verify rows of a speculative step: row i is sampled after drafts[:i], so it carries the
        mask of the matcher's state there.  Drafts stop being usable at the first token the language refuses,
        and at a token that completes it (the row sampling that token ends the request, nothing follows it).
        Returns (masks, the usable drafts); the matcher is left where it was."""
        masks, used = [self.mask()], 0
        try:
            for t in drafts:
                t = int(t)
                cur = masks[-1]
                if t < 0 or (t >> 5) >= len(cur) or not (int(cur[t >> 5]) >> (t & 31)) & 1:
                    break
                if not self.m.consume_token(t):
                    break
                used += 1
                if self.m.is_stopped():
                    used -= 1
                    self.rollback(1)
                    break
                masks.append(self.mask())
        finally:
            keep = len(masks) - 1
            self.rollback(used)
        return masks[:keep + 1], list(drafts[:keep])
