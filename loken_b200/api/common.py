"""Pieces every API dialect shares: the model registry, request -> GenerationParams mapping with
the reference's bounds, API-key auth, the token-bucket rate limiter, the priority request gate,
request ids and error envelopes.

Bounds and defaults follow `src/api/handlers/sampling.rs:10-45`, `:380-395`: max_tokens <= 131072,
<= 4 stop sequences of <= 256 chars, top_logprobs <= 20, n <= 16, <= 4096 messages, <= 1 Mi chars;
frequency + presence penalties are summed, clamped to [-2, 2] and mapped to 1 + pen; an explicit
repeat/repetition penalty wins.  The gate orders Batch < Interactive < Fim (`src/api/gate.rs:21-50`);
a full queue answers 503 with Retry-After from queue depth x mean slot time, the rate limiter 429
with Retry-After (`docs/API.md:406-413`).
"""
from __future__ import annotations

import heapq
import itertools
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..engine.llm import LLM, GenerationParams
from ..serve.params import ParamError, openai_penalty

MAX_MESSAGES = 4096
MAX_CHARS = 1 << 20


class ApiError(Exception):
    def __init__(self, status: int, message: str, kind: str = "invalid_request_error", code: Optional[str] = None,
                 retry_after: Optional[float] = None):
        super().__init__(message)
        self.status, self.message, self.kind, self.code, self.retry_after = status, message, kind, code, retry_after


class ModelRegistry:
    """Loaded models by id.  A request names a model; an unknown name falls back to the default
    model when `strict` is off (one-model servers accept any name, like the reference's
    single-model mode)."""

    def __init__(self, strict: bool = False):
        self.models: Dict[str, LLM] = {}
        self.aliases: Dict[str, str] = {}       # second names of loaded models (/api/copy, /api/create)
        self.last_used: Dict[str, float] = {}   # model id -> time of the last request that named it
        self.default: Optional[str] = None
        self.strict = strict
        self.lock = threading.Lock()

    on_missing = None        # callable(name): may load the model and add it

    def add(self, llm: LLM, default: bool = False):
        with self.lock:
            self.models[llm.model_id] = llm
            if default or self.default is None:
                self.default = llm.model_id

    def remove(self, model_id: str) -> bool:
        with self.lock:
            llm = self.models.pop(model_id, None)
            if llm is None:
                return False
            if self.default == model_id:
                self.default = next(iter(self.models), None)
        llm.close()
        return True

    def alias(self, source: str, name: str):
        """`name` becomes a second name of the loaded model `source`."""
        with self.lock:
            target = self.aliases.get(source, source)
            if target not in self.models:
                raise ApiError(404, f"model '{source}' not found", "not_found_error", "model_not_found")
            if name in self.models:
                raise ApiError(400, f"'{name}' is the name of a loaded model")
            self.aliases[name] = target

    def drop(self, name: str) -> bool:
        """Removes an alias, or unloads a model together with the aliases that point at it."""
        with self.lock:
            if self.aliases.pop(name, None) is not None:
                return True
            if name not in self.models:
                return False
            for k in [k for k, v in self.aliases.items() if v == name]:
                del self.aliases[k]
        return self.remove(name)

    def evict_idle(self) -> Optional[str]:
        """Unloads the model with no request in flight that has gone unused longest; returns its id."""
        with self.lock:
            idle = [m for m in self.models.values() if not getattr(m.worker, "tickets", None)]
            if not idle:
                return None
            victim = min(idle, key=lambda m: self.last_used.get(m.model_id, 0.0)).model_id
        return victim if self.drop(victim) else None

    def get(self, name: Optional[str]) -> LLM:
        llm = self._get(name)
        self.last_used[llm.model_id] = time.time()
        return llm

    def _get(self, name: Optional[str]) -> LLM:
        # a model whose keep-alive ended sleeps on the host (or was unloaded): the request that names it brings
        # it back before the lookup (`api/context.py: ServerContext._wake`)
        if self.on_missing is not None:
            with self.lock:
                known = bool(self.models) if not name else (name in self.models or name in self.aliases)
            if not known:
                try:
                    self.on_missing(name)
                except Exception:
                    pass
        with self.lock:
            if name and name in self.aliases and self.aliases[name] in self.models:
                return self.models[self.aliases[name]]
            if name and name in self.models:
                return self.models[name]
            if name:
                base = name.split(":")[0]
                for k, v in self.models.items():
                    if k.split(":")[0] == base:
                        return v
            if (not name or not self.strict) and self.default:
                return self.models[self.default]
        raise ApiError(404, f"model '{name}' not found", "not_found_error", "model_not_found")

    def list(self) -> List[LLM]:
        with self.lock:
            return list(self.models.values())


# ------------------------------------------------------------------------- parameters
def _get(d: dict, *names, default=None):
    for n in names:
        if n in d and d[n] is not None:
            return d[n]
    return default


def _stops(v) -> List[str]:
    if v is None:
        return []
    if isinstance(v, str):
        return [v]
    return [str(s) for s in v]


def check_messages(messages) -> None:
    if not isinstance(messages, list) or not messages:
        raise ApiError(400, "messages must be a non-empty array")
    if len(messages) > MAX_MESSAGES:
        raise ApiError(400, f"at most {MAX_MESSAGES} messages")
    total = 0
    for m in messages:
        if not isinstance(m, dict) or "role" not in m:
            raise ApiError(400, "each message needs a role")
        c = m.get("content")
        if isinstance(c, str):
            total += len(c)
        elif isinstance(c, list):
            total += sum(len(p.get("text", "")) for p in c if isinstance(p, dict))
    if total > MAX_CHARS:
        raise ApiError(400, f"request text is limited to {MAX_CHARS} characters")


def params_from_openai(body: dict, llm: LLM, chat: bool) -> GenerationParams:
    """OpenAI + vLLM-extension fields -> GenerationParams.  An unnamed sampler field keeps the
    OpenAI default (T 1.0, top_p 1.0, no top-k, no penalty)."""
    lp = body.get("logprobs")
    if chat:
        want_lp = bool(lp)
        top_lp = int(body.get("top_logprobs") or 0)
    else:
        want_lp = lp is not None and lp is not False
        top_lp = int(lp) if isinstance(lp, int) and not isinstance(lp, bool) else 0
    bias = {}
    for k, v in (body.get("logit_bias") or {}).items():
        try:
            bias[int(k)] = max(-100.0, min(100.0, float(v)))
        except (TypeError, ValueError):
            raise ApiError(400, "logit_bias maps token ids to numbers")
    bad_words = []
    for w in body.get("bad_words") or []:
        for variant in (w, " " + w):
            ids = llm.tokenize(variant, add_special=False)
            if ids:
                bad_words.append(ids)
    if body.get("prompt_logprobs") is not None:
        raise ApiError(400, "prompt_logprobs is not offered: log-probabilities cover the answer's tokens")
    if body.get("chat_template") is not None:
        raise ApiError(400, "a request does not bring its own chat_template; the model's template is used")
    if body.get("continue_final_message") and body.get("add_generation_prompt") is True:
        raise ApiError(400, "continue_final_message and add_generation_prompt: true contradict each other")
    if body.get("truncation_side") not in (None, "left", "right"):
        raise ApiError(400, "truncation_side is left or right")
    p = GenerationParams(
        temperature=float(_get(body, "temperature", default=1.0)),
        top_p=float(_get(body, "top_p", default=1.0)),
        top_k=max(0, int(_get(body, "top_k", default=0))),
        min_p=float(_get(body, "min_p", default=0.0)),
        repeat_penalty=openai_penalty(body.get("frequency_penalty"), body.get("presence_penalty"),
                                      body.get("repetition_penalty"), body.get("repeat_penalty")),
        repeat_last_n=int(_get(body, "repeat_last_n", default=64)),
        max_tokens=_get(body, "max_completion_tokens", "max_tokens"),
        seed=body.get("seed"),
        stop=_stops(body.get("stop")),
        stop_token_ids=[int(t) for t in body.get("stop_token_ids") or []],
        ignore_eos=bool(body.get("ignore_eos", False)),
        include_stop_str_in_output=bool(body.get("include_stop_str_in_output", False)),
        logprobs=want_lp, top_logprobs=top_lp, logit_bias=bias,
        allowed_token_ids=body.get("allowed_token_ids"),
        bad_words_ids=bad_words,
        min_tokens=int(body.get("min_tokens") or 0),
        n=int(body.get("n") or 1),
        skip_special_tokens=bool(body.get("skip_special_tokens", True)),
        echo=bool(body.get("echo", False)),
        thinking_token_budget=body.get("thinking_token_budget"),
        truncate_prompt_tokens=body.get("truncate_prompt_tokens"),
        truncation_side=str(body.get("truncation_side") or "left"),
        cache_salt=body.get("cache_salt"),
        context_shift=bool(body.get("context_shift", False)),
        num_keep=max(0, int(body.get("num_keep", 1))),
        resume_position=int(body.get("resume_position") or 0),
    )
    if p.max_tokens is not None:
        p.max_tokens = int(p.max_tokens)
    from ..text.grammar import spec_from_request

    try:
        p.grammar = spec_from_request(body)
    except ValueError as e:
        raise ApiError(400, f"bad structured-output request: {e}")
    try:
        return p.validate()
    except ParamError as e:
        raise ApiError(400, str(e))


def params_from_ollama(options: dict, body: dict, llm: LLM) -> GenerationParams:
    """Ollama `options` bag; defaults T 0.8, top_p 0.9, top_k 40, repeat_penalty 1.0 over the
    last 64 tokens (`src/inference/engine/llm_engine/generation_defaults.rs:12-21`)."""
    o = options or {}
    num_predict = o.get("num_predict")
    p = GenerationParams(
        temperature=float(o.get("temperature", 0.8)), top_p=float(o.get("top_p", 0.9)),
        top_k=max(0, int(o.get("top_k", 40))), min_p=float(o.get("min_p", 0.0)),
        repeat_penalty=float(o.get("repeat_penalty", 1.0)), repeat_last_n=int(o.get("repeat_last_n", 64)),
        max_tokens=int(num_predict) if num_predict is not None and int(num_predict) > 0 else None,
        seed=o.get("seed"), stop=_stops(o.get("stop")),
        # a generation that reaches the window slides it (the first num_keep tokens and the newer half stay)
        # unless `shift` is false; an unbounded num_predict is what makes that matter
        context_shift=bool(o.get("shift", True)), num_keep=max(0, int(o.get("num_keep", 1))),
    )
    fmt = body.get("format")
    if fmt == "json":
        p.grammar = ("json_schema", {"type": "object"})
    elif isinstance(fmt, dict):
        p.grammar = ("json_schema", fmt)
    try:
        return p.validate()
    except ParamError as e:
        raise ApiError(400, str(e))


def params_from_messages(body: dict, llm: LLM) -> GenerationParams:
    """Anthropic Messages fields.  max_tokens is required there."""
    if "max_tokens" not in body:
        raise ApiError(400, "max_tokens is required")
    p = GenerationParams(
        temperature=float(_get(body, "temperature", default=1.0)), top_p=float(_get(body, "top_p", default=1.0)),
        top_k=max(0, int(_get(body, "top_k", default=0))), max_tokens=int(body["max_tokens"]),
        stop=_stops(body.get("stop_sequences")), repeat_penalty=1.0,
    )
    try:
        return p.validate()
    except ParamError as e:
        raise ApiError(400, str(e))


# ------------------------------------------------------------------------- auth / limits
class Auth:
    """Bearer / x-api-key check.  Each key gets its own cache scope, so one key's cached
    prefixes are never matched by another's requests (`docs/API.md:415-425`)."""

    def __init__(self, keys: Optional[List[str]] = None, required: bool = False):
        self.keys = set(keys or [])
        self.required = required or bool(self.keys)

    def check(self, headers) -> Optional[str]:
        if not self.required:
            return None
        tok = None
        auth = headers.get("authorization")
        if auth and auth.lower().startswith("bearer "):
            tok = auth[7:].strip()
        tok = tok or headers.get("x-api-key")
        if not tok or tok not in self.keys:
            raise ApiError(401, "invalid or missing API key", "authentication_error", "invalid_api_key")
        return tok


class RateLimiter:
    """Token bucket per client key: `rate` requests per second, bursts of `burst`."""

    def __init__(self, rate: float = 0.0, burst: int = 0, clock=time.monotonic):
        self.rate, self.burst, self.clock = rate, max(burst, 1), clock
        self.buckets: Dict[str, List[float]] = {}
        self.lock = threading.Lock()

    def check(self, key: str) -> None:
        if self.rate <= 0:
            return
        now = self.clock()
        with self.lock:
            tokens, last = self.buckets.get(key, [float(self.burst), now])
            tokens = min(self.burst, tokens + (now - last) * self.rate)
            if tokens < 1.0:
                self.buckets[key] = [tokens, now]
                raise ApiError(429, "rate limit exceeded", "rate_limit_error", "rate_limited",
                               retry_after=(1.0 - tokens) / self.rate)
            self.buckets[key] = [tokens - 1.0, now]


PRIORITY = {"batch": 0, "interactive": 1, "fim": 2}


class RequestGate:
    """At most `slots` requests generate at once; the rest wait in priority order (higher first,
    FIFO within a class) up to `max_queue`, beyond which the caller is told when to retry."""

    def __init__(self, slots: int = 256, max_queue: int = 1024):
        self.slots, self.max_queue = slots, max_queue
        self.active = 0
        self.waiting: list = []
        self.counter = itertools.count()
        self.cv = threading.Condition()
        self.mean_slot_s = 1.0
        self.served = 0

    def acquire(self, priority: str = "interactive", timeout: Optional[float] = None) -> float:
        t0 = time.monotonic()
        with self.cv:
            if self.active < self.slots and not self.waiting:
                self.active += 1
                return t0
            if len(self.waiting) >= self.max_queue:
                raise ApiError(503, "server is at capacity", "overloaded_error", "queue_full",
                               retry_after=max(1.0, len(self.waiting) * self.mean_slot_s / max(self.slots, 1)))
            me = (-PRIORITY.get(priority, 1), next(self.counter))
            heapq.heappush(self.waiting, me)
            while not (self.active < self.slots and self.waiting[0] == me):
                left = None if timeout is None else timeout - (time.monotonic() - t0)
                if left is not None and left <= 0:
                    self.waiting.remove(me)
                    heapq.heapify(self.waiting)
                    self.cv.notify_all()
                    raise ApiError(503, "timed out waiting for a slot", "overloaded_error", "queue_timeout",
                                   retry_after=self.mean_slot_s)
                self.cv.wait(left)
            heapq.heappop(self.waiting)
            self.active += 1
            self.cv.notify_all()
            return time.monotonic()

    def release(self, started: float):
        with self.cv:
            self.active -= 1
            self.served += 1
            dt = time.monotonic() - started
            self.mean_slot_s += (dt - self.mean_slot_s) / min(self.served, 50)
            self.cv.notify_all()

    def depth(self) -> dict:
        with self.cv:
            return {"active": self.active, "queued": len(self.waiting), "slots": self.slots,
                    "mean_slot_s": round(self.mean_slot_s, 4)}


def new_request_id(prefix: str = "req") -> str:
    return f"{prefix}-{uuid.uuid4().hex[:24]}"


@dataclass
class Usage:
    prompt_tokens: int = 0
    completion_tokens: int = 0
    cached_tokens: int = 0
    accepted_prediction_tokens: int = 0
    rejected_prediction_tokens: int = 0
    figures: Optional[dict] = None     # the request's own figures (`usage.loken`, utils/figures.py)

    def openai(self) -> dict:
        out = {"prompt_tokens": self.prompt_tokens, "completion_tokens": self.completion_tokens,
               "total_tokens": self.prompt_tokens + self.completion_tokens,
               "prompt_tokens_details": {"cached_tokens": self.cached_tokens},
               "completion_tokens_details": {"accepted_prediction_tokens": self.accepted_prediction_tokens,
                                             "rejected_prediction_tokens": self.rejected_prediction_tokens}}
        if self.figures:
            out["loken"] = self.figures
        return out


def prefill_comment(progress) -> bytes:
    """SSE comment line that reports how far a prompt has been read (clients that follow the SSE
    specification ignore comment lines)."""
    import json as _json

    return (": loken-prefill " + _json.dumps({"done": int(progress[0]), "total": int(progress[1])}) + "\n\n").encode()
