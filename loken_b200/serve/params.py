"""Per-request sampling parameters and their defaults / bounds.

Defaults when the request and the model say nothing: T 0.8, top_p 0.9, top_k 40,
repeat_penalty 1.0, repeat_last_n 64 on the Ollama routes
(`src/inference/engine/llm_engine/generation_defaults.rs:12-21`); an unnamed penalty on the
OpenAI / Messages routes is none; frequency + presence penalties are summed, clamped to
[-2, 2] and mapped to 1 + pen (`src/api/handlers/sampling.rs:380-395`).  Bounds:
max_tokens <= 131072, <= 4 stop sequences of <= 256 chars, top_logprobs <= 20, n <= 16
(`src/api/handlers/sampling.rs:10-45`).
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Dict, List, Optional

MAX_TOKENS_BOUND = 131072
MAX_STOPS = 4
MAX_STOP_CHARS = 256
MAX_TOP_LOGPROBS = 20
MAX_N = 16


class ParamError(ValueError):
    pass


@dataclass
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.9
    min_p: float = 0.0
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    max_tokens: Optional[int] = None
    seed: Optional[int] = None
    stop: List[str] = field(default_factory=list)
    stop_token_ids: List[int] = field(default_factory=list)
    ignore_eos: bool = False
    include_stop_str_in_output: bool = False
    logprobs: bool = False
    top_logprobs: int = 0
    logit_bias: Dict[int, float] = field(default_factory=dict)
    allowed_token_ids: Optional[List[int]] = None
    bad_words_ids: List[List[int]] = field(default_factory=list)
    min_tokens: int = 0
    n: int = 1
    grammar: Optional[tuple] = None      # (kind, source): json_schema | regex | lark | choice
    # a generation that reaches the window keeps its first `num_keep` tokens and the newer half of the rest
    # (the cache is shifted and its keys re-phased) instead of ending with "length"
    context_shift: bool = False
    num_keep: int = 1
    # a generation resumed on another node: how many of its tokens were already sampled (they arrive as part of
    # the prompt); the draw for token N depends on (seed, N) alone, so the stream continues where it stopped
    resume_position: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-7

    def validate(self) -> "SamplingParams":
        if self.max_tokens is not None and not (0 < self.max_tokens <= MAX_TOKENS_BOUND):
            raise ParamError(f"max_tokens must be in 1..{MAX_TOKENS_BOUND}")
        if len(self.stop) > MAX_STOPS:
            raise ParamError(f"at most {MAX_STOPS} stop sequences")
        if any(len(s) > MAX_STOP_CHARS for s in self.stop):
            raise ParamError(f"a stop sequence is limited to {MAX_STOP_CHARS} characters")
        if not (0 <= self.top_logprobs <= MAX_TOP_LOGPROBS):
            raise ParamError(f"top_logprobs must be in 0..{MAX_TOP_LOGPROBS}")
        if not (1 <= self.n <= MAX_N):
            raise ParamError(f"n must be in 1..{MAX_N}")
        if self.temperature < 0 or self.temperature > 5:
            raise ParamError("temperature must be in 0..5")
        if not (0 < self.top_p <= 1.0):
            raise ParamError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ParamError("top_k must be >= 0")
        if not (0 <= self.min_p < 1.0):
            raise ParamError("min_p must be in [0, 1)")
        if self.repeat_penalty <= 0:
            raise ParamError("repeat_penalty must be > 0")
        if self.resume_position < 0:
            raise ParamError("resume_position must be >= 0")
        return self

    def rng(self, seq_index: int = 0):
        """One generator per request: a seeded request is reproducible, an unseeded one gets a fresh seed.
        The uniform for a token is a function of (seed, its index in the output) only (`serve/replay.py`)."""
        from .replay import PositionRng, _mix

        seed = self.seed if self.seed is not None else random.SystemRandom().getrandbits(63)
        return PositionRng(seed if seq_index == 0 else _mix(seed, 0, seq_index), self.resume_position)


def openai_penalty(frequency: Optional[float], presence: Optional[float], repetition: Optional[float] = None,
                   repeat: Optional[float] = None) -> float:
    """An explicit repeat/repetition penalty wins; otherwise frequency + presence, clamped to
    [-2, 2], becomes 1 + pen; unnamed means none."""
    if repeat is not None:
        return float(repeat)
    if repetition is not None:
        return float(repetition)
    if frequency is None and presence is None:
        return 1.0
    pen = max(-2.0, min(2.0, (frequency or 0.0) + (presence or 0.0)))
    return 1.0 + pen


GREEDY = SamplingParams(temperature=0.0, top_k=0, top_p=1.0)
