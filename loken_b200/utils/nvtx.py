"""NVTX ranges around the engine's stages, for timelines taken with a system profiler.

Off unless `LOKEN_NVTX=1` (or `enable()`): a range is two library calls per stage and step, which a
decode step of a few milliseconds should not pay for nothing.  The names are the stages of
`utils/metrics.py` (schedule, prefill, decode, verify, sample) plus the layer index inside a forward
when `LOKEN_NVTX=2`.  The reference marks the same stages with its tracing spans
(`src/inference/serve/continuous_serve.rs`, the `stage_perf` counters).
"""
from __future__ import annotations

import contextlib
import os

LEVEL = int(os.environ.get("LOKEN_NVTX", "0") or 0)
_nvtx = None


def enable(level: int = 1):
    global LEVEL
    LEVEL = level


def _lib():
    global _nvtx
    if _nvtx is None:
        import torch

        _nvtx = torch.cuda.nvtx
    return _nvtx


@contextlib.contextmanager
def span(name: str, level: int = 1):
    if LEVEL < level:
        yield
        return
    n = _lib()
    n.range_push(name)
    try:
        yield
    finally:
        n.range_pop()


def mark(name: str, level: int = 1):
    if LEVEL >= level:
        _lib().mark(name)
