"""Measurement core of `bench.py --config 1|2|4|5`: whole serving runs through the public engine API.

A run submits every request at time zero (`LLMEngine.add_request`), then calls `LLMEngine.step()`
until all of them have finished: scheduler, chunked prefill, continuous batching, pinned-host
staging and the H2D copy of every step's inputs, captured decode graphs, sampling on the device,
the D2H copy of the new tokens.  The run is bracketed by a barrier + synchronize on both sides and
timed with CUDA events on the launching stream (max over ranks); the figure is whole-job output
tokens per second, with the p50 time to first token beside it.  A shorter warm-up run with other
prompts goes first so graph capture and allocator growth stay outside the timed region.
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import _lib
from ..serve.params import SamplingParams


def _barrier_sync(world: int):
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def _max_over_ranks(v: float, world: int, device) -> float:
    if world == 1:
        return v
    t = torch.tensor([v], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_requests(engine, prompts: Sequence[Sequence[int]], sp: SamplingParams, world: int, clock_sampler=None) -> dict:
    dev = engine.device
    runner = engine.runner
    _barrier_sync(world)
    h2d0, d2h0 = runner.h2d_bytes, runner.d2h_bytes
    l0 = runner.kernel_launches + _lib.launch_count()
    steps0 = engine.stats.steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if clock_sampler:
        clock_sampler.start()
    e0.record()
    t0 = time.perf_counter()
    ids = [engine.add_request(list(p), sp) for p in prompts]
    while engine.has_work():
        engine.step()
    e1.record()
    _barrier_sync(world)
    clocks = clock_sampler.stop() if clock_sampler else {}
    ms = _max_over_ranks(e0.elapsed_time(e1), world, dev)
    seqs = [engine.seqs.pop(i) for i in ids]
    for i in ids:
        engine.rngs.pop(i, None)
    n_out = sum(len(s.output) for s in seqs)
    ttfts = sorted((s.first_token_time - t0) for s in seqs if s.first_token_time is not None)
    steps = max(1, engine.stats.steps - steps0)
    return dict(ms=ms, out_tokens=n_out, tok_s=n_out / (ms / 1e3), steps=steps,
                ttft_p50_s=ttfts[len(ttfts) // 2] if ttfts else None,
                h2d_bytes_per_step=(runner.h2d_bytes - h2d0) / steps, d2h_bytes_per_step=(runner.d2h_bytes - d2h0) / steps,
                gpu_launches=int(runner.kernel_launches + _lib.launch_count() - l0), clocks=clocks,
                accepted=sum(s.accepted_drafts for s in seqs), rejected=sum(s.rejected_drafts for s in seqs),
                cached_tokens=sum(s.cached_tokens for s in seqs), prompt_tokens=sum(len(s.prompt) for s in seqs),
                preemptions=engine.stats.preemptions)


def random_prompts(vocab: int, lens: Sequence[int], seed: int, prefix: Optional[List[int]] = None) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [(prefix or []) + torch.randint(0, vocab, (int(n),), generator=g).tolist() for n in lens]


def serving_run(engine, *, lens: Sequence[int], out_tokens: int, sp: SamplingParams, world: int, seed: int = 1234,
                prefix_len: int = 0, clock_sampler=None, warm_out: int = 6) -> dict:
    """Warm-up run (other prompts, `warm_out` tokens each), cache reset, then the timed run."""
    import dataclasses

    vocab = engine.cfg.vocab
    g = torch.Generator().manual_seed(seed + 7)
    warm_prefix = torch.randint(0, vocab, (prefix_len,), generator=g).tolist() if prefix_len else None
    warm = random_prompts(vocab, lens, seed + 1, warm_prefix)
    run_requests(engine, warm, dataclasses.replace(sp, max_tokens=warm_out), world)
    engine.reset_prefix_cache()
    prefix = torch.randint(0, vocab, (prefix_len,), generator=torch.Generator().manual_seed(seed + 3)).tolist() \
        if prefix_len else None
    prompts = random_prompts(vocab, lens, seed, prefix)
    r = run_requests(engine, prompts, dataclasses.replace(sp, max_tokens=out_tokens), world, clock_sampler)
    r["requests"] = len(prompts)
    return r
