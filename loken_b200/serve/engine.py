"""LLMEngine: the continuous-batching engine a user (or the HTTP server, or bench.py) drives.

    eng = LLMEngine("llama-3.3-70b")            # random-init weights of that shape
    rid = eng.add_request(prompt_ids, SamplingParams(...))
    for out in eng.step(): ...                   # one scheduler iteration
    results = eng.generate(list_of_prompt_ids, params)

One `step()` = plan (scheduler) -> prefill forward for admitted prompts -> decode forward for
running sequences -> sample -> finish checks, like the reference's `ContinuousBatchEngine`
(`src/inference/serve/continuous_batch.rs:167-449`): EOS / length finish, cancel flags, and a
step error ends the requests that had started while queued ones stay queued.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence as Seq, Union

import torch

from ..models.config import ModelConfig, get_config
from ..models.weights import ModelWeights, random_weights
from ..utils import nvtx
from .kv_manager import PagedKvAllocator
from .params import SamplingParams
from .runner import ModelRunner
from .scheduler import Scheduler, Sequence, StepPlan


@dataclass
class StepOutput:
    seq_id: int
    new_tokens: List[int]
    finished: bool = False
    finish_reason: Optional[str] = None
    logprobs: Optional[List[tuple]] = None     # per new token: (logprob, [(token id, logprob), ...])
    figures: Optional[dict] = None             # filled by the worker on the last output of a request
    cached_tokens: int = 0


@dataclass
class GenerationResult:
    seq_id: int
    prompt_tokens: int
    cached_tokens: int
    output: List[int]
    finish_reason: Optional[str]
    ttft_s: Optional[float]
    total_s: float
    accepted_drafts: int = 0
    rejected_drafts: int = 0


@dataclass
class EngineStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    step_errors: int = 0
    consecutive_errors: int = 0
    context_shifts: int = 0


def kv_bytes_per_token(cfg: ModelConfig, n_kv_local: int) -> int:
    per = cfg.head_dim + (cfg.head_dim // 32) * 2 if cfg.kv_format == "q8" else cfg.head_dim * 2
    return 2 * cfg.n_layers * n_kv_local * per


class LLMEngine:
    def __init__(self, model: Union[str, ModelConfig], *, weights: Optional[ModelWeights] = None, device=None,
                 tp_rank: int = 0, tp_size: int = 1, comm=None, num_blocks: Optional[int] = None,
                 block_size: int = 16, max_seqs: int = 256, max_prefill_tokens: int = 8192, max_ctx: int = 8192,
                 kv_memory_fraction: float = 0.85, seed: int = 0, eos_token_ids: Optional[List[int]] = None,
                 use_graphs: bool = True, enable_prefix_cache: bool = True, moe_runner_factory=None,
                 lookahead: int = 0, pipeline=None, kv_disk_dir: Optional[str] = None, kv_disk_host_mb: int = 256,
                 kv_disk_max_gb: float = 0.0):
        self.cfg = get_config(model) if isinstance(model, str) else model
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if weights is None:
            weights = random_weights(self.cfg, self.device, seed=seed, tp_rank=tp_rank, tp_size=tp_size,
                                     ep_rank=tp_rank, ep_size=tp_size)
        self.weights = weights
        if self.cfg.kv_format == "q8" and self.cfg.qk_norm:
            # keys are stored as int8 with one step per 32 lanes: fold a per-lane scale into the Q / K norm
            # weights so the lanes of a block carry comparable magnitudes (scores are unchanged)
            from ..models.key_scale import apply_key_scale

            apply_key_scale(weights)
        if num_blocks is None:
            free, _total = torch.cuda.mem_get_info(self.device)
            reserve = 6 << 30     # activations, graphs, workspaces
            per_block = kv_bytes_per_token(self.cfg, weights.n_kv_local) * block_size
            num_blocks = max(64, int((free - reserve) * kv_memory_fraction) // per_block)
            num_blocks = min(num_blocks, (max_seqs * max_ctx) // block_size + 64)
        self.alloc = PagedKvAllocator(num_blocks, block_size, enable_prefix_cache)
        self.sched = Scheduler(self.alloc, max_running=max_seqs, max_prefill_tokens=max_prefill_tokens,
                               lookahead=lookahead)
        moe_runner = moe_runner_factory(self.cfg, weights, max(max_prefill_tokens, max_seqs), comm) \
            if moe_runner_factory else None
        if self.cfg.is_moe and moe_runner is None:
            from ..models.moe import MoeRunner

            moe_runner = MoeRunner(self.cfg, weights, max(max_prefill_tokens, max_seqs), comm)
        self.runner = ModelRunner(self.cfg, weights, num_blocks=num_blocks, block_size=block_size,
                                  max_seqs=max_seqs, max_tokens=max_prefill_tokens, max_ctx=max_ctx, comm=comm,
                                  moe_runner=moe_runner,
                                  # a runner that plans on the host inside the step (host-streamed experts) cannot be captured
                                  use_graphs=use_graphs and not getattr(moe_runner, "plans_on_host", False),
                                  device=self.device,
                                  pipeline=pipeline)
        self.eos = set(eos_token_ids or [])
        self.runner.end_ids = sorted(self.eos)
        self.max_ctx = max_ctx
        self.seqs: Dict[int, Sequence] = {}
        self.rngs: Dict[int, object] = {}
        self.cancelled: set = set()
        self._imports = 0
        self._stash: List[StepOutput] = []
        self.next_id = 0
        self.stats = EngineStats()
        self.spec = None            # a serve.speculative.Speculator while a drafter is attached
        # the cache's disk tier: finished sequences leave their full 256-token blocks, new prompts find them
        # (one engine, one cache: under tensor parallelism every rank holds a shard and the tier stays off)
        self.disk = None
        if kv_disk_dir and tp_size == 1 and pipeline is None:
            from .kv_disk import KvDiskTier
            from .kv_persist import DiskPersistence

            tier = KvDiskTier(kv_disk_dir, compress=False, max_bytes=int(kv_disk_max_gb * (1 << 30)) or None,
                              host_bytes=int(kv_disk_host_mb) << 20)
            self.disk = DiskPersistence(self.runner, self.alloc, tier)
            self.sched.on_finish = lambda seq, n: (self.disk.save(seq.seq_id, seq.tokens, n, seq.salt)
                                                   if getattr(seq, "prompt_embeds", None) is None and seq.shifts == 0 else 0)
        self.grammar_factory = None  # callable((kind, source)) -> session; set by whoever owns the tokenizer

    # ---- requests ----
    def add_request(self, prompt: Seq[int], params: Optional[SamplingParams] = None, salt: int = 0,
                    embeds=None) -> int:
        """`embeds` (or a `prompt` object carrying `.embeds`): float rows [len(prompt), hidden] that stand
        in for the prompt's token embeddings (`prompt_embeds`); `prompt` then holds placeholder ids."""
        params = (params or SamplingParams()).validate()
        embeds = embeds if embeds is not None else getattr(prompt, "embeds", None)
        if embeds is not None:
            import zlib

            import numpy as np

            arr = np.ascontiguousarray(np.asarray(embeds, dtype=np.float32))
            if arr.ndim != 2 or arr.shape[1] != self.cfg.hidden:
                raise ValueError(f"prompt embeddings must be [rows, {self.cfg.hidden}]")
            prompt = [0] * arr.shape[0]
            if not salt:
                salt = (1 << 40) | zlib.crc32(arr.tobytes())     # equal embeddings share cached blocks, nothing else does
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if len(prompt) >= self.max_ctx:
            raise ValueError(f"prompt of {len(prompt)} tokens does not fit the {self.max_ctx}-token window")
        if self.alloc.blocks_needed(len(prompt) + 1 + self.sched.lookahead) > self.alloc.num_blocks:
            # refused before an id is taken, so ranks that mirror this engine keep the same ids
            raise ValueError(f"a request of {len(prompt)} tokens needs more KV blocks than the pool has "
                             f"({self.alloc.num_blocks} x {self.alloc.block_size} tokens)")
        sid = self.next_id
        self.next_id += 1
        seq = Sequence(sid, list(prompt), params, arrival=time.perf_counter(), salt=salt)
        if embeds is not None:
            seq.prompt_embeds = torch.from_numpy(arr).to(self.device).to(torch.bfloat16)
        if params.grammar is not None:
            if self.grammar_factory is None:
                raise ValueError("structured output needs a tokenizer: load the model through LLM")
            seq.grammar = self.grammar_factory(params.grammar)
        self.seqs[sid] = seq
        self.rngs[sid] = params.rng(0)
        if self.disk is not None and embeds is None:
            self.disk.restore(seq.tokens, salt)       # rows this prompt left on disk in an earlier life join the prefix cache
        self.sched.add_request(seq)
        return sid

    def abort(self, seq_id: int):
        self.cancelled.add(seq_id)

    # ---- KV hand-over (disaggregated prefill) ----
    def export_prefix(self, prompt: Seq[int], salt: int = 0) -> bytes:
        """Prefills `prompt` through the ordinary path (other requests keep running) and returns its
        cache as a hand-over container (`cluster/handover.py`).  Call between steps."""
        from ..cluster.handover import export_sequence

        if getattr(self.runner.w, "tp_size", 1) > 1:
            raise ValueError("a tensor-parallel model holds one cache shard per rank; hand-over is per engine")
        sp = SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True)
        sid = self.add_request(list(prompt), sp, salt=salt)
        def advance():
            # other requests' tokens produced meanwhile are handed out by the caller's next step()
            self._stash += [o for o in self._step() if o.seq_id != sid]

        try:
            while not self.seqs[sid].output:
                advance()
            return export_sequence(self.runner, self.alloc, sid, list(prompt), len(prompt))
        finally:
            self.abort(sid)
            advance()            # the cancelled sequence is dropped at the top of a step

    def import_prefix(self, blob: bytes, salt: int = 0) -> int:
        """Writes a handed-over cache into free blocks and publishes it in the prefix cache, so the
        request that follows with the same prompt starts from it.  Returns the positions imported."""
        from ..cluster.handover import import_sequence

        tmp = -1 - self._imports
        self._imports += 1
        n = import_sequence(self.runner, self.alloc, tmp, blob, salt)
        self.alloc.free(tmp)     # the blocks stay published (evictable) under their content hashes
        return n

    def reset_prefix_cache(self) -> int:
        """Drops the idle cached blocks; returns how many.  Call between steps."""
        return int(self.alloc.reset_prefix_cache() or 0)

    def embed(self, tokens, pooling: str = "last"):
        """Unit-norm embedding of a prompt (not batched with generation; call between steps)."""
        if len(tokens) == 0 or len(tokens) >= self.max_ctx:
            raise ValueError("the input must have between 1 and max_ctx - 1 tokens")
        return self.runner.embed(list(tokens), self.alloc, pooling)

    def layer_perf(self, n_tokens: int = 1):
        """Times one decode-shaped forward of `n_tokens` rows layer by layer (scratch cache blocks)."""
        return self.runner.layer_perf(self.alloc, n_tokens)

    # ---- speculative decoding ----
    def attach_speculator(self, spec):
        """From the next step on, running sequences are decoded by draft-and-verify cycles."""
        from .speculative import DRAFT_MAX

        self.sched.lookahead = max(self.sched.lookahead, DRAFT_MAX)
        self.spec = spec

    def detach_speculator(self):
        spec, self.spec = self.spec, None
        self.sched.lookahead = 0
        if spec is not None:
            for sid in list(getattr(spec.drafter, "known", {})):
                spec.drafter.release(sid)

    def has_work(self) -> bool:
        return self.sched.has_work()

    # ---- one iteration ----
    def _finish_check(self, seq: Sequence, tok: int) -> Optional[str]:
        p = seq.params
        n_out = len(seq.output)
        if not p.ignore_eos and n_out >= p.min_tokens and (tok in self.eos or tok in p.stop_token_ids):
            return "stop"
        if p.max_tokens is not None and n_out >= p.max_tokens:
            return "length"
        if seq.total_len >= self.max_ctx and not self._can_shift(seq):
            return "length"
        return None

    # ---- context shift ----
    def _can_shift(self, seq: Sequence) -> bool:
        cfg = self.cfg
        return bool(seq.params.context_shift and seq.prompt_embeds is None and self.spec is None
                    and getattr(self.runner, "pipeline", None) is None and not cfg.sliding_window)

    def context_shift(self, seq_id: int, n_keep: Optional[int] = None, n_discard: Optional[int] = None) -> int:
        """Makes room in a running sequence's window: cache positions [n_keep, n_keep + n_discard) are
        dropped, the later ones move down and their keys are turned back by n_discard positions (the
        rotary phase comes from the layer's own frequency table, so scaled and factored frequencies need
        nothing special).  Defaults: keep `params.num_keep` tokens, drop the older half of the rest.
        Returns the number of positions dropped (0 when the pool has no room for the copy).  A re-phased
        key is not bit for bit the key a fresh prefill of the shorter text would produce.  Sliding-window
        layers, prompts given as embeddings, pipelines and speculative decoding do not shift
        (the reference lists the same exclusions, `docs/STATUS.md:111-123`)."""
        seq = self.seqs[seq_id]
        if seq.state != "running" or seq.computed < seq.total_len - 1:
            raise ValueError("only a sequence that is decoding can shift its context")
        if self.cfg.sliding_window or seq.prompt_embeds is not None:
            raise ValueError("this sequence's cache cannot be shifted")
        have = seq.computed                                   # cache positions that hold K/V
        n_keep = max(0, min(seq.params.num_keep if n_keep is None else n_keep, have - 2))
        if n_discard is None:
            n_discard = (have - n_keep) // 2
        n_discard = min(n_discard, have - n_keep - 1)
        if n_discard <= 0:
            return 0
        self.alloc.trim(seq_id, have)                         # lookahead slots go back first
        moved = self.alloc.shift(seq_id, n_keep, n_discard)
        if moved is None:
            return 0
        self.runner.kv_shift(*moved)
        seq.drop_positions(n_keep, n_discard)
        seq.computed = have - n_discard
        self.stats.context_shifts += 1
        return n_discard

    def _emit(self, seq: Sequence, tok: int, outs: Dict[int, StepOutput], lp: Optional[tuple] = None):
        if seq.first_token_time is None:
            seq.first_token_time = time.perf_counter()
        seq.output.append(int(tok))
        o = outs.setdefault(seq.seq_id, StepOutput(seq.seq_id, []))
        o.new_tokens.append(int(tok))
        if lp is not None:
            seq.logprobs.append(lp)
            o.logprobs = (o.logprobs or []) + [lp]
        reason = self._finish_check(seq, int(tok))
        if seq.grammar is not None and not reason:
            # the matcher follows what was sampled; once it accepts and stops, so does the request
            if not seq.grammar.accept(int(tok)) or seq.grammar.done():
                reason = "stop"
        if reason:
            o.finished, o.finish_reason = True, reason
            self.sched.finish(seq, reason)

    def step(self) -> List[StepOutput]:
        outs = self._step()
        if self._stash:
            outs, self._stash = self._stash + outs, []
        return outs

    def _step(self) -> List[StepOutput]:
        outs: Dict[int, StepOutput] = {}
        for sid in list(self.cancelled):
            seq = self.seqs.get(sid)
            if seq is not None and seq.state != "finished":
                self.sched.finish(seq, "cancelled")
                outs[sid] = StepOutput(sid, [], True, "cancelled")
        self.cancelled.clear()
        for seq in list(self.sched.running):
            # a generation at the end of its window slides it before the scheduler asks for the next slot
            if seq.state == "running" and seq.total_len + 1 + self.sched.lookahead > self.max_ctx \
                    and seq.computed >= seq.total_len - 1 and self._can_shift(seq):
                if self.context_shift(seq.seq_id) == 0:
                    self.sched.finish(seq, "length")
                    outs[seq.seq_id] = StepOutput(seq.seq_id, [], True, "length")
        with nvtx.span("schedule"):
            plan = self.sched.schedule()
        self.stats.preemptions += len(plan.preempted)
        for seq in plan.rejected:
            outs[seq.seq_id] = StepOutput(seq.seq_id, [], True, "error")
        if plan.empty:
            return list(outs.values())
        lps: Dict[int, tuple] = {}
        try:
            with nvtx.span("prefill"):
                first = self.runner.prefill(plan.prefills, self.alloc, self.rngs) if plan.prefills else {}
            if first:
                done = [it.seq for it in plan.prefills if it.seq.seq_id in first]
                self._logprobs(done, [first[s.seq_id] for s in done], lps)
            spec = self.spec
            commits = None
            if plan.decodes and spec is not None:
                with nvtx.span("verify"):
                    commits = spec.step(self, list(plan.decodes))
                toks = []
            else:
                with nvtx.span("decode"):
                    toks = self.runner.decode(plan.decodes, self.alloc, self.rngs) if plan.decodes else []
                if plan.decodes:
                    self._logprobs(list(plan.decodes), toks, lps)
            self.runner.check_status()
        except Exception:
            # a failed step ends the requests that had started; queued ones stay queued
            self.stats.step_errors += 1
            self.stats.consecutive_errors += 1
            for s in [it.seq for it in plan.prefills] + list(plan.decodes):
                if s.state != "finished":
                    self.sched.finish(s, "error")
            raise
        self.stats.consecutive_errors = 0
        self.sched.on_step_done(plan)
        self.stats.steps += 1
        self.stats.prefill_tokens += sum(it.end - it.start for it in plan.prefills)
        self.stats.decode_tokens += len(plan.decodes)
        for it in plan.prefills:
            if it.seq.seq_id in first:
                self._emit(it.seq, first[it.seq.seq_id], outs, lps.get(it.seq.seq_id))
        if commits is not None:
            for seq in plan.decodes:
                base = seq.total_len                 # the carried token's K/V is in the cache: computed == base
                n_done = 0
                for tok in commits.get(seq.seq_id, []):
                    self._emit(seq, tok, outs)
                    n_done += 1
                    if seq.state == "finished":
                        break
                if seq.state != "finished":
                    # accepted drafts' rows stay valid; the last committed token is carried to the next step
                    seq.computed = base + n_done - 1
                else:
                    spec.drafter.release(seq.seq_id)
            self.stats.decode_tokens += sum(len(v) for v in commits.values()) - len(plan.decodes)
        for seq, tok in zip(plan.decodes, toks):
            self._emit(seq, tok, outs, lps.get(seq.seq_id))
        return list(outs.values())

    def _logprobs(self, seqs, toks, into: Dict[int, tuple]):
        """Log-probabilities of the tokens just sampled for the sequences that asked for them;
        `seqs` are in the row order of the runner's last logits."""
        want = [(i, s) for i, s in enumerate(seqs) if s.params.logprobs]
        if not want:
            return
        top_n = max(s.params.top_logprobs for _, s in want)
        got = self.runner.logprobs_of([i for i, _ in want], [toks[i] for i, _ in want], top_n)
        for (i, s), (lp, top) in zip(want, got):
            into[s.seq_id] = (lp, top[:s.params.top_logprobs])

    # ---- convenience ----
    def generate(self, prompts: Iterable[Seq[int]], params: Union[SamplingParams, Seq[SamplingParams], None] = None
                 ) -> List[GenerationResult]:
        prompts = list(prompts)
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        t0 = time.perf_counter()
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        while self.has_work():
            self.step()
        t1 = time.perf_counter()
        res = []
        for sid in ids:
            s = self.seqs.pop(sid)
            self.rngs.pop(sid, None)
            ttft = (s.first_token_time - s.arrival) if s.first_token_time else None
            res.append(GenerationResult(sid, len(s.prompt), s.cached_tokens, s.output, s.finish_reason, ttft, t1 - t0,
                                        s.accepted_drafts, s.rejected_drafts))
        return res
