"""Speculative decoding for the batched engine.

Cycle (per engine step, for every running sequence at once): a drafter proposes up to k tokens;
the target runs ONE forward over k+1 rows per sequence (the carried token + the drafts, through
the decode kernels with a block-table row per query row); every row is sampled with the target's
own sampler; the accepted prefix is the longest run where draft[i] == sample[i], and the sample
after it is committed as well ("bonus").  The output is therefore exactly what plain decoding
with the same sampler and seed would have produced; rejected rows' cache entries are cut back
with `Scheduler.trim`.  This is the reference's verify-commit rule
(`src/inference/engine/decode_step.rs:259-317`), which it applies to one conversation at a time;
here all sequences of the batch are verified in the same forward.

Drafters: `PromptLookupDrafter` (n-gram cascade 4..2 over the sequence's own tokens,
`src/inference/serve/prompt_lookup.rs:23`) and `ModelDrafter` (a smaller model with the same
vocabulary and its own paged cache, `llm_engine/mod.rs:388-890`).  `DraftLength` learns how many
tokens are worth drafting from per-position survival counts and measured cycle times
(`decode_step.rs:330-384`).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence as Seq

from .kv_manager import PagedKvAllocator
from .params import GREEDY
from .scheduler import Sequence

DRAFT_MAX = 8


class _RowView:
    """What the sampler needs to know about one verify row: the sequence's parameters and the
    history the row is sampled after (real tokens + the drafts before the row)."""

    def __init__(self, seq: Sequence, extra: List[int]):
        self.seq_id = seq.seq_id
        self.params = seq.params
        self._base = seq
        self._extra = extra
        self.mask = None             # int32 words: the grammar's mask after this row's history, for constrained requests

    @property
    def tokens(self) -> List[int]:
        return self._base.tokens + self._extra

    @property
    def output(self) -> List[int]:
        return self._base.output + self._extra


# ------------------------------------------------------------------------------ drafters
class PromptLookupDrafter:
    """Finds the latest earlier occurrence of the sequence's last n tokens (n = 4, 3, 2) and
    proposes the tokens that followed it."""
    name = "prompt_lookup"

    def __init__(self, max_ngram: int = 4, min_ngram: int = 2):
        self.max_ngram, self.min_ngram = max_ngram, min_ngram
        self.seconds_per_token = 0.0

    def propose(self, seqs: Seq[Sequence], k: int) -> List[List[int]]:
        out = []
        for s in seqs:
            toks = s.tokens
            draft: List[int] = []
            for n in range(self.max_ngram, self.min_ngram - 1, -1):
                if len(toks) <= n:
                    continue
                tail = toks[-n:]
                # scan right to left, skipping the tail itself
                for i in range(len(toks) - n - 1, -1, -1):
                    if toks[i:i + n] == tail:
                        draft = toks[i + n:i + n + k]
                        break
                if draft:
                    break
            out.append(draft)
        return out

    def commit(self, seq: Sequence, new_len: int):
        pass

    def release(self, seq_id: int):
        pass

    def status(self) -> dict:
        return {"method": self.name, "ngram": [self.min_ngram, self.max_ngram]}


class ModelDrafter:
    """A second, smaller model with its own runner and paged cache.  Each cycle it first feeds
    whatever the target committed since its last visit (one multi-row forward), then decodes
    greedily k - 1 more steps."""
    name = "model"

    def __init__(self, cfg, weights, *, max_seqs: int, max_ctx: int, block_size: int = 16, comm=None,
                 model_id: str = "draft"):
        from .runner import ModelRunner

        self.cfg = cfg
        self.model_id = model_id
        blocks = max_seqs * ((max_ctx + DRAFT_MAX + block_size - 1) // block_size + 1) + 8
        self.alloc = PagedKvAllocator(blocks, block_size, enable_prefix_cache=False)
        self.runner = ModelRunner(cfg, weights, num_blocks=blocks, block_size=block_size, max_seqs=max_seqs,
                                  max_tokens=max(max_seqs * (DRAFT_MAX + 2), 8192), max_ctx=max_ctx + DRAFT_MAX,
                                  comm=comm, use_graphs=False)
        self.known: Dict[int, List[int]] = {}      # tokens whose K/V the draft cache holds, per sequence
        self.shadow: Dict[int, Sequence] = {}
        self.rngs: Dict[int, object] = {}
        self.seconds_per_token = 0.0

    def _sync(self, s: Sequence) -> int:
        """Brings the draft cache's view of `s` to a prefix of its real tokens; returns its length."""
        toks = s.tokens
        if getattr(s, "prompt_embeds", None) is not None:
            return -1                            # embeddings of the target's width: the drafter cannot read them
        have = self.known.get(s.seq_id)
        if have is None:
            if not self.alloc.allocate(s.seq_id, len(toks) + DRAFT_MAX):
                return -1
            self.known[s.seq_id] = []
            return 0
        n = 0
        lim = min(len(have), len(toks) - 1)      # the last real token is always fed again: its logits are needed
        while n < lim and have[n] == toks[n]:
            n += 1
        del have[n:]
        want = len(toks) + DRAFT_MAX
        cur = self.alloc.length(s.seq_id)
        if want > cur and not self.alloc.append(s.seq_id, want - cur):
            return -1
        return n

    CATCH_UP_ROWS = 16      # more pending tokens than this go through the prefill kernels, not as verify rows

    def _catch_up(self, items):
        """A sequence the drafter meets for the first time (or after a long gap) has its whole prompt
        pending.  All but its last token are written to the draft cache by variable-length prefill
        forwards, as many chunks per forward as the runner's row budget holds; what is left (the
        last token, whose logits start the draft) goes on as verify rows."""
        from .scheduler import PrefillItem

        budget = self.runner.d_rows.shape[1]
        max_items = self.runner.d_bt.shape[0]
        out, todo = [], []
        for s, toks, start in items:
            if len(toks) > self.CATCH_UP_ROWS:
                todo.append((s, start, start + len(toks) - 1))
                out.append((s, toks[-1:], start + len(toks) - 1))
            else:
                out.append((s, toks, start))
        batch, used = [], 0
        while todo:
            s, a, b = todo.pop(0)
            n = min(b - a, budget - used)
            batch.append(PrefillItem(s, a, a + n, False))
            used += n
            if a + n < b:
                todo.insert(0, (s, a + n, b))
            if used >= budget or len(batch) >= max_items or not todo:
                self.runner.prefill(batch, self.alloc, None)
                batch, used = [], 0
        return out

    def propose(self, seqs: Seq[Sequence], k: int) -> List[List[int]]:
        t0 = time.perf_counter()
        items, live = [], []
        for s in seqs:
            n = self._sync(s)
            if n < 0:
                continue
            toks = s.tokens
            items.append((s, toks[n:], n))
            live.append(s)
        drafts: Dict[int, List[int]] = {s.seq_id: [] for s in seqs}
        if not live or k <= 0:
            return [drafts[s.seq_id] for s in seqs]
        items = self._catch_up(items)
        logits = self.runner.forward_rows(items, self.alloc, last_only=True)
        views = [_RowView(_greedy_twin(s), []) for s in live]
        first = self.runner.sample_rows(logits, views, [0.0] * len(live))
        for s, t in zip(live, first):
            self.known[s.seq_id] = list(s.tokens)
            drafts[s.seq_id].append(int(t))
        for step in range(1, k):
            items = [(s, [drafts[s.seq_id][-1]], len(s.tokens) + step - 1) for s in live]
            logits = self.runner.forward_rows(items, self.alloc, last_only=True)
            nxt = self.runner.sample_rows(logits, views, [0.0] * len(live))
            for s, t in zip(live, nxt):
                self.known[s.seq_id].append(drafts[s.seq_id][-1])
                drafts[s.seq_id].append(int(t))
        dt = time.perf_counter() - t0
        self.seconds_per_token += (dt / max(k, 1) - self.seconds_per_token) * 0.2
        return [drafts[s.seq_id] for s in seqs]

    def commit(self, seq: Sequence, new_len: int):
        pass        # the next _sync compares tokens, which covers accepted and rejected drafts alike

    def release(self, seq_id: int):
        if seq_id in self.known:
            self.alloc.free(seq_id)
            self.known.pop(seq_id, None)

    def status(self) -> dict:
        return {"method": self.name, "model": self.model_id, "sequences": len(self.known),
                "seconds_per_token": round(self.seconds_per_token, 6)}


def _greedy_twin(s: Sequence) -> Sequence:
    return Sequence(s.seq_id, s.prompt, GREEDY, output=s.output)


# ------------------------------------------------------------------------------ learned length
@dataclass
class DraftLength:
    """Chooses k from what has been observed: reached[i] / kept[i] count how often draft position
    i was verified and survived; cycle seconds are kept per length; the choice maximises expected
    committed tokens per second, longer on ties.  A losing drafter is held off for 48 plain steps,
    doubling up to 1536, and a winning cycle restores the hold-off."""
    k_max: int = DRAFT_MAX
    fixed: Optional[int] = None
    reached: List[int] = field(default_factory=lambda: [0] * DRAFT_MAX)
    kept: List[int] = field(default_factory=lambda: [0] * DRAFT_MAX)
    cycle_s: Dict[int, float] = field(default_factory=dict)
    plain_s: float = 0.0
    cycles: int = 0
    holdoff: int = 0
    next_holdoff: int = 48
    PROBE_CYCLES = 4

    def observe(self, k: int, accepted: int, seconds: float, n_seqs: int = 1):
        for i in range(k):
            self.reached[i] += 1
            if i < accepted:
                self.kept[i] += 1
        prev = self.cycle_s.get(k)
        self.cycle_s[k] = seconds if prev is None else prev + 0.2 * (seconds - prev)
        self.cycles += 1

    def observe_plain(self, seconds: float):
        self.plain_s = seconds if self.plain_s == 0 else self.plain_s + 0.2 * (seconds - self.plain_s)
        if self.holdoff > 0:
            self.holdoff -= 1

    def survival(self, i: int) -> float:
        return self.kept[i] / self.reached[i] if self.reached[i] else 0.5

    def expected_tokens(self, k: int) -> float:
        e, p = 1.0, 1.0            # the bonus token always lands
        for i in range(k):
            p *= self.survival(i)
            e += p
        return e

    def choose(self) -> int:
        if self.fixed is not None:
            return self.fixed
        if self.holdoff > 0:
            return 0
        if self.cycles < self.PROBE_CYCLES:
            return min(4, self.k_max)
        best_k, best_rate = 0, (1.0 / self.plain_s if self.plain_s > 0 else 0.0)
        base = min(self.cycle_s.values()) if self.cycle_s else None
        for k in range(1, self.k_max + 1):
            t = self.cycle_s.get(k)
            if t is None:
                if base is None:
                    continue
                near = min(self.cycle_s, key=lambda kk: abs(kk - k))
                t = self.cycle_s[near] * (1.0 + 0.05 * (k - near))
            rate = self.expected_tokens(k) / max(t, 1e-9)
            if rate >= best_rate:
                best_k, best_rate = k, rate
        if best_k == 0:
            self.holdoff = self.next_holdoff
            self.next_holdoff = min(self.next_holdoff * 2, 1536)
        else:
            self.next_holdoff = 48
        return best_k


# ------------------------------------------------------------------------------ the cycle
class Speculator:
    """Owned by the engine: replaces the plain decode step for the sequences it is given."""

    def __init__(self, drafter, k: Optional[int] = 4):
        self.drafter = drafter
        self.length = DraftLength(fixed=k)
        self.accepted = 0
        self.rejected = 0
        self.cycles = 0

    def step(self, engine, seqs: List[Sequence]) -> Dict[int, List[int]]:
        """One verify cycle over `seqs` (all in decode state, cache grown by the scheduler's
        lookahead).  Returns the tokens to commit per sequence id, in order."""
        t0 = time.perf_counter()
        live = {s.seq_id for s in engine.sched.running}
        for sid in list(getattr(self.drafter, "known", {})):
            if sid not in live:
                self.drafter.release(sid)       # finished or cancelled elsewhere
        k = min(self.length.choose(), engine.sched.lookahead, DRAFT_MAX)
        drafts = self.drafter.propose(seqs, k) if k > 0 else [[] for _ in seqs]
        items, views, uniforms, states = [], [], [], []
        for s, d in zip(seqs, drafts):
            room = engine.max_ctx - s.total_len - 1
            d = list(d[:max(0, min(k, room))])
            toks = s.tokens
            masks = None
            if getattr(s, "grammar", None) is not None:
                # a constrained request: every row is masked for its own history, drafts the language refuses are cut
                masks, d = s.grammar.rows_for_drafts(d)
            items.append((s, [toks[-1]] + d, len(toks) - 1))
            rng = engine.rngs[s.seq_id]
            st = rng.getstate()
            for i in range(len(d) + 1):
                v = _RowView(s, d[:i])
                if masks is not None:
                    v.mask = masks[i]
                views.append(v)
                uniforms.append(rng.random() if not s.params.greedy else 0.0)
            states.append((rng, st, d))
        logits = engine.runner.forward_rows(items, engine.alloc)
        sampled = engine.runner.sample_rows(logits, views, uniforms)
        # a draft head reads the target's final hidden states of the rows that are about to be committed
        watch = getattr(self.drafter, "observe", None)
        hidden = engine.runner.model.buf.x if watch is not None else None
        out: Dict[int, List[int]] = {}
        row = 0
        n_acc_total = 0
        for s, (rng, st, d) in zip(seqs, states):
            n = len(d) + 1
            mine = sampled[row:row + n]
            row0 = row
            row += n
            commit: List[int] = []
            acc = 0
            for i in range(n):
                commit.append(int(mine[i]))
                if i < len(d) and d[i] == mine[i]:
                    acc += 1
                    continue
                break
            # the generator advances by exactly the number of tokens committed
            rng.setstate(st)
            if not s.params.greedy:
                for _ in commit:
                    rng.random()
            s.accepted_drafts += acc
            s.rejected_drafts += len(d) - acc
            self.accepted += acc
            self.rejected += len(d) - acc
            n_acc_total += acc
            out[s.seq_id] = commit
            if watch is not None:
                watch(s, len(s.tokens) - 1, hidden[row0:row0 + len(commit)], commit)
        self.cycles += 1
        dt = time.perf_counter() - t0
        if k > 0:
            self.length.observe(k, n_acc_total // max(len(seqs), 1), dt, len(seqs))
        else:
            self.length.observe_plain(dt)
        return out

    def status(self) -> dict:
        tot = self.accepted + self.rejected
        return {"attached": True, "drafter": self.drafter.status(), "k": self.length.fixed,
                "cycles": self.cycles, "accepted": self.accepted, "rejected": self.rejected,
                "acceptance": round(self.accepted / tot, 4) if tot else None}


def attach_draft(llm, draft: Optional[str], k: int = 4, method: str = "model") -> dict:
    """Attaches a drafter to a loaded model at run time (`/api/draft/attach`).  `draft` is a GGUF
    path or a built-in shape name; the drafter must share the target's vocabulary.  Under tensor
    parallelism a drafter is attached on every rank at load time instead (`LLM.load(draft=...)`):
    the ranks' schedules have to change at the same step."""
    if hasattr(llm.engine, "_e"):
        raise RuntimeError("under tensor parallelism a drafter is attached on every rank at load time "
                           "([inference] draft_model / --draft-model), not at run time")
    return attach_draft_engine(llm.engine, draft, k, method)


def attach_draft_engine(eng, draft: Optional[str], k: int = 4, method: str = "model", tp_rank: int = 0,
                        tp_size: int = 1, comm=None) -> dict:
    """The same on a bare engine.  Every tensor-parallel rank holds a whole copy of the (small)
    drafter and runs it redundantly, so all ranks propose the same tokens without a collective."""
    del tp_rank, tp_size, comm
    if method == "prompt_lookup" or (not draft and method != "head"):
        drafter = PromptLookupDrafter()
    elif method == "head":
        # a draft head on the target's own hidden states: a directory with an EAGLE or MTP head in safetensors,
        # or "random:eagle" / "random:mtp" for a random-init head of the target's width
        import os

        from .draft_head import HeadDrafter, load_draft_head, random_draft_head

        if eng.weights.tp_size > 1:
            raise ValueError("a draft head reads the whole residual stream: not available under tensor parallelism")
        if draft and os.path.isdir(draft):
            head = load_draft_head(draft, eng.cfg, eng.device)
        else:
            head = random_draft_head(eng.cfg, eng.device, kind=(draft or "random:eagle").split(":")[-1])
        drafter = HeadDrafter(eng.weights, head, max_seqs=eng.sched.max_running, max_ctx=eng.max_ctx,
                              model_id=os.path.basename(os.path.normpath(draft)) if draft else "random")
    else:
        import os

        import torch

        from ..models.config import get_config
        from ..models.weights import random_weights

        if os.path.exists(draft):
            from ..models.loader import load_gguf

            w, _ = load_gguf(draft, eng.device)
            cfg = w.cfg
        else:
            cfg = get_config(draft)
            w = random_weights(cfg, eng.device, seed=1)
        if cfg.vocab != eng.cfg.vocab:
            raise ValueError(f"the drafter's vocabulary ({cfg.vocab}) differs from the target's ({eng.cfg.vocab})")
        drafter = ModelDrafter(cfg, w, max_seqs=eng.sched.max_running, max_ctx=eng.max_ctx,
                               model_id=os.path.basename(draft))
        del torch
    eng.attach_speculator(Speculator(drafter, k))
    return eng.spec.status()


def detach_draft(llm) -> dict:
    llm.engine.detach_speculator()
    return {"attached": False}
