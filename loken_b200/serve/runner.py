"""ModelRunner: turns a scheduler plan into device work.

One step = pinned-host staging of the step's inputs -> one H2D copy -> the decoder forward (a
CUDA graph per (batch bucket, split count) for decode, eager for prefill) -> penalties +
sampler kernels -> one D2H copy of the sampled token ids.  The reference's batch worker does
the same per step (`src/inference/serve/continuous_serve.rs:376-613`: batch padded to a power
of two, device slot / seq_lens / block_table buffers refreshed, graph launch, sampler).
Unlike the reference, sampling always runs on the device and the graph also covers MoE,
sinks and sliding windows.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence as Seq, Tuple

import numpy as np
import torch

from ..models.config import ModelConfig
from ..models.transformer import DecoderModel, StepInputs, make_kv_cache
from ..models.weights import ModelWeights
from ..ops import attention, sampling
from ..ops._lib import Workspace, check, cuda_lib, ptr, stream
from .scheduler import PrefillItem, Sequence

RECENT = 64
RULES = 512        # (token id, value) pairs per row the token-rules kernel takes
FLAG_PENALTY, FLAG_RULES, FLAG_MASK = 1, 2, 4
VERIFY_ROWS = 9    # rows one sequence may carry in a verify step: the carried token + up to 8 drafts


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class ModelRunner:
    def __init__(self, cfg: ModelConfig, weights: ModelWeights, *, num_blocks: int, block_size: int = 16,
                 max_seqs: int = 256, max_tokens: int = 8192, max_ctx: int = 8192, comm=None, moe_runner=None,
                 use_graphs: bool = True, device=None, pipeline=None):
        self.cfg, self.w = cfg, weights
        if pipeline is not None:
            use_graphs = False          # stage hand-offs are point-to-point transfers issued per step
        self.device = device or weights.embed.device
        self.block_size = block_size
        self.max_seqs = max_seqs
        self.max_blocks = (max_ctx + block_size - 1) // block_size
        self.num_slots = num_blocks * block_size
        self.use_graphs = use_graphs
        cap = max(max_tokens, max_seqs)
        samp_cap = min(cap, max_seqs * VERIFY_ROWS)      # sampler rows: one per sequence, or per verify row
        self.samp_cap = samp_cap
        self.kv = make_kv_cache(cfg, weights.n_kv_local, num_blocks, block_size, self.device,
                                layer_range=getattr(weights, "layer_range", None))
        self.model = DecoderModel(weights, self.kv, block_size, cap, comm=comm, moe_runner=moe_runner)
        if pipeline is not None:
            from ..parallel.pipeline import PipelineStage

            self.model = PipelineStage(self.model, pipeline)
        dev = self.device
        i32 = dict(dtype=torch.int32, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        # static device inputs: [tokens | positions | slots | seq_lens] packed so one copy moves them
        self.d_rows = torch.zeros(4, cap, **i32)
        self.d_bt = torch.zeros(max_seqs, self.max_blocks, **i32)
        self.d_samp_f = torch.zeros(5, samp_cap, **f32)     # temperature, top_p, min_p, uniform, penalty
        self.d_topk = torch.zeros(samp_cap, **i32)
        self.d_recent = torch.full((samp_cap, RECENT), -1, **i32)
        self.d_rule_ids = torch.full((samp_cap, RULES), -1, **i32)
        self.d_rule_vals = torch.zeros(samp_cap, RULES, **f32)
        self.d_rule_meta = torch.zeros(2, samp_cap, **i32)   # counts, modes
        self.mask_words = (weights.vocab_local * max(weights.tp_size, 1) + 31) // 32
        # one mask row per sampler row: a constrained sequence's verify rows each carry the mask of their own history
        self.d_mask = torch.zeros(samp_cap, self.mask_words, **i32)
        self.d_mask_has = torch.zeros(samp_cap, **i32)
        self.h_mask = torch.zeros(samp_cap, self.mask_words, dtype=torch.int32, pin_memory=torch.cuda.is_available())
        self.h_mask_has = torch.zeros(samp_cap, dtype=torch.int32, pin_memory=torch.cuda.is_available())
        self.n_mask, self.n_mask_has = self.h_mask.numpy(), self.h_mask_has.numpy()
        self.d_sampled = torch.zeros(cap, **i32)
        self.d_row_seq = torch.zeros(cap, **i32)
        self.h_row_seq = torch.zeros(cap, dtype=torch.int32, pin_memory=torch.cuda.is_available())
        self.n_row_seq = self.h_row_seq.numpy()
        self.d_hist = torch.zeros(max_seqs, 64, **i32)
        self.d_hist_base = torch.zeros(max_seqs, **i32)
        # pinned host mirrors
        pin = dict(pin_memory=torch.cuda.is_available())
        self.h_rows = torch.zeros(4, cap, dtype=torch.int32, **pin)
        self.h_bt = torch.zeros(max_seqs, self.max_blocks, dtype=torch.int32, **pin)
        self.h_samp_f = torch.zeros(5, samp_cap, dtype=torch.float32, **pin)
        self.h_topk = torch.zeros(samp_cap, dtype=torch.int32, **pin)
        self.h_recent = torch.full((samp_cap, RECENT), -1, dtype=torch.int32, **pin)
        self.h_rule_ids = torch.full((samp_cap, RULES), -1, dtype=torch.int32, **pin)
        self.h_rule_vals = torch.zeros(samp_cap, RULES, dtype=torch.float32, **pin)
        self.h_rule_meta = torch.zeros(2, samp_cap, dtype=torch.int32, **pin)
        self.h_sampled = torch.zeros(cap, dtype=torch.int32, **pin)
        self.h_hist = torch.zeros(max_seqs, 64, dtype=torch.int32, **pin)
        self.n_rows, self.n_bt = self.h_rows.numpy(), self.h_bt.numpy()
        self.n_samp_f, self.n_topk, self.n_recent = self.h_samp_f.numpy(), self.h_topk.numpy(), self.h_recent.numpy()
        self.n_rule_ids, self.n_rule_vals = self.h_rule_ids.numpy(), self.h_rule_vals.numpy()
        self.n_rule_meta = self.h_rule_meta.numpy()
        self.end_ids: List[int] = []     # set by the engine: tokens that end a sequence (held back by min_tokens)
        self.last_logits: Optional[torch.Tensor] = None
        self.graphs: Dict[Tuple[int, int, int], torch.cuda.CUDAGraph] = {}
        self.graph_logits: Dict[Tuple[int, int, int], torch.Tensor] = {}
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.kernel_launches = 0        # kernels of this library launched through graph replays
        self.graph_launch_n: Dict[Tuple[int, int, bool], int] = {}
        self.wsp = Workspace.get(dev)

    # ---- staging ----
    def _rules_of(self, s: Sequence):
        """(ids, values, mode) of the token rules that apply to the sequence's next token: logit
        bias, banned words (a multi-token word bans its last token once its head has been
        produced), end tokens held back until min_tokens, and the allow-list
        (`src/inference/sample/token_rules.rs:15-136`)."""
        p = s.params
        if not (p.logit_bias or p.bad_words_ids or p.allowed_token_ids is not None or
                (p.min_tokens and len(s.output) < p.min_tokens)):
            return None
        ninf = float("-inf")
        bias = dict(p.logit_bias)
        for w in p.bad_words_ids:
            if not w:
                continue
            head = w[:-1]
            if not head or s.tokens[-len(head):] == list(head):
                bias[w[-1]] = ninf
        if p.min_tokens and len(s.output) < p.min_tokens:
            for t in list(self.end_ids) + list(p.stop_token_ids):
                bias[t] = ninf
        if p.allowed_token_ids is not None:
            ids = list(dict.fromkeys(p.allowed_token_ids))[:RULES]
            return ids, [bias.get(t, 0.0) for t in ids], 1
        ids = list(bias)[:RULES]
        return ids, [bias[t] for t in ids], 0

    def _stage_sampling(self, seqs: Seq[Sequence], rngs) -> int:
        """Fills the per-row sampler parameters; returns FLAG_PENALTY | FLAG_RULES as used."""
        any_pen = False
        any_rules = False
        for i, s in enumerate(seqs):
            p = s.params
            self.n_samp_f[0, i] = p.temperature
            self.n_samp_f[1, i] = p.top_p
            self.n_samp_f[2, i] = p.min_p
            self.n_samp_f[3, i] = rngs[s.seq_id].random() if not p.greedy else 0.0
            self.n_samp_f[4, i] = p.repeat_penalty
            self.n_topk[i] = p.top_k
            if p.repeat_penalty != 1.0:
                any_pen = True
                toks = s.tokens[-p.repeat_last_n:] if p.repeat_last_n > 0 else []
                self.n_recent[i, :] = -1
                self.n_recent[i, :len(toks)] = toks[-RECENT:]
            rules = self._rules_of(s)
            if rules is None:
                self.n_rule_meta[0, i] = 0
                self.n_rule_meta[1, i] = 0
            else:
                any_rules = True
                ids, vals, mode = rules
                self.n_rule_ids[i, :len(ids)] = ids
                self.n_rule_vals[i, :len(ids)] = vals
                self.n_rule_meta[0, i] = len(ids)
                self.n_rule_meta[1, i] = mode
        n = len(seqs)
        any_mask = False
        if n <= self.samp_cap:
            for i, s in enumerate(seqs):
                g = getattr(s, "grammar", None)
                if g is None:
                    self.n_mask_has[i] = 0
                else:
                    any_mask = True
                    self.n_mask_has[i] = 1
                    m = g.mask()
                    self.n_mask[i, :len(m)] = m
                    self.n_mask[i, len(m):] = 0
        self.d_samp_f[:, :n].copy_(self.h_samp_f[:, :n], non_blocking=True)
        self.d_topk[:n].copy_(self.h_topk[:n], non_blocking=True)
        self.h2d_bytes += 6 * 4 * n
        if any_pen:
            self.d_recent[:n].copy_(self.h_recent[:n], non_blocking=True)
            self.h2d_bytes += n * RECENT * 4
        if any_rules:
            self.d_rule_ids[:n].copy_(self.h_rule_ids[:n], non_blocking=True)
            self.d_rule_vals[:n].copy_(self.h_rule_vals[:n], non_blocking=True)
            self.d_rule_meta[:, :n].copy_(self.h_rule_meta[:, :n], non_blocking=True)
            self.h2d_bytes += n * (RULES * 8 + 8)
        if any_mask:
            self.d_mask[:n].copy_(self.h_mask[:n], non_blocking=True)
            self.d_mask_has[:n].copy_(self.h_mask_has[:n], non_blocking=True)
            self.h2d_bytes += n * (self.mask_words * 4 + 4)
        return (FLAG_PENALTY if any_pen else 0) | (FLAG_RULES if any_rules else 0) | (FLAG_MASK if any_mask else 0)

    def _sample(self, logits: torch.Tensor, n: int, flags: int):
        flags = int(flags)
        self.last_logits = logits
        if flags & FLAG_PENALTY:
            sampling.repeat_penalty_(logits, self.d_recent, self.d_samp_f[4], rows=n)
        if flags & FLAG_RULES:
            sampling.token_rules_(logits, self.d_rule_ids, self.d_rule_vals, self.d_rule_meta[0], self.d_rule_meta[1],
                                  rows=n)
        if flags & FLAG_MASK:
            sampling.token_bitmask_(logits, self.d_mask, self.d_mask_has, rows=min(n, self.samp_cap))
        sampling.sample(logits, self.d_samp_f[0], self.d_samp_f[3], top_k=self.d_topk, top_p=self.d_samp_f[1],
                        min_p=self.d_samp_f[2], out=self.d_sampled, rows=n)

    def logprobs_of(self, rows: Seq[int], tokens: Seq[int], top_n: int):
        """Log-probabilities of the last step's sampled tokens (after penalties and rules, before
        temperature) and the `top_n` most likely alternatives, for the given logits rows."""
        lg = self.last_logits[list(rows)].float()
        lse = torch.logsumexp(lg, dim=-1, keepdim=True)
        lp = lg - lse
        chosen = lp.gather(1, torch.tensor(list(tokens), device=lp.device, dtype=torch.int64)[:, None])[:, 0]
        out = []
        if top_n > 0:
            tv, ti = torch.topk(lp, top_n, dim=-1)
            tv, ti = tv.tolist(), ti.tolist()
        ch = chosen.tolist()
        for j in range(len(ch)):
            out.append((ch[j], list(zip(ti[j], tv[j])) if top_n > 0 else []))
        return out

    def _decode_inputs(self, B: int, nsplit: int) -> StepInputs:
        r = self.d_rows
        return StepInputs(T=B, tokens=r[0], positions=r[1], slots=r[2], mode="decode", block_table=self.d_bt,
                          seq_lens=r[3], nsplit=nsplit)

    def _advance(self, B: int):
        r = self.d_rows
        check(cuda_lib().lk_advance_decode(ptr(r[0]), ptr(r[1]), ptr(r[2]), ptr(r[3]), ptr(self.d_sampled),
                                           ptr(self.d_bt), self.max_blocks, self.block_size, B,
                                           C.c_longlong(self.num_slots), ptr(self.d_hist), self.d_hist.shape[1],
                                           ptr(self.d_hist_base), ptr(self.wsp.status), stream()),
              "lk_advance_decode")

    def _decode_body(self, Bp: int, nsplit: int, with_penalty: bool):
        logits = self.model.forward(self._decode_inputs(Bp, nsplit))
        self._sample(logits, Bp, with_penalty)
        self._advance(Bp)

    def _run_decode_graph(self, Bp: int, nsplit: int, with_penalty: bool):
        if not self.use_graphs:
            self._decode_body(Bp, nsplit, with_penalty)
            return
        key = (Bp, nsplit, int(with_penalty))
        g = self.graphs.get(key)
        if g is None:
            # the graph is captured after an eager warm-up of the same shape, on a side stream;
            # the warm-up advances the static inputs, so they are saved and put back
            saved = (self.d_rows.clone(), self.d_sampled.clone())
            self._decode_body(Bp, nsplit, with_penalty)
            torch.cuda.synchronize()
            self.d_rows.copy_(saved[0])
            g = torch.cuda.CUDAGraph()
            from ..ops._lib import launch_count

            n0 = launch_count()
            with torch.cuda.graph(g):
                self._decode_body(Bp, nsplit, with_penalty)
            self.graph_launch_n[key] = launch_count() - n0
            self.graph_logits[key] = self.last_logits
            self.graphs[key] = g
            self.d_rows.copy_(saved[0])
            self.d_sampled.copy_(saved[1])
            # the capture-time warm-up wrote KV rows for the staged slots; the replay rewrites them
        g.replay()
        self.last_logits = self.graph_logits[key]
        self.kernel_launches += self.graph_launch_n[key]

    # ---- decode ----
    def _stage_decode(self, seqs: Seq[Sequence], alloc) -> Tuple[int, int]:
        B = len(seqs)
        Bp = min(_bucket(B), self.d_rows.shape[1])
        nr, nbt = self.n_rows, self.n_bt
        max_len = 1
        for i, s in enumerate(seqs):
            pos = s.total_len - 1
            nr[0, i] = s.tokens[-1]
            nr[1, i] = pos
            nr[2, i] = alloc.slot(s.seq_id, pos)
            nr[3, i] = pos + 1
            bt = alloc.block_table(s.seq_id)
            nbt[i, :len(bt)] = bt
            max_len = max(max_len, pos + 1)
        if Bp > B:
            nr[0, B:Bp] = 0
            nr[1, B:Bp] = 0
            nr[2, B:Bp] = -1
            nr[3, B:Bp] = 0
        self.d_rows[:, :Bp].copy_(self.h_rows[:, :Bp], non_blocking=True)
        self.d_bt[:B].copy_(self.h_bt[:B], non_blocking=True)
        self.h2d_bytes += 16 * Bp + B * self.max_blocks * 4
        # split count: fixed per (bucket, context bucket of 1024) so graphs are reused
        ctx_bucket = (max_len + 1023) // 1024 * 1024
        nsplit = attention.pick_decode_splits(Bp, self.w.n_kv_local, ctx_bucket)
        return Bp, nsplit

    def decode(self, seqs: Seq[Sequence], alloc, rngs) -> List[int]:
        """One decode step for `seqs` (each feeds its last token); returns one new token each."""
        B = len(seqs)
        Bp, nsplit = self._stage_decode(seqs, alloc)
        pen = self._stage_sampling(seqs, rngs)
        self._run_decode_graph(Bp, nsplit, pen)
        self.h_sampled[:B].copy_(self.d_sampled[:B], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += 4 * B
        return self.h_sampled[:B].tolist()

    def decode_multi(self, seqs: Seq[Sequence], alloc, rngs, steps: int) -> List[List[int]]:
        """`steps` decode steps back to back with no host round trip in between: the sampled
        token is fed back on the device.  The allocator must already hold blocks for
        `steps` more positions of every sequence.  Uniforms are drawn once per call and
        reused by each of its steps only for greedy rows; sampled rows take steps == 1."""
        B = len(seqs)
        assert steps <= self.d_hist.shape[1]
        Bp, nsplit = self._stage_decode(seqs, alloc)
        pen = self._stage_sampling(seqs, rngs)
        self.d_hist_base[:Bp].copy_(self.d_rows[1, :Bp])
        for _ in range(steps):
            self._run_decode_graph(Bp, nsplit, pen)
        self.h_hist[:B, :steps].copy_(self.d_hist[:B, :steps], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += 4 * B * steps
        return self.h_hist[:B, :steps].tolist()

    # ---- several rows per sequence through the decode kernels (verification, draft catch-up) ----
    def forward_rows(self, items, alloc, last_only: bool = False, embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        """items: (seq, tokens, start) — feed `tokens` at positions start.. of `seq`, whose cache
        already holds positions < start and has blocks for the new rows.  Every row attends to
        the keys at or before its own position (rows of one sequence see the rows before them:
        all K/V are written before any attention runs).  Returns logits [rows or items, vocab].
        `embeds` [rows, hidden] bf16 takes the embedding table's place for every row (a draft head's input)."""
        nr, nbt = self.n_rows, self.n_bt
        T, max_len, last = 0, 1, []
        for j, (s, toks, start) in enumerate(items):
            n = len(toks)
            nr[0, T:T + n] = toks
            nr[1, T:T + n] = np.arange(start, start + n, dtype=np.int32)
            nr[2, T:T + n] = alloc.slots_for_range(s.seq_id, start, start + n)
            nr[3, T:T + n] = np.arange(start + 1, start + n + 1, dtype=np.int32)
            self.n_row_seq[T:T + n] = j
            bt = alloc.block_table(s.seq_id)
            nbt[j, :len(bt)] = bt
            max_len = max(max_len, start + n)
            T += n
            last.append(T - 1)
        assert T <= self.d_rows.shape[1], "more rows than the runner's max_tokens"
        nb = len(items)
        self.d_rows[:, :T].copy_(self.h_rows[:, :T], non_blocking=True)
        self.d_row_seq[:T].copy_(self.h_row_seq[:T], non_blocking=True)
        self.d_bt[:nb].copy_(self.h_bt[:nb], non_blocking=True)
        self.h2d_bytes += 20 * T + nb * self.max_blocks * 4
        ctx_bucket = (max_len + 1023) // 1024 * 1024
        nsplit = attention.pick_decode_splits(T, self.w.n_kv_local, ctx_bucket)
        r = self.d_rows
        lr, n_l = None, 0
        if last_only:
            lr = torch.tensor(last, dtype=torch.int64, device=self.device)
            n_l = len(last)
        inp = StepInputs(T=T, tokens=r[0], positions=r[1], slots=r[2], mode="decode", block_table=self.d_bt,
                         seq_lens=r[3], nsplit=nsplit, row_seq=self.d_row_seq, logit_rows=lr, n_logit_rows=n_l,
                         embed_overrides=[(0, embeds[:T])] if embeds is not None else None)
        return self.model.forward(inp)

    def forward_hidden(self, seq_id: int, hidden: torch.Tensor, pos0: int, alloc, lo: int, hi: int,
                       last: bool) -> torch.Tensor:
        """A pipeline segment's forward: `hidden` [T, H] bf16 is the residual stream of positions
        pos0 .. pos0 + T of one sequence as the previous segment left it; layers [lo, hi) run over it (every
        row attends to the cached keys of earlier positions and to the rows before it).  Returns the
        residual stream after layer hi - 1, or, with `last`, the fp32 logits of the final row."""
        T = hidden.shape[0]
        assert T <= self.d_rows.shape[1], "more rows than the runner's max_tokens"
        nr = self.n_rows
        nr[0, :T] = 0
        nr[1, :T] = np.arange(pos0, pos0 + T, dtype=np.int32)
        nr[2, :T] = alloc.slots_for_range(seq_id, pos0, pos0 + T)
        nr[3, :T] = np.arange(pos0 + 1, pos0 + T + 1, dtype=np.int32)
        self.n_row_seq[:T] = 0
        bt = alloc.block_table(seq_id)
        self.n_bt[0, :len(bt)] = bt
        self.d_rows[:, :T].copy_(self.h_rows[:, :T], non_blocking=True)
        self.d_row_seq[:T].copy_(self.h_row_seq[:T], non_blocking=True)
        self.d_bt[:1].copy_(self.h_bt[:1], non_blocking=True)
        self.h2d_bytes += 20 * T + self.max_blocks * 4 + hidden.numel() * 2
        ctx_bucket = (pos0 + T + 1023) // 1024 * 1024
        nsplit = attention.pick_decode_splits(T, self.w.n_kv_local, ctx_bucket)
        r = self.d_rows
        lr = torch.tensor([T - 1], dtype=torch.int64, device=self.device) if last else None
        inp = StepInputs(T=T, tokens=r[0], positions=r[1], slots=r[2], mode="decode", block_table=self.d_bt,
                         seq_lens=r[3], nsplit=nsplit, row_seq=self.d_row_seq, logit_rows=lr,
                         n_logit_rows=1 if last else 0)
        m = self.model
        m.buf.x[:T].copy_(hidden)
        m._delta_local = False
        delta = m.run_layers(inp, lo, hi)
        if last:
            return m.head(inp, delta).clone()
        return m.fold_residual(inp, delta).clone()

    def sample_rows(self, logits: torch.Tensor, views, uniforms: Seq[float]) -> List[int]:
        """Samples one token per logits row.  `views[i]` looks like a Sequence (params, tokens,
        output) and describes the history row i is sampled after."""
        n = len(views)
        assert n <= self.samp_cap
        # rows of one sequence differ in history (the drafts before them), so they are staged row by row
        any_pen = any_rules = False
        for i, v in enumerate(views):
            p = v.params
            self.n_samp_f[0, i] = p.temperature
            self.n_samp_f[1, i] = p.top_p
            self.n_samp_f[2, i] = p.min_p
            self.n_samp_f[3, i] = uniforms[i] if not p.greedy else 0.0
            self.n_samp_f[4, i] = p.repeat_penalty
            self.n_topk[i] = p.top_k
            if p.repeat_penalty != 1.0:
                any_pen = True
                toks = v.tokens[-p.repeat_last_n:] if p.repeat_last_n > 0 else []
                self.n_recent[i, :] = -1
                self.n_recent[i, :len(toks)] = toks[-RECENT:]
            rules = self._rules_of(v)
            if rules is None:
                self.n_rule_meta[0, i] = 0
                self.n_rule_meta[1, i] = 0
            else:
                any_rules = True
                ids, vals, mode = rules
                self.n_rule_ids[i, :len(ids)] = ids
                self.n_rule_vals[i, :len(ids)] = vals
                self.n_rule_meta[0, i] = len(ids)
                self.n_rule_meta[1, i] = mode
        self.d_samp_f[:, :n].copy_(self.h_samp_f[:, :n], non_blocking=True)
        self.d_topk[:n].copy_(self.h_topk[:n], non_blocking=True)
        if any_pen:
            self.d_recent[:n].copy_(self.h_recent[:n], non_blocking=True)
        if any_rules:
            self.d_rule_ids[:n].copy_(self.h_rule_ids[:n], non_blocking=True)
            self.d_rule_vals[:n].copy_(self.h_rule_vals[:n], non_blocking=True)
            self.d_rule_meta[:, :n].copy_(self.h_rule_meta[:, :n], non_blocking=True)
        any_mask = False
        for i, v in enumerate(views):
            m = getattr(v, "mask", None)          # the grammar's mask after this row's history (serve/speculative.py)
            if m is None:
                self.n_mask_has[i] = 0
            else:
                any_mask = True
                self.n_mask_has[i] = 1
                self.n_mask[i, :len(m)] = m
                self.n_mask[i, len(m):] = 0
        if any_mask:
            self.d_mask[:n].copy_(self.h_mask[:n], non_blocking=True)
            self.d_mask_has[:n].copy_(self.h_mask_has[:n], non_blocking=True)
        flags = (FLAG_PENALTY if any_pen else 0) | (FLAG_RULES if any_rules else 0) | (FLAG_MASK if any_mask else 0)
        self._sample(logits, n, flags)
        self.h_sampled[:n].copy_(self.d_sampled[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += 4 * n
        return self.h_sampled[:n].tolist()

    # ---- prefill ----
    def prefill(self, items: Seq[PrefillItem], alloc, rngs) -> Dict[int, int]:
        """Runs every item's [start, end) rows in one variable-length forward; returns a sampled
        token for each sequence whose prompt is now complete."""
        nr = self.n_rows
        T = 0
        q_lens, kv_lens, last_rows, done = [], [], [], []
        overrides = []
        for j, it in enumerate(items):
            s, n = it.seq, it.end - it.start
            toks = s.tokens
            pe = getattr(s, "prompt_embeds", None)
            if pe is not None and it.start < len(s.prompt):
                p_end = min(it.end, len(s.prompt))
                overrides.append((T, pe[it.start:p_end]))
            nr[0, T:T + n] = toks[it.start:it.end]
            nr[1, T:T + n] = np.arange(it.start, it.end, dtype=np.int32)
            nr[2, T:T + n] = alloc.slots_for_range(s.seq_id, it.start, it.end)
            bt = alloc.block_table(s.seq_id)
            self.n_bt[j, :len(bt)] = bt
            q_lens.append(n)
            kv_lens.append(it.end)
            if it.is_last_chunk:
                last_rows.append(T + n - 1)
                done.append(s)
            T += n
        assert T <= self.d_rows.shape[1], "prefill step larger than the runner's max_tokens"
        nb = len(items)
        self.d_rows[:3, :T].copy_(self.h_rows[:3, :T], non_blocking=True)
        self.d_bt[:nb].copy_(self.h_bt[:nb], non_blocking=True)
        self.h2d_bytes += 12 * T + nb * self.max_blocks * 4
        plan = attention.plan_prefill(q_lens, kv_lens, self.cfg.n_q // self.cfg.n_kv, self.device)
        r = self.d_rows
        n_l = len(last_rows)
        lr = torch.tensor(last_rows if last_rows else [0], dtype=torch.int64, device=self.device)
        inp = StepInputs(T=T, tokens=r[0], positions=r[1], slots=r[2], mode="prefill", block_table=self.d_bt,
                         plan=plan, logit_rows=lr, n_logit_rows=max(n_l, 1), embed_overrides=overrides or None)
        logits = self.model.forward(inp)
        if not done:
            return {}
        pen = self._stage_sampling(done, rngs)
        self._sample(logits, n_l, pen)
        self.h_sampled[:n_l].copy_(self.d_sampled[:n_l], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += 4 * n_l
        out = self.h_sampled[:n_l].tolist()
        return {s.seq_id: t for s, t in zip(done, out)}

    def kv_shift(self, src: Seq[int], dst: Seq[int], delta: Seq[int]):
        """Moves cache positions `src` -> `dst` on every layer this rank holds, turning key i by delta[i]
        positions (`ops/rows.py:kv_shift`)."""
        from ..ops import rows

        dev = self.device
        t = torch.tensor([list(src), list(dst), list(delta)], dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        m = self.model
        for cache in m.kv:
            if cache is not None:
                rows.kv_shift(cache, t[0], t[1], t[2], m.w.inv_freq, rope_dim=self.cfg.rope_dim or self.cfg.head_dim,
                              pairing=self.cfg.rope_pairing)
        self.h2d_bytes += 12 * len(src)

    def layer_perf(self, alloc, n_tokens: int = 1):
        sid = -1 - len(alloc.seqs)
        n = max(1, min(n_tokens, self.max_seqs))
        if not alloc.allocate(sid, 1):
            raise MemoryError("[oom] no cache block for the profiling pass")
        try:
            slot = alloc.slot(sid, 0)
            self.n_rows[0, :n] = 0
            self.n_rows[1, :n] = 0
            self.n_rows[2, :n] = slot
            self.n_rows[3, :n] = 1
            bt = alloc.block_table(sid)
            for j in range(n):
                self.n_bt[j, :len(bt)] = bt
            self.d_rows[:, :n].copy_(self.h_rows[:, :n], non_blocking=True)
            self.d_bt[:n].copy_(self.h_bt[:n], non_blocking=True)
            inp = self._decode_inputs(n, 1)
            self.model.profile_layers(inp)          # warm-up
            return self.model.profile_layers(inp)
        finally:
            alloc.free(sid)

    # ---- embeddings ----
    def embed(self, tokens: Seq[int], alloc, pooling: str = "last") -> torch.Tensor:
        """Hidden state of a prompt after the output norm, as a unit vector: the last token's
        ("last") or the mean over the prompt ("mean").  Uses scratch cache blocks that are
        released before returning."""
        n = len(tokens)
        assert 0 < n <= self.d_rows.shape[1]
        sid = -1 - len(alloc.seqs)          # a scratch id no request uses
        if not alloc.allocate(sid, n):
            raise MemoryError("[oom] no cache blocks for the embedding pass")
        try:
            nr = self.n_rows
            nr[0, :n] = tokens
            nr[1, :n] = np.arange(n, dtype=np.int32)
            nr[2, :n] = alloc.slots_for_range(sid, 0, n)
            bt = alloc.block_table(sid)
            self.n_bt[0, :len(bt)] = bt
            self.d_rows[:3, :n].copy_(self.h_rows[:3, :n], non_blocking=True)
            self.d_bt[:1].copy_(self.h_bt[:1], non_blocking=True)
            plan = attention.plan_prefill([n], [n], self.cfg.n_q // self.cfg.n_kv, self.device)
            r = self.d_rows
            rows_idx = torch.arange(n, dtype=torch.int64, device=self.device) if pooling == "mean" else \
                torch.tensor([n - 1], dtype=torch.int64, device=self.device)
            inp = StepInputs(T=n, tokens=r[0], positions=r[1], slots=r[2], mode="prefill", block_table=self.d_bt,
                             plan=plan, logit_rows=rows_idx, n_logit_rows=int(rows_idx.numel()))
            self.model.forward(inp)
            h = self.model.buf.hsel[:rows_idx.numel()].float()
            v = h.mean(0) if pooling == "mean" else h[0]
            v = v / v.norm().clamp_min(1e-12)
            torch.cuda.current_stream().synchronize()
            return v.cpu()
        finally:
            alloc.free(sid)

    def check_status(self):
        code = self.wsp.read_status()
        if code:
            self.wsp.clear_status()
            raise RuntimeError(f"device status word = {code & 0xff} (site {code >> 8})")
