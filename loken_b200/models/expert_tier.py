"""Host-streamed experts: the routed experts of a mixture live in pinned host memory and only a
fixed number of slots per layer on the GPU.

Per layer and step: route on the device, read the chosen expert ids back (a few hundred bytes),
bring the missing experts into slots with `cudaMemcpyAsync` on a side stream (event-ordered
against the compute stream), rewrite the routed ids to slot numbers with a device table, and run
the ordinary grouped GEMMs over the slot stacks.  A batch that routes to more distinct experts
than there are slots is processed in rounds, each round accumulating into the output.

Slot policy, after the reference's expert tier (`src/inference/generic_transformer/expert_tier.rs:1-28`,
`:97-113`): every expert has a heat that decays (x0.7 every 10 tokens) and grows by its routed
count; a missing expert that is needed now always gets a slot, evicting the coldest slot that is
not needed in this round.  As in the reference, misses of a decode-size step are computed on the host
cores beside the card (`cpu/moe_host.py`, over the same pinned planes the copies read): a pair's expert is
read once from host memory instead of crossing the bus, the resident experts' pairs run on the GPU as
usual, and the hottest missing expert is promoted into the coldest idle slot behind the step.  Larger
steps take the copies, in rounds.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..ops import quant
from .moe import MoeRunner, MoeWeights


def _rows_of(w, lo: int, hi: int):
    """Row slice [lo, hi) of a stacked expert weight (bf16 tensor or QuantWeight planes)."""
    if isinstance(w, torch.Tensor):
        return [w[lo:hi]]
    return [w.codes[lo:hi], w.scales[lo:hi]]


@dataclass
class TierStats:
    hits: int = 0
    misses: int = 0
    rounds: int = 0
    bytes_copied: int = 0
    host_pairs: int = 0          # (token, expert) pairs computed on the host cores

    def hit_rate(self) -> Optional[float]:
        n = self.hits + self.misses
        return self.hits / n if n else None


class TieredLayer:
    """One layer's experts: full set pinned on the host, `slots` of them resident on the device."""

    def __init__(self, moe: MoeWeights, slots: int, rows_gu: int, rows_dn: int):
        assert moe.e_lo == 0, "host streaming holds the whole expert set on one rank"
        self.E = moe.e_cnt
        self.S = min(slots, self.E)
        self.rows_gu, self.rows_dn = rows_gu, rows_dn
        dev = moe.router_w.device
        pin = lambda t: t.cpu().pin_memory() if torch.cuda.is_available() else t.cpu()
        self.host_gu = [pin(p) for p in _rows_of(moe.gate_up, 0, self.E * rows_gu)]
        self.host_dn = [pin(p) for p in _rows_of(moe.down, 0, self.E * rows_dn)]
        self.host_gub = pin(moe.gate_up_b) if moe.gate_up_b is not None else None
        self.host_dnb = pin(moe.down_b) if moe.down_b is not None else None
        # the same pinned buffers as stacks the host kernel reads
        as_w = lambda w, parts: parts[0] if isinstance(w, torch.Tensor) else quant.QuantWeight(
            w.aq_fmt, w.ggml_type, w.rows, w.K, parts[0], parts[1])
        self.host_gu_w, self.host_dn_w = as_w(moe.gate_up, self.host_gu), as_w(moe.down, self.host_dn)
        from ..cpu.moe_host import plane_format

        self.host_ok = plane_format(self.host_gu_w) is not None and plane_format(self.host_dn_w) is not None

        def slot_stack(w, rows):
            if isinstance(w, torch.Tensor):
                return w[:self.S * rows].clone()
            return quant.QuantWeight(w.aq_fmt, w.ggml_type, self.S * rows, w.K, w.codes[:self.S * rows].clone(),
                                     w.scales[:self.S * rows].clone())

        self.dev = MoeWeights(moe.router_w, moe.router_b, slot_stack(moe.gate_up, rows_gu),
                              slot_stack(moe.down, rows_dn),
                              moe.gate_up_b[:self.S].clone() if moe.gate_up_b is not None else None,
                              moe.down_b[:self.S].clone() if moe.down_b is not None else None, 0, self.S, moe.fmt)
        self.slot_expert: List[int] = list(range(self.S))          # expert in each slot
        self.expert_slot: Dict[int, int] = {e: e for e in range(self.S)}
        self.heat = [0.0] * self.E
        self.table = torch.full((self.E,), self.S, dtype=torch.int32, device=dev)   # expert -> slot, S = absent
        self.table[:self.S] = torch.arange(self.S, dtype=torch.int32, device=dev)
        self.tokens_since_decay = 0

    def expert_bytes(self) -> int:
        n = 0
        for planes, rows in ((self.host_gu, self.rows_gu), (self.host_dn, self.rows_dn)):
            for p in planes:
                n += rows * p.stride(0) * p.element_size()
        return n

    def load(self, e: int, slot: int, stream: torch.cuda.Stream) -> int:
        """Copies expert `e` into `slot` on `stream`; returns bytes moved."""
        moved = 0
        with torch.cuda.stream(stream):
            for host, devw, rows in ((self.host_gu, self.dev.gate_up, self.rows_gu),
                                     (self.host_dn, self.dev.down, self.rows_dn)):
                for hp, dp in zip(host, _rows_of(devw, slot * rows, (slot + 1) * rows)):
                    src = hp[e * rows:(e + 1) * rows]
                    dp.copy_(src, non_blocking=True)
                    moved += src.numel() * src.element_size()
            if self.host_gub is not None:
                self.dev.gate_up_b[slot].copy_(self.host_gub[e], non_blocking=True)
                self.dev.down_b[slot].copy_(self.host_dnb[e], non_blocking=True)
        old = self.slot_expert[slot]
        if old in self.expert_slot and self.expert_slot[old] == slot:
            del self.expert_slot[old]
        self.slot_expert[slot] = e
        self.expert_slot[e] = slot
        return moved

    def decay(self, tokens: int):
        self.tokens_since_decay += tokens
        while self.tokens_since_decay >= 10:
            self.tokens_since_decay -= 10
            self.heat = [h * 0.7 for h in self.heat]


class TieredMoeRunner(MoeRunner):
    """`MoeRunner` whose expert stacks are slot caches over host memory."""
    plans_on_host = True        # the round plan reads the router's choices on the host: no CUDA-graph capture

    HOST_PAIRS_MAX = 64          # up to this many pairs a step's misses are computed on the host; 0: always copy

    def __init__(self, cfg, weights, cap: int, comm=None, slots: int = 8, host_threads: int = 0):
        super().__init__(cfg, weights, cap, comm)
        import os

        self.host_threads = host_threads or max(1, min(32, (os.cpu_count() or 8) // 2))
        I, H = cfg.expert_intermediate, cfg.hidden
        self.layers: Dict[int, TieredLayer] = {}
        for il, lw in enumerate(weights.layers):
            if lw is None or lw.moe is None:
                continue
            self.layers[il] = TieredLayer(lw.moe, slots, 2 * I, H)
            # the full device stacks are no longer needed: the layer keeps only its slots
            lw.moe = self.layers[il].dev
        from .moe import MoePlan

        S = next(iter(self.layers.values())).S
        self.plan = MoePlan(cap, cfg.top_k, S, self.device)
        self.ids_slot = torch.zeros_like(self.plan.ids)
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self.stats = TierStats()

    def forward(self, il: int, moe: MoeWeights, h: torch.Tensor, out: torch.Tensor, T: int):
        import ctypes as C

        from ..ops._lib import check, cuda_lib, ptr, stream

        tl = self.layers[il]
        cfg, pl = self.cfg, self.plan
        self.route(tl.dev, h, T)
        ids = pl.ids[:T].cpu()                       # synchronises: the round plan is made on the host
        counts: Dict[int, int] = {}
        for e in ids.flatten().tolist():
            counts[e] = counts.get(e, 0) + 1
        tl.decay(T)
        for e, c in counts.items():
            tl.heat[e] += c
        needed = sorted(counts, key=lambda e: -counts[e])
        S = tl.S
        if self.HOST_PAIRS_MAX and T * cfg.top_k <= self.HOST_PAIRS_MAX and tl.host_ok \
                and (self.comm is None or self.comm.size == 1):
            return self._forward_with_host_misses(tl, h, out, T, ids, counts)
        first = True
        for r0 in range(0, len(needed), S):
            chunk = needed[r0:r0 + S]
            inround = set(chunk)
            missing = [e for e in chunk if e not in tl.expert_slot]
            self.stats.hits += len(chunk) - len(missing)
            self.stats.misses += len(missing)
            if missing:
                # coldest slots whose expert is not needed in this round go first
                victims = sorted((s for s in range(S) if tl.slot_expert[s] not in inround),
                                 key=lambda s: tl.heat[tl.slot_expert[s]])
                self.copy_stream.wait_stream(torch.cuda.current_stream(self.device))   # slots may still be read
                for e, s in zip(missing, victims):
                    self.stats.bytes_copied += tl.load(e, s, self.copy_stream)
                torch.cuda.current_stream(self.device).wait_stream(self.copy_stream)
            tbl = [S] * tl.E
            for e in chunk:
                tbl[e] = tl.expert_slot[e]
            tl.table.copy_(torch.tensor(tbl, dtype=torch.int32), non_blocking=False)
            torch.index_select(tl.table, 0, pl.ids[:T].flatten().long(), out=self.ids_slot[:T].view(-1))
            P = T * cfg.top_k
            from .moe import pick_group_bn

            pl.bn = pick_group_bn(P, S, not isinstance(tl.dev.gate_up, torch.Tensor))
            check(cuda_lib().lk_moe_plan(ptr(self.ids_slot), P, S + 1, 0, S, pl.bn, pl.max_tiles, ptr(pl.offsets),
                                         ptr(pl.pair_row), ptr(pl.tile_expert), ptr(pl.tile_row0), ptr(pl.tile_rows),
                                         ptr(pl.ntiles), ptr(self.wsp.status), stream()), "lk_moe_plan")
            self.experts(tl.dev, h, T, out, accumulate=not first)
            first = False
            self.stats.rounds += 1
        if self.comm is not None and self.comm.size > 1:
            self.comm.all_reduce(out, T)
        del C

    def _forward_with_host_misses(self, tl: TieredLayer, h: torch.Tensor, out: torch.Tensor, T: int, ids: torch.Tensor,
                                  counts: Dict[int, int]):
        """A decode-size step: pairs of resident experts on the GPU (one round, nothing copied for it), pairs of
        missing experts on the host cores; then the hottest missing expert takes the coldest idle slot."""
        from ..cpu.moe_host import moe_pairs
        from ..ops._lib import check, cuda_lib, ptr, stream
        from .moe import pick_group_bn

        cfg, pl, S = self.cfg, self.plan, tl.S
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self.copy_stream)                       # a promotion of an earlier step may still be landing
        resident = [e for e in counts if e in tl.expert_slot]
        missing = [e for e in counts if e not in tl.expert_slot]
        self.stats.hits += len(resident)
        self.stats.misses += len(missing)
        if resident:
            tbl = [S] * tl.E
            for e in resident:
                tbl[e] = tl.expert_slot[e]
            tl.table.copy_(torch.tensor(tbl, dtype=torch.int32), non_blocking=False)
            torch.index_select(tl.table, 0, pl.ids[:T].flatten().long(), out=self.ids_slot[:T].view(-1))
            P = T * cfg.top_k
            pl.bn = pick_group_bn(P, S, not isinstance(tl.dev.gate_up, torch.Tensor))
            check(cuda_lib().lk_moe_plan(ptr(self.ids_slot), P, S + 1, 0, S, pl.bn, pl.max_tiles, ptr(pl.offsets),
                                         ptr(pl.pair_row), ptr(pl.tile_expert), ptr(pl.tile_row0), ptr(pl.tile_rows),
                                         ptr(pl.ntiles), ptr(self.wsp.status), stream()), "lk_moe_plan")
            self.experts(tl.dev, h, T, out, accumulate=False)
            self.stats.rounds += 1
        else:
            out[:T].zero_()
        if not missing:
            return
        miss = set(missing)
        wts = pl.wts[:T].cpu()
        x = h[:T].float().cpu()
        tok, exp, w = [], [], []
        for t in range(T):
            for j in range(cfg.top_k):
                e = int(ids[t, j])
                if e in miss:
                    tok.append(t)
                    exp.append(e)
                    w.append(float(wts[t, j]))
        y = torch.zeros(T, cfg.hidden, dtype=torch.float32)
        moe_pairs(tl.host_gu_w, tl.host_dn_w, x, tok, exp, w, H=cfg.hidden, I=cfg.expert_intermediate, out=y,
                  gu_bias=tl.host_gub, dn_bias=tl.host_dnb, glu=(cfg.glu_mode, cfg.glu_alpha, cfg.glu_limit),
                  threads=self.host_threads)
        out[:T] += y.to(self.device).to(out.dtype)
        self.stats.host_pairs += len(tok)
        # promotion: the hottest missing expert replaces the coldest slot that this step did not use, if it is hotter
        idle = [s for s in range(S) if tl.slot_expert[s] not in counts]
        if idle:
            hot = max(missing, key=lambda e: tl.heat[e])
            victim = min(idle, key=lambda s: tl.heat[tl.slot_expert[s]])
            if tl.heat[hot] > tl.heat[tl.slot_expert[victim]]:
                self.copy_stream.wait_stream(cur)               # the slot may still be read by an earlier launch
                self.stats.bytes_copied += tl.load(hot, victim, self.copy_stream)

    def status(self) -> dict:
        tl = next(iter(self.layers.values()))
        return {"slots": tl.S, "experts": tl.E, "hit_rate": self.stats.hit_rate(), "rounds": self.stats.rounds,
                "bytes_copied": self.stats.bytes_copied, "expert_bytes": tl.expert_bytes(),
                "host_pairs": self.stats.host_pairs}
