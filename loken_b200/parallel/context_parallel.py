"""Attention over a context that is held in ranges of positions, one range per GPU.

Each range answers a query on its own with a *part*: per query head and row the maximum of the scores it
saw, the sum of their exponentials taken from that maximum, and the values weighed by those exponentials
(not yet divided).  Parts of all the ranges make the attention over the whole context once each is
rescaled to the greatest maximum, so no range ever needs the keys of another, and what crosses NVLink per
layer is `rows x heads x (head_dim + 2)` floats instead of the cache
(reference: `src/inference/generic_transformer/context_parallel.rs:1-140`: `partial`, `merge`, `finish`).

    ranges = plan_ranges(total_positions, world)         # contiguous, 16-aligned: whole cache blocks
    part   = decode_part(q, cache, block_table, lens)    # this rank's range, on the decode kernel
    out    = gather_merge(part, group)                   # the same [rows, n_q * hd] on every rank

`partial` is the same computation in plain PyTorch (any device, causal mask by absolute positions, grouped
heads): the definition the kernel path is tested against, and the path prompts take.  Maxima here are in
natural-log units; the kernel's parts carry log2 units and are converted on the way in.  Attention sinks
join at `finish` (a sink adds exp(sink - max) to the sum and nothing to the values).  Sliding-window layers
are not split: a window already bounds what a layer reads.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

LN2 = math.log(2.0)


@dataclass
class Part:
    max: torch.Tensor     # [rows, heads, 1]   natural-log units of the scaled scores; -inf where no key was seen
    sum: torch.Tensor     # [rows, heads, 1]
    out: torch.Tensor     # [rows, heads, hd]  sum_j exp(s_j - max) v_j

    def to(self, device) -> "Part":
        return Part(self.max.to(device), self.sum.to(device), self.out.to(device))


def plan_ranges(total: int, world: int, align: int = 16) -> List[Tuple[int, int]]:
    """`world` contiguous ranges [lo, hi) covering [0, total), every boundary but the last a multiple of `align`
    (whole cache blocks), sizes as equal as that allows.  Ranks beyond the data get empty ranges."""
    if world <= 0:
        raise ValueError("world must be positive")
    units = (total + align - 1) // align
    base, extra = divmod(units, world)
    out, lo = [], 0
    for r in range(world):
        hi = min(total, lo + (base + (1 if r < extra else 0)) * align)
        out.append((lo, hi))
        lo = hi
    return out


def owner_of(position: int, ranges: Sequence[Tuple[int, int]]) -> int:
    """The rank whose range holds `position`; a position past the end belongs to the last rank with room to
    grow (the newest token is appended there)."""
    for r, (lo, hi) in enumerate(ranges):
        if lo <= position < hi:
            return r
    return len(ranges) - 1


def partial(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, q_pos: int, k_pos: int) -> Part:
    """The part of q [rows, n_q, hd] over keys / values [t, n_kv, hd] of one range.  Row i stands at position
    q_pos + i, key j at k_pos + j; a key past a row's position is masked out."""
    rows, n_q, hd = q.shape
    t, n_kv, _ = k.shape
    g = n_q // max(n_kv, 1)
    qf = q.float().view(rows, n_kv, g, hd)
    kf, vf = k.float(), v.float()
    s = torch.einsum("rngd,tnd->rngt", qf, kf) * scale                       # [rows, n_kv, g, t]
    qi = torch.arange(rows, device=q.device)[:, None] + q_pos
    kj = torch.arange(t, device=q.device)[None, :] + k_pos
    s = s.masked_fill((kj > qi)[:, None, None, :], float("-inf"))
    if t == 0:
        mx = torch.full((rows, n_kv, g, 1), float("-inf"), device=q.device)
    else:
        mx = s.amax(-1, keepdim=True)
    safe = torch.where(torch.isfinite(mx), mx, torch.zeros_like(mx))          # a row that saw no key: weights 0, no NaN
    w = torch.exp(s - safe)
    w = torch.where(torch.isfinite(s), w, torch.zeros_like(w))
    out = torch.einsum("rngt,tnd->rngd", w, vf)
    return Part(mx.reshape(rows, n_q, 1), w.sum(-1, keepdim=True).reshape(rows, n_q, 1), out.reshape(rows, n_q, hd))


def merge(a: Optional[Part], b: Part) -> Part:
    """Both parts rescaled to the greater maximum and added."""
    if a is None:
        return b
    mx = torch.maximum(a.max, b.max)
    safe = torch.where(torch.isfinite(mx), mx, torch.zeros_like(mx))
    wa = torch.where(torch.isfinite(a.max), torch.exp(a.max - safe), torch.zeros_like(mx))
    wb = torch.where(torch.isfinite(b.max), torch.exp(b.max - safe), torch.zeros_like(mx))
    return Part(mx, a.sum * wa + b.sum * wb, a.out * wa + b.out * wb)


def finish(p: Part, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The attention a merged part stands for, [rows, n_q * hd] f32.  `sinks` [n_q]: one more score per head
    that takes probability mass and carries no value."""
    mx, sm, out = p.max, p.sum, p.out
    if sinks is not None:
        sk = sinks.float().view(1, -1, 1).to(mx.device)
        m2 = torch.maximum(mx, sk)
        wa = torch.where(torch.isfinite(mx), torch.exp(mx - m2), torch.zeros_like(mx))
        sm = sm * wa + torch.exp(sk - m2)
        out = out * wa
    res = out / sm.clamp_min(1e-38)
    res = torch.where(sm > 0, res, torch.zeros_like(res))
    return res.reshape(res.shape[0], -1)


def from_kernel(parts: torch.Tensor) -> Part:
    """f32 [rows, n_q, hd + 2] as `ops.attention.decode(parts_out=...)` writes it (maximum in log2 units)."""
    hd = parts.shape[-1] - 2
    return Part(parts[..., hd:hd + 1] * LN2, parts[..., hd + 1:hd + 2], parts[..., :hd])


def decode_part(q: torch.Tensor, cache, block_table: torch.Tensor, seq_lens: torch.Tensor, *, block_size: int,
                scale: Optional[float] = None, row_seq: Optional[torch.Tensor] = None, nsplit: int = 1,
                rows: Optional[int] = None, parts: Optional[torch.Tensor] = None) -> Part:
    """This rank's part of a decode step: q [rows, n_q, hd] bf16 over the keys its paged cache holds
    (`seq_lens` = how many of each row's positions live here, 0 included)."""
    from ..ops import attention

    R = rows if rows is not None else q.shape[0]
    if parts is None:
        parts = torch.empty(q.shape[0], q.shape[1], q.shape[2] + 2, dtype=torch.float32, device=q.device)
    attention.decode(q, cache, block_table, seq_lens, block_size=block_size, scale=scale, row_seq=row_seq, nsplit=nsplit,
                     rows=R, parts_out=parts)
    return from_kernel(parts[:R])


def gather_merge(part: Part, group=None, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All ranks' parts gathered and merged in rank order (so every rank computes the same bits); returns the
    attention [rows, n_q * hd] f32.  One all-gather of rows x heads x (hd + 2) floats."""
    import torch.distributed as dist

    packed = torch.cat([part.out, part.max, part.sum], -1).contiguous()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return finish(part, sinks)
    bufs = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(bufs, packed, group=group)
    hd = part.out.shape[-1]
    acc = None
    for b in bufs:
        acc = merge(acc, Part(b[..., hd:hd + 1], b[..., hd + 1:hd + 2], b[..., :hd]))
    return finish(acc, sinks)


def attention_over_ranges(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ranges: Sequence[Tuple[int, int]],
                          scale: float, q_pos: int, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Single-process form: the parts of every range of k / v [T, n_kv, hd] merged.  Equals the attention over
    the whole context; used by the tests and by a one-GPU run that only wants bounded score temporaries."""
    acc = None
    for lo, hi in ranges:
        acc = merge(acc, partial(q, k[lo:hi], v[lo:hi], scale, q_pos, lo))
    return finish(acc, sinks)
