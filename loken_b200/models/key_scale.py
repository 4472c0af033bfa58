"""The channel scale a quantised key store holds its keys under.

A layer that norms its queries and keys can fold one scale per key lane into the two norm weights:
the K norm weight is divided by the scale and the Q norm weight multiplied by it, so every score is
the same (a lane of the key is divided by what the same lane of the query is multiplied by).  The
scale is the magnitude of the K norm weight, equalised over the two lanes a rotation turns together,
so the rotation turns the scaled pair as it turns the plain one.  The scaled lanes of a key then
carry comparable magnitudes, and a 32-lane block of the int8 store shares its step among lanes of one
size: a lane with a large norm weight no longer sets the step of the lanes beside it.

Every store of a scaled layer holds scaled keys (paged cache, disk tier, hand-over), and the queries
are scaled wherever they are computed, because the weight carries the scale; nothing downstream
needs to know.  The reference describes the same fold in
`src/inference/generic_transformer/key_scale.rs:1-27`; its second form (a power of two folded into
the projections of layers without a K norm) is not built here.
"""
from __future__ import annotations

from typing import Optional

import torch


def rotation_partner(lane: int, rotated: int, adjacent: bool) -> Optional[int]:
    """The lane a rotation turns together with `lane`; None for a lane it leaves alone."""
    if lane >= rotated:
        return None
    if adjacent:
        return lane ^ 1
    half = rotated // 2
    return lane + half if lane < half else lane - half


def lane_scale(k_norm: torch.Tensor, rotated: int, adjacent: bool, floor: float = 1e-6) -> torch.Tensor:
    """One scale per key lane: |k_norm|, the larger of the two on a rotation pair."""
    s = k_norm.detach().float().abs().clamp_min(floor)
    hd = s.numel()
    idx = torch.tensor([p if (p := rotation_partner(i, rotated, adjacent)) is not None else i for i in range(hd)],
                       device=s.device)
    return torch.maximum(s, s[idx])


def apply_key_scale(weights, rotated: Optional[int] = None) -> int:
    """Folds the lane scale into every layer that has Q and K norm weights; returns how many."""
    cfg = weights.cfg
    hd = cfg.head_dim
    rot = (getattr(cfg, "rope_dim", None) or hd) if rotated is None else rotated
    adjacent = getattr(cfg, "rope_pairing", 1) == 0          # 0: (2i, 2i + 1) pairs; 1: (i, i + rot / 2)
    n = 0
    for lw in weights.layers:
        if lw is None or lw.q_norm is None or lw.k_norm is None or getattr(lw, "key_scaled", False):
            continue
        s = lane_scale(lw.k_norm, rot, adjacent)
        lw.k_norm = (lw.k_norm.float() / s).to(lw.k_norm.dtype)
        lw.q_norm = (lw.q_norm.float() * s).to(lw.q_norm.dtype)
        lw.key_scaled = True
        n += 1
    return n
