"""Mixture experts computed on the host cores.

    moe_pairs(gate_up, down, x, pair_tok, pair_expert, pair_w, H=..., I=..., out=out)

`gate_up` / `down` are the stacked expert matrices of a layer in HOST memory, as bf16 tensors or as
`QuantWeight` planes (Q8_0 / Q6_K / Q4_K in the device layouts, so the pinned buffers an expert tier copies
from are the ones this reads).  For every pair p the expert `pair_expert[p]` is applied to row `pair_tok[p]` of
x and added, times `pair_w[p]`, to the same row of `out` (f32).  An expert that is not resident on the GPU at
decode size is cheaper to compute where its bytes are than to send over the bus: the reference does the same
for misses of its expert tier (`src/inference/moe_cuda_cpu/`, `generic_transformer/expert_tier.rs`).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np
import torch

from .engine import _lib

_FMT_OF_AQ = {1: 1, 2: 2, 3: 3, 4: 4}    # ops/quant.py: AQ_W8, AQ_W8G16 (Q6_K), AQ_W4 (Q4_K), AQ_MX4


def plane_format(w) -> Optional[int]:
    """The host kernel's format code of an expert stack, or None when it cannot read it."""
    if isinstance(w, torch.Tensor):
        return 0 if w.dtype == torch.bfloat16 and w.is_contiguous() and not w.is_cuda else None
    f = _FMT_OF_AQ.get(getattr(w, "aq_fmt", None))
    if f is None or w.codes.is_cuda or not w.codes.is_contiguous() or w.scales.stride(1) != 1:
        return None
    if f != 4 and not w.scales.is_contiguous():
        return None
    return f


def _p(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def moe_pairs(gate_up, down, x: torch.Tensor, pair_tok: Sequence[int], pair_expert: Sequence[int],
              pair_w: Sequence[float], *, H: int, I: int, out: torch.Tensor, gu_bias: Optional[torch.Tensor] = None,
              dn_bias: Optional[torch.Tensor] = None, glu=(0, 1.702, 7.0), threads: int = 8, max_level: int = -1):
    fg, fd = plane_format(gate_up), plane_format(down)
    if fg is None or fd is None:
        raise ValueError("the host expert kernel reads bf16 tensors and Q8_0 / Q6_K / Q4_K planes in host memory")
    assert x.dtype == torch.float32 and out.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    assert not x.is_cuda and not out.is_cuda and x.shape[1] == H == out.shape[1]
    n = len(pair_tok)
    tok = np.ascontiguousarray(pair_tok, dtype=np.int32)
    exp = np.ascontiguousarray(pair_expert, dtype=np.int32)
    wts = np.ascontiguousarray(pair_w, dtype=np.float32)
    gc, gs = (gate_up, None) if fg == 0 else (gate_up.codes, gate_up.scales)
    dc, ds = (down, None) if fd == 0 else (down.codes, down.scales)
    fp = lambda t: _p(t.float().contiguous()) if t is not None else None
    gb, db = (gu_bias.float().contiguous() if gu_bias is not None else None,
              dn_bias.float().contiguous() if dn_bias is not None else None)
    rc = _lib().lkcpu_moe_pairs(fg, _p(gc), _p(gs), fd, _p(dc), _p(ds), _p(gb), _p(db), H, I, _p(x),
                                tok.ctypes.data_as(C.c_void_p), exp.ctypes.data_as(C.c_void_p),
                                wts.ctypes.data_as(C.c_void_p), n, int(glu[0]), C.c_float(glu[1]), C.c_float(glu[2]),
                                _p(out), threads, max_level,
                                C.c_longlong(gs.stride(0) if fg == 4 else 0), C.c_longlong(ds.stride(0) if fd == 4 else 0))
    if rc != 0:
        raise ValueError(f"lkcpu_moe_pairs refused its arguments (rc {rc})")
    del fp
    return out
