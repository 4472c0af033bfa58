"""Block-scaled (microscaling) linear layers: MXFP4 weights run as stored on the tensor cores.

`tcgen05.mma.kind::mxf8f6f4.block_scale` multiplies E2M1 weights by e4m3 activations and applies
one E8M0 exponent per operand row per 32 values of K in hardware (csrc/cuda/gemm_mx.cu), so the
MXFP4 blocks of a GGUF or safetensors checkpoint are never expanded: the nibbles stream from HBM
at half a byte per value.  Activations are quantised to e4m3 with E8M0 exponents per 32 values by
`quant_mx8` (csrc/cuda/mx_quant.cu), fused with the MoE row gather or with the GLU.

The reference's MXFP4 path: `cuda/moe/mxfp4_moe.cuh:14-40` (int8 table + dp4a against q8 activations).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from ._lib import GemmArgs, Workspace, check, cuda_lib, ptr, stream
from .quant import AQ_MX4, QuantWeight


def sf_pitch(K: int) -> int:
    """Bytes per row of an exponent plane: four per 128 values of K, so every stage reads one word."""
    return (K + 127) // 128 * 4


assert sf_pitch(2880) == 92


@dataclass
class MxAct:
    """e4m3 rows [rows, K] + E8M0 exponents [rows, sf_pitch(K)] (bytes past K / 32 stay zero)."""
    data: torch.Tensor
    sf: torch.Tensor


@dataclass
class MxWeight:
    """MXFP4 weight [rows, K] (rows = E * N for stacked experts): nibbles [rows, K / 2] and E8M0
    exponents [rows, sf_pitch(K)], zero-padded."""
    codes: torch.Tensor
    sf: torch.Tensor
    rows: int
    K: int

    def nbytes(self) -> int:
        return self.codes.numel() + self.rows * (self.K // 32)


def alloc_mx_act(rows: int, K: int, device) -> MxAct:
    return MxAct(torch.empty(rows, K, dtype=torch.float8_e4m3fn, device=device),
                 torch.zeros(rows, sf_pitch(K), dtype=torch.uint8, device=device))


def mx_weight(q: QuantWeight) -> MxWeight:
    """The planes of an MXFP4 `QuantWeight` with the exponent rows padded to whole stages."""
    assert q.aq_fmt == AQ_MX4 and q.K % 32 == 0
    ld = sf_pitch(q.K)
    if q.scales.dim() == 2 and q.scales.shape[1] == ld and q.codes.is_contiguous():
        # the planes are shared, not copied: a slot cache that rewrites an expert's rows in place
        # (models/expert_tier.py) is seen by the GEMM without further ado
        return MxWeight(q.codes, q.scales, q.rows, q.K)
    sf = torch.zeros(q.rows, ld, dtype=torch.uint8, device=q.codes.device)
    sf[:, :q.K // 32] = q.scales.reshape(q.rows, -1)[:, :q.K // 32]
    return MxWeight(q.codes.contiguous(), sf, q.rows, q.K)


def quant_mx8(x: torch.Tensor, out: Optional[MxAct] = None, rows: Optional[int] = None, *, K: Optional[int] = None,
              pair_row: Optional[torch.Tensor] = None, kdiv: int = 1, glu_mode: Optional[int] = None,
              alpha: float = 1.702, limit: float = 7.0) -> MxAct:
    """bf16 rows -> MxAct.  `pair_row`: row p of the output plan takes x[p // kdiv] (MoE permute);
    `glu_mode` (0 SwiGLU, 1 clamped): x is [rows, 2K] (gate | up) and the activation is quantised."""
    R = rows if rows is not None else (pair_row.numel() if pair_row is not None else x.shape[0])
    if K is None:
        K = x.shape[1] // 2 if glu_mode is not None else x.shape[1]
    if out is None:
        out = alloc_mx_act(R if pair_row is None else R, K, x.device)
    mode = 1 if pair_row is not None else 2 if glu_mode is not None else 0
    check(cuda_lib().lk_quant_mx8(ptr(x), C.c_longlong(x.stride(0)), R, K, mode, ptr(pair_row), kdiv,
                                  int(glu_mode or 0), C.c_float(alpha), C.c_float(limit), ptr(out.data),
                                  C.c_longlong(out.data.stride(0)), ptr(out.sf), C.c_longlong(out.sf.stride(0)),
                                  stream()), "lk_quant_mx8")
    return out


def _args(x: MxAct, w: MxWeight, out: torch.Tensor, bias, rows: int) -> GemmArgs:
    a = GemmArgs()
    a.kind = 1
    a.B = ptr(x.data)
    a.Rb, a.K, a.ldb = rows, w.K, x.data.stride(0)
    a.b_scale, a.b_ld = ptr(x.sf), x.sf.stride(0)
    a.aq_fmt, a.aq, a.aq_scale = AQ_MX4, ptr(w.codes), ptr(w.sf)
    a.aq_ld, a.aq_sld = w.codes.stride(0), w.sf.stride(0)
    a.Ra = w.rows
    a.out, a.out_sa, a.out_sb = ptr(out), 1, out.stride(0)
    a.out_fp32 = int(out.dtype == torch.float32)
    a.bias, a.bias_on_a = ptr(bias), 1
    a.status = ptr(Workspace.get(out.device).status)
    return a


def linear_mx(x: MxAct, w: MxWeight, *, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
              rows: Optional[int] = None, bn: int = 0) -> torch.Tensor:
    """x [M, K] (MxAct) @ W.T -> bf16 [M, N]: weights on the MMA M side, tokens on N."""
    M = rows if rows is not None else x.data.shape[0]
    if out is None:
        out = torch.empty(M, w.rows, dtype=torch.bfloat16, device=x.data.device)
    a = _args(x, w, out, bias, M)
    a.bn = bn
    check(cuda_lib().lk_gemm_mx(C.byref(a), stream()), "lk_gemm_mx")
    return out


def grouped_linear_mx(xs: MxAct, w: MxWeight, rows_per_expert: int, plan, bias: Optional[torch.Tensor],
                      out: torch.Tensor) -> torch.Tensor:
    """out[r] = W[expert(r)] xs[r] (+ bias[expert(r)]) over the plan's tile list (sorted token rows)."""
    a = _args(xs, w, out, bias, xs.data.shape[0])
    a.bn = min(plan.bn, 128)
    a.g_rows_per_expert, a.g_max_tiles = rows_per_expert, plan.max_tiles
    a.g_tile_expert, a.g_tile_row0, a.g_tile_rows = ptr(plan.tile_expert), ptr(plan.tile_row0), ptr(plan.tile_rows)
    a.g_ntiles = ptr(plan.ntiles)
    check(cuda_lib().lk_gemm_mx(C.byref(a), stream()), "lk_gemm_mx (grouped)")
    return out


# ---- references (plain torch) ------------------------------------------------------------------

def quant_mx8_ref(x: torch.Tensor) -> MxAct:
    """Per 32 values: exponent = smallest power of two s with amax / s <= 448, values = e4m3(x / s)."""
    R, K = x.shape
    g = x.float().view(R, K // 32, 32)
    amax = g.abs().amax(2)
    t = amax / 448.0
    e = torch.where(amax > 0, torch.ceil(torch.log2(t.clamp_min(1e-45))), torch.zeros_like(t)).clamp(-127, 127)
    # log2 of an exact power of two may round either way: fix up with exact arithmetic
    e = torch.where((amax > 0) & (torch.exp2(e - 1) * 448.0 >= amax), e - 1, e)
    e = torch.where((amax > 0) & (torch.exp2(e) * 448.0 < amax), e + 1, e)
    q = (g / torch.exp2(e)[:, :, None]).view(R, K).to(torch.float8_e4m3fn)
    sf = torch.zeros(R, sf_pitch(K), dtype=torch.uint8, device=x.device)
    sf[:, :K // 32] = (e + 127).to(torch.uint8)
    return MxAct(q, sf)


def dequant_mx_act(a: MxAct, rows: Optional[int] = None) -> torch.Tensor:
    R = rows if rows is not None else a.data.shape[0]
    K = a.data.shape[1]
    s = torch.exp2(a.sf[:R, :K // 32].float() - 127.0)
    return (a.data[:R].float().view(R, K // 32, 32) * s[:, :, None]).view(R, K)
