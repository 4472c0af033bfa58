"""Linear layers on the tcgen05 GEMM core (csrc/cuda/gemm_tc.cuh).

`linear(x, w)` computes x @ w.T for x [M, K] and w [N, K].  Small M (decode) runs in the swapped
form: the weight rows ride the MMA M dimension and the M tokens its N dimension, so a batch of
16..256 tokens costs no padding work and the kernel is a pure weight stream; large M (prefill)
runs tokens-on-M with 128x256 tiles.  Split-K keeps all 148 SMs streaming when N is small.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import GemmArgs, Workspace, check, cuda_lib, ptr, stream

NUM_SMS = 148
KIND_BF16, KIND_F8BLK = 0, 1
SCALE_NONE, SCALE_WBLOCK, SCALE_ACT_T = 0, 1, 2


@dataclass
class Fp8Weight:
    """e4m3 weight [N, K] with one f32 scale per 128x128 block, scale [ceil(N/128), ceil(K/128)]
    (the `weight` / `weight_scale_inv` pair of block-fp8 checkpoints)."""
    data: torch.Tensor
    scale: torch.Tensor
    _pow2: Optional[bool] = None
    tiled: Optional[torch.Tensor] = None     # the same values tile-major (`tile_major`), read by lk_gemm_mx

    @property
    def shape(self):
        return self.data.shape

    def tile_major(self) -> torch.Tensor:
        """[ceil(N/128), ceil(K/128), 128, 128]: every 128 x 128 tile is 16 KB in one piece, so the box a
        CTA fetches per stage is one contiguous read instead of 128 pieces of 128 bytes a row pitch apart."""
        if self.tiled is None:
            N, K = self.data.shape
            n128, k128 = (N + 127) // 128, (K + 127) // 128
            raw = self.data.view(torch.uint8)
            if N % 128 or K % 128:
                raw = torch.nn.functional.pad(raw, (0, k128 * 128 - K, 0, n128 * 128 - N))
            self.tiled = raw.view(n128, 128, k128, 128).permute(0, 2, 1, 3).contiguous()
        return self.tiled

    @property
    def pow2(self) -> bool:
        """Every block scale is a power of two (E8M0 checkpoints): the block-scaled MMA applies them."""
        if self._pow2 is None:
            m, _ = torch.frexp(self.scale.float())
            self._pow2 = bool(((m == 0.5) & (self.scale > 0)).all().item())
        return self._pow2


@dataclass
class Fp8Act:
    """e4m3 activations [M, K] with one f32 scale per token per 128 values, stored transposed
    as scale_t [K/128, ld] (ld >= M, a multiple of 4)."""
    data: torch.Tensor
    scale_t: torch.Tensor


def _pick_bn(rows: int) -> int:
    bn = 16
    while bn < rows and bn < 256:
        bn *= 2
    return bn


SPLIT_OVERRIDE = 0      # measurement hook: K splits of GEMMs with fewer tiles than SMs (0 = _pick_splits)


def _pick_splits(tiles: int, nkb: int) -> int:
    if SPLIT_OVERRIDE:
        return max(1, min(SPLIT_OVERRIDE, nkb))
    # up to eight K blocks the split's hand-over (workspace, counter, owner sum: ~5 us) costs more than
    # the K loop it saves (measured 9.0 vs 10.8 us on 8192 x 1024)
    if tiles >= NUM_SMS or nkb <= 8:
        return 1
    s = max(1, NUM_SMS // tiles)
    return int(min(s, max(1, nkb // 2), 16))


def gemm_raw(kind, A, B, out, out_sa, out_sb, *, bias=None, bias_on_a=False, residual=None, a_scale=None, a_mode=0,
             a_ld=0, b_scale=None, b_mode=0, b_ld=0, bn=0, splits=0, out_fp32=False, symm=None):
    lib = cuda_lib()
    Ra, K = A.shape
    Rb = B.shape[0]
    assert B.shape[1] == K and A.stride(1) == 1 and B.stride(1) == 1
    wsp = Workspace.get(A.device)
    if bn <= 0:
        bn = _pick_bn(Rb)
    kb = 64 if kind == KIND_BF16 else 128
    tiles = ((Ra + 127) // 128) * ((Rb + bn - 1) // bn)
    if splits <= 0:
        # fewer tiles than SMs: split K so the grid covers the chip; otherwise 0 = the launcher runs
        # whole tiles for the full rounds and splits only the remainder
        splits = _pick_splits(tiles, (K + kb - 1) // kb) if tiles < NUM_SMS else 0
    a = GemmArgs()
    a.kind = kind
    a.A, a.B = ptr(A), ptr(B)
    a.Ra, a.Rb, a.K = Ra, Rb, K
    a.lda, a.ldb = A.stride(0), B.stride(0)
    a.out, a.out_sa, a.out_sb, a.out_fp32 = ptr(out), out_sa, out_sb, int(out_fp32)
    a.bias, a.bias_on_a = ptr(bias), int(bias_on_a)
    a.residual = ptr(residual)
    a.a_scale, a.a_mode, a.a_ld = ptr(a_scale), a_mode, a_ld
    a.b_scale, a.b_mode, a.b_ld = ptr(b_scale), b_mode, b_ld
    a.bn, a.splits = bn, splits
    a.ws, a.ws_floats = ptr(wsp.ws), wsp.ws.numel()
    a.counters, a.n_counters = ptr(wsp.counters), wsp.counters.numel()
    a.status = ptr(wsp.status)
    fused = False
    if symm is not None and symm.world > 1 and not out_fp32:
        # fused GEMM -> all-reduce: every tile's owner CTA waits on its peers, so the whole grid has
        # to be resident at once, the output has to fit a receive slot and each tile needs a flag
        nkb = (K + kb - 1) // kb
        s_eff = max(1, min(splits, nkb))
        rows_out, ld_out = (Ra, out_sa) if out_sb == 1 else (Rb, out_sb)
        if tiles * s_eff <= NUM_SMS and tiles <= symm.max_chunks and rows_out * ld_out * 2 <= symm.slot_bytes:
            a.symm_view = C.cast(C.pointer(symm.view), C.c_void_p)
            fused = True
    check(lib.lk_gemm_tc(C.byref(a), stream()), "lk_gemm_tc")
    gemm_raw.last_fused = fused
    return out


SWAP_MAX_M = 256
FP8_MX = True           # block-fp8 weights with power-of-two scales run on the block-scaled MMA (lk_gemm_mx)
# ... up to this many tokens (tokens on the MMA N side).  Measured on 57344 x 8192 with three weight tiles
# per token tile: 16 tokens 76 us against 90 us for the fold kernel, 64 tokens 97 against 105, 128 tokens 122
# against 114.  The MMA loop itself ends after 64 - 70 us at every batch (6.7 - 7.3 TB/s of weights); what
# follows is the epilogue (four warps move 128 x BN values through shared memory: memory instructions of one
# warp per scheduler issue about twenty cycles apart) and the K-split remainder, both exposed when a CTA has
# a single unit.  Matrices without whole rounds of three-tile units (fewer than 3 x 148 weight tiles) keep
# the fold kernel above FP8_MX_MAX_M tokens.
FP8_MX_MAX_M = 32
FP8_MX_WIDE_MAX_M = 64  # ... and this many tokens when the matrix has at least 3 x 148 tiles of 128 rows
FP8_MX_BN = 0           # measurement hook: N tile of that path (0 = the launcher's choice)
FP8_MX_TILED = False    # measurement hook: read the weights tile-major (Fp8Weight.tile_major)
FP8_MX_PROF = None      # measurement hook: int64 tensor [296, 8] that receives the kernel's per-CTA counters (loken_cuda.h)
FP8_MX_PLAN = (0, 0, 0) # measurement hook: (weight tiles per unit, tiles per remainder unit, K splits); 0 = cost model
# fp8 carries one activation scale per token in the swapped form: measured faster only for a handful of tokens
FP8_BN_OVERRIDE = 0     # measurement hook: N-tile width of the tokens-on-M form (0 = the rule in linear_fp8)
FP8_SWAP_MAX_M = 16     # measured: up to 16 tokens the weights-on-M form is faster (93 vs 107 us on 57344 x 8192)


def linear_bf16(x: torch.Tensor, w: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                out_fp32: bool = False, splits: int = 0, symm=None) -> torch.Tensor:
    """x [M, K] bf16, w [N, K] bf16 -> [M, N]; bias f32 [N]; residual bf16 [M, N]."""
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=x.device)
    ldo = out.stride(0)
    if M <= SWAP_MAX_M:
        gemm_raw(KIND_BF16, w, x, out, 1, ldo, bias=bias, bias_on_a=True, residual=residual, splits=splits,
                 out_fp32=out_fp32, symm=symm)
    else:
        gemm_raw(KIND_BF16, x, w, out, ldo, 1, bias=bias, bias_on_a=False, residual=residual, bn=256,
                 splits=splits, out_fp32=out_fp32, symm=symm)
    return out


def linear_fp8(x: Fp8Act, w: Fp8Weight, *, bias: Optional[torch.Tensor] = None,
               residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               out_fp32: bool = False, splits: int = 0, rows: Optional[int] = None, symm=None) -> torch.Tensor:
    """Block-scaled fp8 linear: x e4m3 [M, K] (+ per-token-group scales), w e4m3 [N, K]
    (+ 128x128 block scales) -> bf16 [M, N]."""
    xd = x.data if rows is None else x.data[:rows]
    M, K = xd.shape
    N = w.data.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=xd.device)
    ldo = out.stride(0)
    sld = x.scale_t.stride(0)
    mx_max_m = FP8_MX_WIDE_MAX_M if N >= 3 * NUM_SMS * 128 else FP8_MX_MAX_M
    if FP8_MX and M <= max(FP8_MX_MAX_M, mx_max_m) and symm is None and not out_fp32 and residual is None and w.pow2:
        # power-of-two block scales: one accumulation over all of K on the block-scaled MMA (gemm_mx.cu)
        wsp = Workspace.get(xd.device)
        a = GemmArgs()
        a.kind = KIND_F8BLK
        a.A, a.B = ptr(w.data), ptr(xd)
        a.Ra, a.Rb, a.K = N, M, K
        a.lda, a.ldb = w.data.stride(0), xd.stride(0)
        if FP8_MX_TILED or w.tiled is not None:
            a.A, a.a_tiled, a.lda = ptr(w.tile_major()), 1, 128
        a.out, a.out_sa, a.out_sb = ptr(out), 1, ldo
        a.bias, a.bias_on_a = ptr(bias), 1
        a.a_scale, a.a_mode, a.a_ld = ptr(w.scale), SCALE_WBLOCK, w.scale.stride(0)
        a.b_scale, a.b_mode, a.b_ld = ptr(x.scale_t), SCALE_ACT_T, sld
        a.bn, a.splits = FP8_MX_BN, FP8_MX_PLAN[2] or splits
        a.mt, a.rem_mt = FP8_MX_PLAN[0], FP8_MX_PLAN[1]
        a.prof = ptr(FP8_MX_PROF)
        a.ws, a.ws_floats = ptr(wsp.ws), wsp.ws.numel()
        a.counters, a.n_counters = ptr(wsp.counters), wsp.counters.numel()
        a.status = ptr(wsp.status)
        check(cuda_lib().lk_gemm_mx(C.byref(a), stream()), "lk_gemm_mx (fp8)")
        gemm_raw.last_fused = False
        return out
    if M <= FP8_SWAP_MAX_M:
        gemm_raw(KIND_F8BLK, w.data, xd, out, 1, ldo, bias=bias, bias_on_a=True, residual=residual,
                 a_scale=w.scale, a_mode=SCALE_WBLOCK, a_ld=w.scale.stride(0), b_scale=x.scale_t,
                 b_mode=SCALE_ACT_T, b_ld=sld, splits=splits, out_fp32=out_fp32, symm=symm)
    else:
        gemm_raw(KIND_F8BLK, xd, w.data, out, ldo, 1, bias=bias, bias_on_a=False, residual=residual,
                 a_scale=x.scale_t, a_mode=SCALE_ACT_T, a_ld=sld, b_scale=w.scale, b_mode=SCALE_WBLOCK,
                 b_ld=w.scale.stride(0), bn=FP8_BN_OVERRIDE or (128 if M <= 512 else 256), splits=splits,
                 out_fp32=out_fp32, symm=symm)
    return out


# ---- quantisers used at load time and by the tests (plain torch, not a hot path) -------------

def pow2_ceil(t: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= t (t > 0), exactly (no log2 rounding)."""
    m, e = torch.frexp(t)            # t = m * 2^e, m in [0.5, 1)
    return torch.ldexp(torch.ones_like(t), torch.where(m == 0.5, e - 1, e))


WEIGHT_SCALE_UE8M0 = True    # random-init block-fp8 weights get power-of-two (E8M0) block scales


def quantize_weight_fp8(w: torch.Tensor, ue8m0: Optional[bool] = None) -> Fp8Weight:
    """[N, K] float -> e4m3 with one f32 scale per 128x128 block.  `ue8m0` (the default): the scale is
    the smallest power of two with amax / scale <= 448, the E8M0 `.scale` variant of block-fp8
    checkpoints, which the block-scaled MMA applies in hardware; otherwise amax / 448 (`weight_scale_inv`)."""
    ue8m0 = WEIGHT_SCALE_UE8M0 if ue8m0 is None else ue8m0
    N, K = w.shape
    nb, kb = (N + 127) // 128, (K + 127) // 128
    wp = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, 128, kb, 128)
    amax = blocks.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    if ue8m0:
        scale = pow2_ceil(scale)
    q = (blocks / scale[:, None, :, None]).clamp(-448, 448).view(nb * 128, kb * 128)[:N, :K]
    return Fp8Weight(q.to(torch.float8_e4m3fn).contiguous(), scale.contiguous())


def dequantize_weight_fp8(w: Fp8Weight) -> torch.Tensor:
    N, K = w.data.shape
    s = w.scale.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    return w.data.float() * s


def quantize_act_fp8_ref(x: torch.Tensor, ld: Optional[int] = None) -> Fp8Act:
    """Reference of the activation quantiser: per token per 128 values, scale = the smallest power of
    two with amax / scale <= 448."""
    M, K = x.shape
    assert K % 128 == 0
    g = x.float().view(M, K // 128, 128)
    amax = g.abs().amax(dim=2)
    scale = torch.where(amax > 0, pow2_ceil((amax / 448.0).clamp_min(2.0 ** -126)), torch.ones_like(amax))
    q = (g / scale[:, :, None]).view(M, K).to(torch.float8_e4m3fn)
    ld = ld or ((M + 3) // 4 * 4)
    st = torch.zeros(K // 128, ld, dtype=torch.float32, device=x.device)
    st[:, :M] = scale.t()
    return Fp8Act(q.contiguous(), st)


def dequantize_act_fp8(x: Fp8Act, rows: Optional[int] = None) -> torch.Tensor:
    M, K = x.data.shape
    rows = rows or M
    s = x.scale_t[:, :rows].t().repeat_interleave(128, 1)
    return x.data[:rows].float() * s
