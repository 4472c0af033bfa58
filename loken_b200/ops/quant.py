"""GGUF-quantised weights on the device and the dequant-fused GEMM that runs them.

A GGUF tensor (Q8_0, Q4_K, Q6_K, MXFP4) is repacked once at load time from its file blocks into
two planes that are aligned for 16-byte loads (csrc/cuda/dequant.cuh); codes and scales keep
their file values, so the numbers the kernel multiplies by are exactly the format's own
(`dequantize_weight` here reproduces them in PyTorch for the tests).  `linear_gguf` then runs
x @ W.T on the tcgen05 core with the weight rows on the MMA M side: four warps expand each
128 x 64 weight tile to bf16 straight into swizzled shared memory while TMA brings the tokens.

Counterparts in the reference: the MMVQ mat-vec family (`src/inference/cuda/mmvq_gguf.cu`) for
decode and the MMQ tiles (`cuda/mmq_gguf/mmq_gguf.cuh`) for prefill, with the host-side dispatch
of `src/tensor/quantized/kernel_matmul.rs`.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from ..formats import gguf
from ._lib import GemmArgs, GemvPre, Workspace, check, cuda_lib, ptr, stream
from .gemm import KIND_BF16, NUM_SMS

AQ_W8, AQ_W8G16, AQ_W4, AQ_MX4 = 1, 2, 3, 4
AQ_W4G128 = 5         # AWQ: nibbles, per 128 values one f16 scale and one f16 minimum (zero point x scale)
GEMV_FORMATS = (AQ_W8, AQ_W8G16, AQ_W4, AQ_W4G128)
MX_NATIVE = True      # MXFP4 on the block-scaled MMA (False: expanded to bf16 by the dequant warps)
FMT_OF_TYPE = {gguf.Q8_0: AQ_W8, gguf.Q6_K: AQ_W8G16, gguf.Q4_K: AQ_W4, gguf.MXFP4: AQ_MX4}
TYPE_OF_NAME = {"q8_0": gguf.Q8_0, "q4_k": gguf.Q4_K, "q6_k": gguf.Q6_K, "mxfp4": gguf.MXFP4}


@dataclass
class QuantWeight:
    """[rows, K] weight (rows = E * N for stacked experts) in a device block format."""
    aq_fmt: int
    ggml_type: int
    rows: int
    K: int
    codes: torch.Tensor      # uint8 [rows, code bytes per row]
    scales: torch.Tensor     # uint8 [rows, scale bytes per row]

    @property
    def shape(self):
        return (self.rows, self.K)

    @property
    def device(self):
        return self.codes.device

    def rows_float(self, ids: torch.Tensor) -> torch.Tensor:
        """fp32 [n, K]: the decoded rows `ids` (an embedding lookup in a quantised table, on any device)."""
        ids = ids.long().to(self.codes.device)
        sub = QuantWeight(self.aq_fmt, self.ggml_type, int(ids.numel()), self.K, self.codes[ids], self.scales[ids])
        return dequantize_weight(sub)

    def nbytes(self) -> int:
        if self.aq_fmt == AQ_MX4:
            return self.codes.numel() + self.rows * (self.K // 32)       # without the pitch padding
        return self.codes.numel() + self.scales.numel()


def mx_sf_pitch(K: int) -> int:
    """Bytes per row of an MXFP4 exponent plane: four per 128 values of K."""
    return (K + 127) // 128 * 4


def _pack_nibbles(v: np.ndarray) -> np.ndarray:
    """[..., K] values 0..15 -> [..., K/2] bytes, value k in byte k/2, low nibble for even k."""
    return (v[..., 0::2] | (v[..., 1::2] << 4)).astype(np.uint8)


def repack_blocks(raw: np.ndarray, ggml_type: int, rows: int, K: int):
    """GGUF file blocks of a [rows, K] tensor -> (codes, scales) uint8 planes, numpy."""
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    if ggml_type == gguf.Q8_0:
        b = raw.reshape(rows, K // 32, 34)
        return b[:, :, 2:].reshape(rows, K).copy(), b[:, :, :2].reshape(rows, K // 32 * 2).copy()
    if ggml_type == gguf.MXFP4:
        b = raw.reshape(rows, K // 32, 17)
        qs = b[:, :, 1:]
        v = np.concatenate([qs & 0xF, qs >> 4], axis=2)          # [rows, K/32, 32] in value order
        # exponent rows are padded with zeros to four per 128 values of K: the block-scaled GEMM reads one
        # 32-bit word of exponents per row and stage
        ex = np.zeros((rows, mx_sf_pitch(K)), dtype=np.uint8)
        ex[:, :K // 32] = b[:, :, 0]
        return _pack_nibbles(v).reshape(rows, K // 2), ex
    if ggml_type == gguf.Q4_K:
        b = raw.reshape(rows, K // 256, 144)
        sc12 = b[:, :, 4:16].astype(np.uint8)
        qs = b[:, :, 16:].reshape(rows, K // 256, 4, 32)
        v = np.concatenate([qs & 0xF, qs >> 4], axis=3)          # [.., 4, 64]: low nibbles then high
        codes = _pack_nibbles(v.reshape(rows, K // 256, 256)).reshape(rows, K // 2)
        sc = np.empty(b.shape[:2] + (8,), dtype=np.uint8)
        mn = np.empty_like(sc)
        sc[:, :, :4] = sc12[:, :, 0:4] & 63
        mn[:, :, :4] = sc12[:, :, 4:8] & 63
        sc[:, :, 4:] = (sc12[:, :, 8:12] & 0xF) | ((sc12[:, :, 0:4] >> 6) << 4)
        mn[:, :, 4:] = (sc12[:, :, 8:12] >> 4) | ((sc12[:, :, 4:8] >> 6) << 4)
        rec = np.concatenate([b[:, :, 0:4], sc, mn], axis=2)      # d, dmin, sc[8], m[8] = 20 bytes
        return codes, rec.reshape(rows, K // 256 * 20).copy()
    if ggml_type == gguf.Q6_K:
        b = raw.reshape(rows, K // 256, 210)
        ql = b[:, :, :128].reshape(rows, K // 256, 2, 64).astype(np.int16)
        qh = b[:, :, 128:192].reshape(rows, K // 256, 2, 32).astype(np.int16)
        q = np.empty((rows, K // 256, 2, 128), dtype=np.int16)
        q[..., 0:32] = (ql[..., 0:32] & 0xF) | (((qh >> 0) & 3) << 4)
        q[..., 32:64] = (ql[..., 32:64] & 0xF) | (((qh >> 2) & 3) << 4)
        q[..., 64:96] = (ql[..., 0:32] >> 4) | (((qh >> 4) & 3) << 4)
        q[..., 96:128] = (ql[..., 32:64] >> 4) | (((qh >> 6) & 3) << 4)
        codes = (q - 32).astype(np.int8).reshape(rows, K).view(np.uint8)
        rec = np.concatenate([b[:, :, 208:210], b[:, :, 192:208]], axis=2)   # d, sc[16] = 18 bytes
        return codes.copy(), rec.reshape(rows, K // 256 * 18).copy()
    raise ValueError(f"no device layout for ggml type {ggml_type}")


def from_blocks(raw: np.ndarray, ggml_type: int, rows: int, K: int, device) -> QuantWeight:
    codes, scales = repack_blocks(raw, ggml_type, rows, K)
    return QuantWeight(FMT_OF_TYPE[ggml_type], ggml_type, rows, K,
                       torch.from_numpy(codes).to(device), torch.from_numpy(scales).to(device))


def quantize_weight(w: torch.Tensor, fmt: str) -> QuantWeight:
    """float [rows, K] -> device block format `fmt` (q8_0 | q4_k | q6_k | mxfp4), through the
    host encoders so the result is what a GGUF file of that type would hold."""
    ty = TYPE_OF_NAME[fmt]
    rows, K = w.shape
    bv, _ = gguf.block_info(ty)
    assert K % max(bv, 64) == 0, f"K={K} must be a multiple of {max(bv, 64)} for {fmt}"
    raw = gguf.quantize(w.detach().float().cpu().numpy(), ty)
    return from_blocks(raw, ty, rows, K, w.device)


def scale_weight_(q: QuantWeight, mul: float) -> QuantWeight:
    """W *= mul in place, by multiplying the half-precision scale fields of every block (the codes stay): what
    folds a per-layer multiplier of a file's metadata into a stored matrix."""
    rows, K = q.rows, q.K
    s = q.scales
    if q.aq_fmt == AQ_W8:
        h = s.view(torch.float16)
        h.copy_((h.float() * mul).half())
    elif q.aq_fmt in (AQ_W8G16, AQ_W4):
        rec_bytes, n_half = (18, 1) if q.aq_fmt == AQ_W8G16 else (20, 2)
        rec = s.view(rows, K // 256, rec_bytes)
        h = rec[:, :, :2 * n_half].contiguous().view(torch.float16)
        rec[:, :, :2 * n_half] = (h.float() * mul).half().view(torch.uint8).view(rows, K // 256, 2 * n_half)
    else:
        raise ValueError("a power-of-two exponent format cannot take an arbitrary multiplier")
    return q


def from_awq(qvals: torch.Tensor, zeros: torch.Tensor, scales: torch.Tensor, device) -> QuantWeight:
    """AWQ's 4-bit weights as device planes: qvals int [out, in] (0..15), zeros int [out, in / 128], scales
    [out, in / 128]; w = (q - zero) * scale.  Codes keep their values (two per byte, the even one in the low
    nibble); a group's record is (scale, zero x scale) in f16, so w = scale * q - minimum as in the K formats."""
    rows, K = qvals.shape
    assert K % 128 == 0 and tuple(zeros.shape) == (rows, K // 128) == tuple(scales.shape)
    codes = _nibble_pack_t(qvals.to(torch.uint8))
    s16 = scales.half()
    rec = torch.stack([s16, (zeros.float() * s16.float()).half()], -1).contiguous()        # [rows, K/128, 2] f16
    return QuantWeight(AQ_W4G128, -1, rows, K, codes.contiguous().to(device),
                       rec.view(torch.uint8).view(rows, K // 128 * 4).contiguous().to(device))


def dequantize_weight(q: QuantWeight) -> torch.Tensor:
    """fp32 [rows, K]: what the kernel multiplies by before its bf16 rounding."""
    rows, K = q.rows, q.K
    c, s = q.codes, q.scales
    if q.aq_fmt == AQ_W4G128:
        v = torch.stack([c & 0xF, c >> 4], dim=2).view(rows, K // 128, 128).float()
        rec = s.view(rows, K // 128, 4).contiguous().view(torch.float16).float()            # [rows, K/128, 2]
        return (v * rec[:, :, 0:1] - rec[:, :, 1:2]).view(rows, K)
    if q.aq_fmt == AQ_W8:
        d = s.view(torch.float16).float()
        return (c.view(torch.int8).float().view(rows, K // 32, 32) * d[:, :, None]).view(rows, K)
    if q.aq_fmt == AQ_W8G16:
        rec = s.view(rows, K // 256, 18)
        d = rec[:, :, :2].contiguous().view(torch.float16).float()            # [rows, K/256, 1]
        sc = rec[:, :, 2:].contiguous().view(torch.int8).float()               # [rows, K/256, 16]
        qv = c.view(torch.int8).float().view(rows, K // 256, 16, 16)
        return ((d * sc)[:, :, :, None] * qv).view(rows, K)
    lo, hi = (c & 0xF), (c >> 4)
    v = torch.stack([lo, hi], dim=2).view(rows, K)
    if q.aq_fmt == AQ_W4:
        rec = s.view(rows, K // 256, 20)
        dd = rec[:, :, :4].contiguous().view(torch.float16).float()           # [rows, K/256, 2]
        sc, mn = rec[:, :, 4:12].float(), rec[:, :, 12:20].float()
        d1 = (dd[:, :, 0:1] * sc)[:, :, :, None]
        m1 = (dd[:, :, 1:2] * mn)[:, :, :, None]
        return (d1 * v.float().view(rows, K // 256, 8, 32) - m1).view(rows, K)
    if q.aq_fmt == AQ_MX4:
        lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6], device=c.device)
        e = s[:, :K // 32].to(torch.int32)
        sc = torch.where(e == 0, torch.full_like(e, 0, dtype=torch.float32) + 2.0 ** -127,
                         torch.exp2((e - 127).float()))
        return (lut[v.long()].view(rows, K // 32, 32) * sc[:, :, None]).view(rows, K)
    raise ValueError(q.aq_fmt)


def _pick_bn(rows: int) -> int:
    return 16 if rows <= 16 else 64 if rows <= 64 else 128


GEMV_MAX_M = 8          # up to this many token rows the dp4a GEMV runs (gemv_q.cu); 0 turns it off
# From this many token rows on, a GGUF matrix is decoded to bf16 once (in row chunks that stay in L2) and
# multiplied by the plain bf16 GEMM: the dequantising warps of the fused kernel decode every weight tile
# again for every 128 tokens and top out near 1e12 values/s, a fifth of what the tensor cores could take
# (Llama-8B gate/up, 1024 tokens: 1.03 ms fused).  0 turns it off.
DEQUANT_ONCE_MIN_M = 129
DEQUANT_CHUNK_BYTES = 48 << 20
_scratch = {}


def dequant_rows(w: QuantWeight, n0: int, n1: int, out: torch.Tensor) -> torch.Tensor:
    """Rows [n0, n1) of `w` (Q8_0 / Q6_K / Q4_K planes) decoded to bf16 into out [n1 - n0, K]."""
    check(cuda_lib().lk_dequant_q(w.aq_fmt, ptr(w.codes[n0:]), C.c_longlong(w.codes.stride(0)), ptr(w.scales[n0:]),
                                  C.c_longlong(w.scales.stride(0)), ptr(out), C.c_longlong(out.stride(0)), n1 - n0, w.K,
                                  stream()), "lk_dequant_q")
    return out


def _linear_dequant_once(x, w: QuantWeight, bias, out, out_fp32):
    from .gemm import linear_bf16

    N, K = w.rows, w.K
    per = max(128, DEQUANT_CHUNK_BYTES // (2 * K) // 128 * 128)
    key = (x.device, per * K)
    buf = _scratch.get(key)
    if buf is None:
        buf = _scratch[key] = torch.empty(per * K, dtype=torch.bfloat16, device=x.device)
    for n0 in range(0, N, per):
        n1 = min(N, n0 + per)
        wt = dequant_rows(w, n0, n1, buf[:(n1 - n0) * K].view(n1 - n0, K))
        linear_bf16(x, wt, bias=None if bias is None else bias[n0:n1], out=out[:, n0:n1], out_fp32=out_fp32)
    return out


def embed_gguf(tokens: torch.Tensor, table: QuantWeight, out: Optional[torch.Tensor] = None, scale: float = 1.0):
    """Rows `tokens` of a quantised embedding table (Q8_0 / Q6_K / Q4_K planes), decoded to bf16 [T, H]."""
    T = tokens.numel()
    if out is None:
        out = torch.empty(T, table.K, dtype=torch.bfloat16, device=table.codes.device)
    check(cuda_lib().lk_embed_q(table.aq_fmt, ptr(tokens), ptr(table.codes), C.c_longlong(table.codes.stride(0)),
                                ptr(table.scales), C.c_longlong(table.scales.stride(0)), ptr(out), T, table.K, table.rows,
                                C.c_float(scale), stream()), "lk_embed_q")
    return out


def gemv_takes(M: int, w, x_stride: int = 0) -> bool:
    """Does a product of M token rows with `w` run as the dp4a GEMV (the form that can take a `GemvFront`)?"""
    return (isinstance(w, QuantWeight) and 0 < M <= GEMV_MAX_M and w.aq_fmt in GEMV_FORMATS
            and x_stride % 8 == 0 and (1 if M == 1 else 2 if M == 2 else 4 if M <= 4 else 8) * w.K * 1.25 <= 200 * 1024)


@dataclass
class GemvFront:
    """What runs in front of a GEMV inside its kernel instead of as kernels of its own.

    norm / eps / delta : the activations are RMSNorm(x + delta) * norm (delta: an update of the residual
                         stream that is still pending, or None); x itself is NOT written
    glu                : (mode, alpha, limit): x is [gate | up], 2K wide, and the activations are the gated unit
    update             : (rows, delta): rows += delta, applied on the side by one CTA: the pending update of
                         an earlier GEMV of the step, whose readers are all done by now.  `rows` must not
                         be this GEMV's own input."""
    norm: Optional[torch.Tensor] = None
    eps: float = 1e-6
    delta: Optional[torch.Tensor] = None
    glu: Optional[tuple] = None
    update: Optional[tuple] = None
    prof: Optional[torch.Tensor] = None        # measurement hook: int64 [CTAs, 8] time stamps (streaming form)

    def pack(self, M: int) -> GemvPre:
        a = GemvPre()
        a.prof = ptr(self.prof)
        if self.norm is not None:
            assert self.norm.dtype == torch.float32
            a.mode, a.gamma, a.eps = 1, ptr(self.norm), float(self.eps)
            if self.delta is not None:
                assert self.delta.dtype == torch.bfloat16 and self.delta.stride(1) == 1
                a.delta, a.ldd = ptr(self.delta), self.delta.stride(0)
        elif self.glu is not None:
            a.mode, a.glu_mode, a.glu_alpha, a.glu_limit = 2, int(self.glu[0]), float(self.glu[1]), float(self.glu[2])
        if self.update is not None:
            ux, ud = self.update
            assert ux.dtype == ud.dtype == torch.bfloat16 and ux.shape[1] == ud.shape[1] and ux.shape[0] >= M
            a.upd_x, a.upd_delta, a.upd_ldx, a.upd_ldd, a.upd_cols = ptr(ux), ptr(ud), ux.stride(0), ud.stride(0), ux.shape[1]
        return a


def gemv_slots_takes(w, n_experts: int) -> bool:
    """Can `gemv_slots` run over this stack of `n_experts` matrices ([n_experts * N, K] planes)?"""
    if not isinstance(w, QuantWeight) or w.aq_fmt not in (AQ_W8, AQ_W8G16, AQ_W4) or w.rows % n_experts:
        return False
    if not w.codes.is_cuda or not w.codes.is_contiguous() or not w.scales.is_contiguous():
        return False
    rc = cuda_lib().lk_gemv_q_slots(w.aq_fmt, None, None, None, C.c_longlong(0), 1, 1, None, 0, n_experts,
                                    w.rows // n_experts, w.K, None, None, C.c_longlong(0), None, None, 1, None)
    return rc == 0


def gemv_slots(x: torch.Tensor, w: QuantWeight, slot_expert: torch.Tensor, slots: int, x_div: int, n_experts: int, *,
               e_lo: int = 0, bias: Optional[torch.Tensor] = None, out: torch.Tensor, glu: Optional[tuple] = None):
    """Decode-size mixture products on the streaming GEMV: slot s takes row s // x_div of x (bf16; with `glu` the row
    is [gate | up], 2K wide) times the matrix of expert slot_expert[s] of the stack `w` ([n_experts * N, K] planes,
    see `gemv_slots_takes`) into row s of out [slots, N].  slot_expert is an int32 device tensor: the routing kernel
    can be the launch right before this one, nothing is planned or permuted on the way."""
    N = w.rows // n_experts
    assert slot_expert.dtype == torch.int32 and slot_expert.numel() >= slots and out.shape[1] == N and out.stride(1) == 1
    assert x.stride(1) == 1 and x.shape[1] == (2 * w.K if glu is not None else w.K)
    pre = GemvFront(glu=glu).pack(1) if glu is not None else None
    check(cuda_lib().lk_gemv_q_slots(w.aq_fmt, ptr(w.codes), ptr(w.scales), ptr(x), C.c_longlong(x.stride(0)), slots, x_div,
                                     ptr(slot_expert), e_lo, n_experts, N, w.K, ptr(bias), ptr(out),
                                     C.c_longlong(out.stride(0)), C.byref(pre) if pre is not None else None,
                                     ptr(Workspace.get(x.device).status), 0, stream()), "lk_gemv_q_slots")
    return out


def linear_gguf(x: torch.Tensor, w: QuantWeight, *, bias: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, splits: int = 0, out_fp32: bool = False,
                front: Optional[GemvFront] = None) -> torch.Tensor:
    """x bf16 [M, K] @ W.T -> bf16 (or f32) [M, N].  Up to eight token rows run as a GEMV on int8 activations;
    beyond that tokens ride the MMA N dimension in tiles of 16 / 64 / 128 with dequantising warps.  `front`
    (GEMV only, see `gemv_takes`) fuses a norm or gated unit in front and a residual update on the side."""
    M = x.shape[0]
    K = w.K
    N = w.rows
    assert x.stride(1) == 1 and x.shape[1] == (2 * K if front is not None and front.glu is not None else K)
    if front is not None and not gemv_takes(M, w, x.stride(0)):
        raise ValueError("a fused front needs the GEMV path (see gemv_takes)")
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=x.device)
    if w.aq_fmt == AQ_MX4 and MX_NATIVE and K % 32 == 0:
        # MXFP4 runs as stored on the block-scaled tensor-core path: activations to e4m3 + E8M0 exponents
        # per 32 values, weights' nibbles and exponents straight into the MMA (ops/mx.py)
        from . import mx

        if getattr(w, "_mx", None) is None:
            w._mx = mx.mx_weight(w)
        xa = mx.quant_mx8(x, rows=M)
        return mx.linear_mx(xa, w._mx, bias=bias, out=out, rows=M)
    if gemv_takes(M, w, x.stride(0)):
        # a handful of token rows: int8 activations and dp4a over the stored codes, every weight byte read once
        check(cuda_lib().lk_gemv_q(w.aq_fmt, ptr(w.codes), C.c_longlong(w.codes.stride(0)), ptr(w.scales),
                                   C.c_longlong(w.scales.stride(0)), ptr(x), C.c_longlong(x.stride(0)), M, N, K,
                                   ptr(bias), ptr(out), C.c_longlong(out.stride(0)), int(out_fp32),
                                   C.byref(front.pack(M)) if front is not None else None,
                                   ptr(Workspace.get(x.device).status), stream()), "lk_gemv_q")
        return out
    if w.aq_fmt == AQ_W4G128 or (DEQUANT_ONCE_MIN_M and M >= DEQUANT_ONCE_MIN_M and w.aq_fmt in GEMV_FORMATS
                                 and K % 8 == 0 and out.stride(0) % 8 == 0):
        # (the AWQ planes have no dequantising-warp form: beyond the GEMV's eight rows they are always decoded once)
        return _linear_dequant_once(x, w, bias, out, out_fp32)
    wsp = Workspace.get(x.device)
    bn = _pick_bn(M)
    tiles = ((N + 127) // 128) * ((M + bn - 1) // bn)
    nkb = K // 64
    if splits <= 0 and tiles < NUM_SMS:
        splits = int(max(1, min(NUM_SMS // tiles, max(1, nkb // 4), 8)))
    a = GemmArgs()
    a.kind = KIND_BF16
    a.A, a.B = None, ptr(x)
    a.Ra, a.Rb, a.K = N, M, K
    a.lda, a.ldb = K, x.stride(0)
    a.out, a.out_sa, a.out_sb, a.out_fp32 = ptr(out), 1, out.stride(0), int(out_fp32)
    a.bias, a.bias_on_a = ptr(bias), 1
    a.bn, a.splits = bn, splits
    a.ws, a.ws_floats = ptr(wsp.ws), wsp.ws.numel()
    a.counters, a.n_counters = ptr(wsp.counters), wsp.counters.numel()
    a.status = ptr(wsp.status)
    a.aq_fmt, a.aq, a.aq_scale = w.aq_fmt, ptr(w.codes), ptr(w.scales)
    a.aq_ld, a.aq_sld = w.codes.stride(0), w.scales.stride(0)
    check(cuda_lib().lk_gemm_tc(C.byref(a), stream()), "lk_gemm_tc (quantised A)")
    return out


# ---- quantisers in torch (any device) ------------------------------------------------------------
# Round-to-nearest encoders that write the device planes directly.  They produce valid blocks of each
# format (what `dequantize_weight` and the kernels decode), with the plain amax scale choice instead
# of the host encoders' error-minimising search; random-init benchmark models of tens of billions of
# values are quantised with these on the GPU in seconds instead of minutes on the host.

_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _nibble_pack_t(v: torch.Tensor) -> torch.Tensor:
    """[..., K] uint8 values 0..15 -> [..., K/2]: value k in byte k/2, low nibble for even k."""
    return (v[..., 0::2] | (v[..., 1::2] << 4)).to(torch.uint8)


def quantize_weight_torch(w: torch.Tensor, fmt: str) -> QuantWeight:
    ty = TYPE_OF_NAME[fmt]
    rows, K = w.shape
    w = w.float()
    dev = w.device
    if fmt == "q8_0":
        g = w.view(rows, K // 32, 32)
        d = (g.abs().amax(2) / 127.0).half()
        df = d.float().clamp_min(1e-30)
        q = torch.round(g / df[:, :, None]).clamp(-127, 127).to(torch.int8)
        return QuantWeight(AQ_W8, ty, rows, K, q.view(rows, K).view(torch.uint8).contiguous(),
                           d.contiguous().view(torch.uint8).view(rows, K // 32 * 2))
    if fmt == "mxfp4":
        g = w.view(rows, K // 32, 32)
        amax = g.abs().amax(2).clamp_min(2.0 ** -120)
        e = torch.floor(torch.log2(amax)) - 2.0            # 6 = 1.5 * 2^2 is the largest magnitude
        e = e.clamp(-126, 127)
        x = g / torch.exp2(e)[:, :, None]
        lut = torch.tensor(_E2M1, device=dev)
        mag = (x.abs().unsqueeze(-1) - lut).abs().argmin(-1).to(torch.uint8)
        code = mag | ((x < 0).to(torch.uint8) << 3)
        codes = _nibble_pack_t(code.view(rows, K))
        ex = torch.zeros(rows, mx_sf_pitch(K), dtype=torch.uint8, device=dev)
        ex[:, :K // 32] = (e + 127).to(torch.uint8)
        return QuantWeight(AQ_MX4, ty, rows, K, codes.contiguous(), ex)
    if fmt == "q4_k":
        g = w.view(rows, K // 256, 8, 32)
        mn = (-g.amin(3)).clamp_min(0.0)
        sc = (g.amax(3) + mn) / 15.0
        d = (sc.amax(2) / 63.0).half()
        dm = (mn.amax(2) / 63.0).half()
        df, dmf = d.float().clamp_min(1e-30), dm.float().clamp_min(1e-30)
        sci = torch.round(sc / df[:, :, None]).clamp(0, 63)
        mni = torch.round(mn / dmf[:, :, None]).clamp(0, 63)
        step = (df[:, :, None] * sci).clamp_min(1e-30)
        q = torch.round((g + (dmf[:, :, None] * mni)[..., None]) / step[..., None]).clamp(0, 15).to(torch.uint8)
        codes = _nibble_pack_t(q.view(rows, K))
        rec = torch.cat([d.view(torch.uint8).view(rows, K // 256, 2), dm.view(torch.uint8).view(rows, K // 256, 2),
                         sci.to(torch.uint8), mni.to(torch.uint8)], dim=2)
        return QuantWeight(AQ_W4, ty, rows, K, codes.contiguous(), rec.view(rows, K // 256 * 20).contiguous())
    if fmt == "q6_k":
        g = w.view(rows, K // 256, 16, 16)
        s = g.abs().amax(3) / 31.0
        d = (s.amax(2) / 127.0).half()
        df = d.float().clamp_min(1e-30)
        sci = torch.round(s / df[:, :, None]).clamp(1, 127)
        q = torch.round(g / (df[:, :, None] * sci)[..., None]).clamp(-32, 31).to(torch.int8)
        rec = torch.cat([d.view(torch.uint8).view(rows, K // 256, 2), sci.to(torch.int8).view(torch.uint8)], dim=2)
        return QuantWeight(AQ_W8G16, ty, rows, K, q.view(rows, K).view(torch.uint8).contiguous(),
                           rec.view(rows, K // 256 * 18).contiguous())
    raise ValueError(fmt)
