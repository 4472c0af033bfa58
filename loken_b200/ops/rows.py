"""Row kernels: embedding gather, residual add + RMSNorm (+ e4m3 quantise), GLU activations
(+ e4m3 quantise), the stand-alone activation quantiser, and fused RoPE + paged KV write."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ._lib import Workspace, check, cuda_lib, ptr, stream
from .gemm import Fp8Act


def _f(x):
    return C.c_float(float(x))


def embed(tokens: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0):
    T = tokens.numel()
    V, H = table.shape
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=table.device)
    check(cuda_lib().lk_embed_bf16(ptr(tokens), ptr(table), ptr(out), T, H, V, _f(scale), stream()), "lk_embed_bf16")
    return out


def alloc_fp8_act(rows: int, K: int, device) -> Fp8Act:
    ld = (rows + 3) // 4 * 4
    return Fp8Act(torch.empty(rows, K, dtype=torch.float8_e4m3fn, device=device),
                  torch.ones(K // 128, ld, dtype=torch.float32, device=device))


def add_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, *, delta: Optional[torch.Tensor] = None,
                delta_f32: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                out_fp8: Optional[Fp8Act] = None, write_x: bool = True, rows: Optional[int] = None):
    """x += delta (in place, bf16 residual stream), then RMSNorm(x) * w into `out` (bf16) and/or
    `out_fp8` (e4m3 + per-128 scales).  w is f32 [H]."""
    T = rows if rows is not None else x.shape[0]
    H = x.shape[1]
    assert w.dtype == torch.float32
    check(cuda_lib().lk_add_rmsnorm(ptr(x), ptr(delta), ptr(delta_f32), ptr(w), _f(eps), T, H, ptr(out),
                                    ptr(out_fp8.data) if out_fp8 else None,
                                    ptr(out_fp8.scale_t) if out_fp8 else None,
                                    C.c_longlong(out_fp8.scale_t.stride(0) if out_fp8 else 0), int(write_x),
                                    stream()), "lk_add_rmsnorm")
    return out if out is not None else out_fp8


def glu(gate_up: torch.Tensor, *, mode: int = 0, alpha: float = 1.702, limit: float = 7.0,
        out: Optional[torch.Tensor] = None, out_fp8: Optional[Fp8Act] = None, rows: Optional[int] = None):
    """gate_up [T, 2I] (gate | up) -> silu(g)*u (mode 0) or the clamped gpt-oss form (mode 1)."""
    T = rows if rows is not None else gate_up.shape[0]
    I = gate_up.shape[1] // 2
    check(cuda_lib().lk_glu(ptr(gate_up), C.c_longlong(gate_up.stride(0)), T, I, mode, _f(alpha), _f(limit),
                            ptr(out), ptr(out_fp8.data) if out_fp8 else None,
                            ptr(out_fp8.scale_t) if out_fp8 else None,
                            C.c_longlong(out_fp8.scale_t.stride(0) if out_fp8 else 0), stream()), "lk_glu")
    return out if out is not None else out_fp8


def quant_fp8(x: torch.Tensor, out: Optional[Fp8Act] = None, rows: Optional[int] = None) -> Fp8Act:
    T = rows if rows is not None else x.shape[0]
    K = x.shape[1]
    if out is None:
        out = alloc_fp8_act(x.shape[0], K, x.device)
    check(cuda_lib().lk_quant_fp8(ptr(x), C.c_longlong(x.stride(0)), T, K, ptr(out.data), ptr(out.scale_t),
                                  C.c_longlong(out.scale_t.stride(0)), stream()), "lk_quant_fp8")
    return out


def add_(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None):
    out = a if out is None else out
    check(cuda_lib().lk_add_bf16(ptr(a), ptr(b), ptr(out), C.c_longlong(a.numel()), stream()), "lk_add_bf16")
    return out


class KVCacheLayer:
    """One layer's paged KV storage.  q8: int8 codes [slots, n_kv, hd] + f16 scales
    [slots, n_kv, hd/32] for K and for V; otherwise bf16 [slots, n_kv, hd]."""

    def __init__(self, num_slots: int, n_kv: int, hd: int, device, q8: bool = True):
        self.num_slots, self.n_kv, self.hd, self.q8 = num_slots, n_kv, hd, q8
        if q8:
            self.k = torch.zeros(num_slots, n_kv, hd, dtype=torch.int8, device=device)
            self.v = torch.zeros(num_slots, n_kv, hd, dtype=torch.int8, device=device)
            self.k_scale = torch.zeros(num_slots, n_kv, hd // 32, dtype=torch.float16, device=device)
            self.v_scale = torch.zeros(num_slots, n_kv, hd // 32, dtype=torch.float16, device=device)
        else:
            self.k = torch.zeros(num_slots, n_kv, hd, dtype=torch.bfloat16, device=device)
            self.v = torch.zeros(num_slots, n_kv, hd, dtype=torch.bfloat16, device=device)
            self.k_scale = self.v_scale = None

    def dequant(self):
        if not self.q8:
            return self.k.float(), self.v.float()
        ks = self.k_scale.float().repeat_interleave(32, dim=2)
        vs = self.v_scale.float().repeat_interleave(32, dim=2)
        return self.k.float() * ks, self.v.float() * vs


def kv_shift(cache: KVCacheLayer, src: torch.Tensor, dst: torch.Tensor, delta: torch.Tensor, inv_freq: torch.Tensor, *,
             rope_dim: Optional[int] = None, pairing: int = 1):
    """Context shift on one layer's cache: position i moves from slot src[i] to slot dst[i] (int32, no
    overlap between the two sets) and its key is turned by delta[i] positions; values are copied."""
    n = src.numel()
    wsp = Workspace.get(cache.k.device)
    check(cuda_lib().lk_kv_shift(ptr(cache.k), ptr(cache.v), ptr(cache.k_scale), ptr(cache.v_scale), ptr(src), ptr(dst),
                                 ptr(delta), n, cache.n_kv, cache.hd, ptr(inv_freq),
                                 rope_dim if rope_dim is not None else cache.hd, pairing,
                                 C.c_longlong(cache.num_slots), int(cache.q8), ptr(wsp.status), stream()), "lk_kv_shift")


def rope_kv(qkv: torch.Tensor, pos: torch.Tensor, slots: torch.Tensor, cache: KVCacheLayer, n_q: int,
            inv_freq: torch.Tensor, *, rope_dim: Optional[int] = None, pairing: int = 1, mscale: float = 1.0,
            q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6,
            q_out: Optional[torch.Tensor] = None, rows: Optional[int] = None, wide_rinv: Optional[torch.Tensor] = None):
    """qkv [T, (n_q + 2 n_kv) * hd] bf16 -> rotated q [T, n_q, hd]; K and V rows stored at `slots`.  With
    `wide_rinv` ([T, 2] f32 scratch) the q / k norm runs over the token's whole projection (weights of
    n_q * hd and n_kv * hd entries) instead of per head."""
    T = rows if rows is not None else qkv.shape[0]
    hd, n_kv = cache.hd, cache.n_kv
    if q_out is None:
        q_out = torch.empty(qkv.shape[0], n_q, hd, dtype=torch.bfloat16, device=qkv.device)
    wsp = Workspace.get(qkv.device)
    if wide_rinv is not None:
        assert q_norm_w.numel() == n_q * hd and k_norm_w.numel() == n_kv * hd and wide_rinv.shape[0] >= T
        check(cuda_lib().lk_rope_kv_wide(ptr(qkv), C.c_longlong(qkv.stride(0)), ptr(pos), ptr(slots), T, n_q, n_kv, hd,
                                         ptr(q_norm_w), ptr(k_norm_w), _f(eps), ptr(inv_freq),
                                         rope_dim if rope_dim is not None else hd, pairing, _f(mscale), ptr(q_out),
                                         ptr(cache.k), ptr(cache.v), ptr(cache.k_scale), ptr(cache.v_scale),
                                         C.c_longlong(cache.num_slots), int(cache.q8), ptr(wsp.status), ptr(wide_rinv),
                                         stream()), "lk_rope_kv_wide")
        return q_out
    check(cuda_lib().lk_rope_kv(ptr(qkv), C.c_longlong(qkv.stride(0)), ptr(pos), ptr(slots), T, n_q, n_kv, hd,
                                ptr(q_norm_w), ptr(k_norm_w), _f(eps), ptr(inv_freq),
                                rope_dim if rope_dim is not None else hd, pairing, _f(mscale), ptr(q_out),
                                ptr(cache.k), ptr(cache.v), ptr(cache.k_scale), ptr(cache.v_scale),
                                C.c_longlong(cache.num_slots), int(cache.q8), ptr(wsp.status), stream()),
          "lk_rope_kv")
    return q_out
