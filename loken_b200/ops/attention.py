"""Attention over the paged KV cache: flash decode (one query row per sequence or per verify
row) and tcgen05 flash prefill (variable-length, chunked, prefix-cached)."""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ._lib import DecodeArgs, PrefillArgs, Workspace, check, cuda_lib, ptr, stream
from .gemm import Fp8Act
from .rows import KVCacheLayer

NUM_SMS = 148
# decode kernel for head_dim 128 + q8 cache + 16-token pages: "tc" = tcgen05 (both products on the
# tensor cores), "tma" = SIMT over TMA-staged pages, "simt" = the first kernel (any shape)
DECODE_KERNEL = "tc"


def pick_decode_splits(rows: int, n_kv: int, max_ctx: int) -> int:
    """Key splits per (row, kv head).  Measured on B200: a block costs ~6 us of set-up, first-page
    latency and split merge on top of ~0.6 us per 128 keys, so splitting only pays while the grid
    does not yet cover the SMs once; beyond that one block per (row, kv head) is fastest.  A split
    keeps at least 256 keys."""
    blocks = max(1, rows * n_kv)
    want = max(1, (NUM_SMS + blocks - 1) // blocks)
    by_len = max(1, max_ctx // 256)
    return int(max(1, min(want, by_len, 64)))


def decode(q: torch.Tensor, cache: KVCacheLayer, block_table: torch.Tensor, seq_lens: torch.Tensor, *,
           block_size: int, scale: Optional[float] = None, window: int = 0, sinks: Optional[torch.Tensor] = None,
           row_seq: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
           out_fp8: Optional[Fp8Act] = None, nsplit: int = 1, rows: Optional[int] = None,
           parts_out: Optional[torch.Tensor] = None):
    """q [rows, n_q, hd] bf16 -> out [rows, n_q*hd] bf16 (and/or e4m3 with per-head scales).  With `parts_out`
    (f32 [rows, n_q, hd + 2]) nothing is normalised or written to `out`: the tensor receives what this cache
    contributes to the attention (weighed values, maximum in log2 units, sum of weights), to be merged with the
    parts of the other ranges of the context (`parallel/context_parallel.py`)."""
    R = rows if rows is not None else q.shape[0]
    n_q, hd = q.shape[1], q.shape[2]
    if parts_out is not None:
        assert parts_out.dtype == torch.float32 and tuple(parts_out.shape[1:]) == (n_q, hd + 2) and sinks is None
        out = parts_out                      # nothing else is written
    if out is None and out_fp8 is None:
        out = torch.empty(q.shape[0], n_q * hd, dtype=torch.bfloat16, device=q.device)
    wsp = Workspace.get(q.device)
    a = DecodeArgs()
    a.q = ptr(q)
    a.k_cache, a.v_cache = ptr(cache.k), ptr(cache.v)
    a.k_scale, a.v_scale = ptr(cache.k_scale), ptr(cache.v_scale)
    a.block_table, a.row_seq, a.seq_lens = ptr(block_table), ptr(row_seq), ptr(seq_lens)
    a.sinks = ptr(sinks)
    a.out = ptr(out)
    a.out_fp8 = ptr(out_fp8.data) if out_fp8 is not None else None
    a.out_scales_t = ptr(out_fp8.scale_t) if out_fp8 is not None else None
    a.scale_ld = out_fp8.scale_t.stride(0) if out_fp8 is not None else 0
    a.ws, a.ws_floats = ptr(wsp.ws), wsp.ws.numel()
    a.counters, a.n_counters = ptr(wsp.counters), wsp.counters.numel()
    a.status = ptr(wsp.status)
    a.num_slots = cache.num_slots
    a.rows, a.n_q, a.n_kv, a.hd = R, n_q, cache.n_kv, hd
    a.max_blocks, a.block_size, a.window = block_table.shape[1], block_size, window
    a.kv_q8, a.nsplit = int(cache.q8), nsplit
    a.scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if parts_out is not None:
        a.out, a.parts_out = None, ptr(parts_out)
        check(cuda_lib().lk_attn_decode(C.byref(a), stream()), "lk_attn_decode (parts)")
        return parts_out
    fast = hd == 128 and cache.q8 and block_size == 16
    if fast and DECODE_KERNEL == "tc" and n_q // cache.n_kv in (1, 2, 4, 8):
        check(cuda_lib().lk_attn_decode_tc(C.byref(a), stream()), "lk_attn_decode_tc")
    elif fast and DECODE_KERNEL in ("tc", "tma") and n_q // cache.n_kv in (1, 2, 4, 8):
        check(cuda_lib().lk_attn_decode_tma(C.byref(a), stream()), "lk_attn_decode_tma")
    else:
        check(cuda_lib().lk_attn_decode(C.byref(a), stream()), "lk_attn_decode")
    return out if out is not None else out_fp8


@dataclass
class PrefillPlan:
    """Device-side description of one variable-length prefill step (built on the host once per
    step, shared by every layer): the 128-row query tiles, where each sequence's keys sit in the
    gathered K / V^T buffers, and the 32-token tiles the gather kernel copies."""
    n_seqs: int
    total_q: int
    total_kv_pad: int
    n_tiles: int
    n_gather_tiles: int
    tile_seq: torch.Tensor
    tile_q0: torch.Tensor
    q_start: torch.Tensor
    q_len: torch.Tensor
    kv_off: torch.Tensor
    kv_len: torch.Tensor
    g_seq: torch.Tensor
    g_tok0: torch.Tensor
    seq_rows: torch.Tensor     # block-table row of each sequence


def plan_prefill(q_lens: Sequence[int], kv_lens: Sequence[int], group: int, device,
                 seq_rows: Optional[Sequence[int]] = None) -> PrefillPlan:
    """q_lens[s] new tokens per sequence, kv_lens[s] total keys (cached prefix + new).
    `group` = query heads per kv head (fixes how many tokens a 128-row tile holds)."""
    group = 1 if group <= 1 else 2 if group <= 2 else 4 if group <= 4 else 8      # the kernel's tile shapes (head slots)
    tq = 128 // group
    tile_seq, tile_q0, q_start, kv_off, g_seq, g_tok0 = [], [], [], [], [], []
    qs = kv = 0
    for s, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        q_start.append(qs)
        kv_off.append(kv)
        for t0 in range(0, ql, tq):
            tile_seq.append(s)
            tile_q0.append(t0)
        pad = (kl + 127) // 128 * 128
        for t0 in range(0, pad, 32):
            g_seq.append(s)
            g_tok0.append(t0)
        qs += ql
        kv += pad
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return PrefillPlan(len(q_lens), qs, max(kv, 128), len(tile_seq), len(g_seq), i32(tile_seq), i32(tile_q0),
                       i32(q_start), i32(list(q_lens)), i32(kv_off), i32(list(kv_lens)), i32(g_seq), i32(g_tok0),
                       i32(list(seq_rows) if seq_rows is not None else list(range(len(q_lens)))))


def kv_gather(cache: KVCacheLayer, block_table: torch.Tensor, plan: PrefillPlan, block_size: int,
              k_out: Optional[torch.Tensor] = None, vt_out: Optional[torch.Tensor] = None):
    """Dequantise the planned sequences' keys/values out of the paged cache into dense bf16
    K [total_kv_pad, n_kv, hd] and V^T [n_kv, hd, total_kv_pad]."""
    dev = cache.k.device
    if k_out is None:
        k_out = torch.empty(plan.total_kv_pad, cache.n_kv, cache.hd, dtype=torch.bfloat16, device=dev)
    if vt_out is None:
        vt_out = torch.empty(cache.n_kv, cache.hd, plan.total_kv_pad, dtype=torch.bfloat16, device=dev)
    bt = block_table.index_select(0, plan.seq_rows.long()).contiguous() if plan.seq_rows is not None else block_table
    check(cuda_lib().lk_kv_gather(ptr(cache.k), ptr(cache.v), ptr(cache.k_scale), ptr(cache.v_scale),
                                  int(cache.q8), cache.n_kv, cache.hd, ptr(bt), bt.shape[1], block_size,
                                  ptr(plan.g_seq), ptr(plan.g_tok0), plan.n_gather_tiles, ptr(plan.kv_len),
                                  ptr(plan.kv_off), ptr(k_out), ptr(vt_out), C.c_longlong(vt_out.shape[2]),
                                  C.c_longlong(cache.num_slots), stream()), "lk_kv_gather")
    return k_out, vt_out


def prefill(q: torch.Tensor, k: torch.Tensor, vt: torch.Tensor, plan: PrefillPlan, *,
            scale: Optional[float] = None, window: int = 0, sinks: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None):
    """q [total_q, n_q, hd], k [total_kv_pad, n_kv, hd], vt [n_kv, hd, total_kv_pad] (all bf16)
    -> out [total_q, n_q*hd]."""
    n_q, hd = q.shape[1], q.shape[2]
    n_kv = k.shape[1]
    if out is None:
        out = torch.empty(q.shape[0], n_q * hd, dtype=torch.bfloat16, device=q.device)
    wsp = Workspace.get(q.device)
    a = PrefillArgs()
    a.q, a.k, a.vt, a.out, a.sinks = ptr(q), ptr(k), ptr(vt), ptr(out), ptr(sinks)
    a.tile_seq, a.tile_q0 = ptr(plan.tile_seq), ptr(plan.tile_q0)
    a.q_start, a.q_len, a.kv_off, a.kv_len = ptr(plan.q_start), ptr(plan.q_len), ptr(plan.kv_off), ptr(plan.kv_len)
    a.status = ptr(wsp.status)
    a.n_tiles, a.total_q, a.total_kv_pad = plan.n_tiles, q.shape[0], vt.shape[2]
    a.n_q, a.n_kv, a.hd, a.window = n_q, n_kv, hd, window
    a.scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    check(cuda_lib().lk_attn_prefill(C.byref(a), stream()), "lk_attn_prefill")
    return out


# ---- fp32 reference used by the tests and the CPU oracle -------------------------------------

def attention_ref(q, k, v, q_pos0: int, *, scale=None, window: int = 0, sinks=None):
    """q [Tq, n_q, hd], k/v [Tk, n_kv, hd] (float32), query i sits at position q_pos0 + i.
    Returns [Tq, n_q*hd]."""
    Tq, n_q, hd = q.shape
    Tk, n_kv, _ = k.shape
    G = n_q // n_kv
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    kk = k.repeat_interleave(G, dim=1)
    vv = v.repeat_interleave(G, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk.float()) * scale
    qi = torch.arange(Tq, device=q.device)[:, None] + q_pos0
    kj = torch.arange(Tk, device=q.device)[None, :]
    mask = kj > qi
    if window > 0:
        mask |= (kj + window) <= qi
    s = s.masked_fill(mask[None], float("-inf"))
    if sinks is not None:
        s = torch.cat([s, sinks.float()[:, None, None].expand(n_q, Tq, 1)], dim=2)
        p = torch.softmax(s, dim=2)[:, :, :-1]
    else:
        p = torch.softmax(s, dim=2)
    o = torch.einsum("hqk,khd->qhd", p, vv.float())
    return o.reshape(Tq, n_q * hd)
