"""Which decode layers may take the fused-GEMV form: host logic only, checked with stand-in objects.

The fused layer calls the quantised GEMVs directly, without the sum over ranks a row-parallel layer
needs, so it must never be chosen under tensor parallelism, in a sharded step, or for formats the
GEMV does not cover."""
from types import SimpleNamespace as NS

import torch

from loken_b200.models import transformer as T
from loken_b200.ops import quant


def _qw(rows, K, fmt=quant.AQ_W4G128):
    return quant.QuantWeight(fmt, 0, rows, K, torch.zeros(1, dtype=torch.uint8), torch.zeros(1, dtype=torch.uint8))


def _layer(K=256, moe=False, kind="gguf"):
    lin = lambda n, k: NS(weight=_qw(n, k), bias=None, kind=kind)
    lw = NS(wqkv=lin(3 * K, K), wo=lin(K, K), w_gate_up=None if moe else lin(4 * K, K), w_down=None if moe else lin(K, 2 * K),
            moe=NS() if moe else None)
    return lw


def _model(comm=None, moe=False, K=256):
    buf = NS(x=torch.zeros(8, K), attn=torch.zeros(8, K), gu=torch.zeros(8, 2 * K))
    return NS(cfg=NS(is_moe=moe), comm=comm, buf=buf)


def test_dense_layer_fuses_on_one_rank_only():
    lw = _layer()
    ok = T.DecoderModel._fused_front_ok
    assert ok(_model(), lw, 1, False)
    assert ok(_model(comm=NS(size=1)), lw, 4, False)
    assert not ok(_model(comm=NS(size=2)), lw, 1, False)          # partial sums must meet between the GEMVs
    assert not ok(_model(), lw, 1, True)                           # a sharded step keeps its own norm kernels
    assert not ok(_model(), lw, quant.GEMV_MAX_M + 1, False)       # beyond the GEMV's rows
    assert not ok(_model(), _layer(kind="bf16"), 1, False)


def test_mixture_layer_fuses_its_attention_half_on_one_rank_only():
    lw = _layer(moe=True)
    ok = T.DecoderModel._fused_attn_ok
    assert ok(_model(moe=True), lw, 1, False)
    assert not ok(_model(moe=True, comm=NS(size=4)), lw, 1, False)
    assert not ok(_model(moe=False), lw, 1, False)
    assert not T.DecoderModel._fused_front_ok(_model(moe=True), lw, 1, False)


def test_switch_off(monkeypatch):
    monkeypatch.setattr(T, "FUSE_GEMV_FRONT", 0)
    assert not T.DecoderModel._fused_front_ok(_model(), _layer(), 1, False)
    assert not T.DecoderModel._fused_attn_ok(_model(moe=True), _layer(moe=True), 1, False)


def test_gemv_takes_bounds_the_row_length():
    assert quant.gemv_takes(1, _qw(8, 8192))
    assert not quant.gemv_takes(8, _qw(8, 32768))                  # the token rows' codes would not fit on chip
    assert not quant.gemv_takes(1, _qw(8, 256), x_stride=260)      # rows must start 16-byte aligned
    assert not quant.gemv_takes(1, torch.zeros(4, 4))
