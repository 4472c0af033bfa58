"""ctypes binding of lib/libloken_cuda.so (the sm_100a kernels) and lib/libloken_host.so.

The libraries are plain C interfaces over raw pointers: a launcher receives device addresses
taken from torch tensors and the current torch CUDA stream, so every launch is stream-ordered
with the surrounding PyTorch work and can be captured in a CUDA graph.  Nothing here falls back
to PyTorch math: a missing library is an error.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_LIBDIR = Path(__file__).resolve().parent.parent / "lib"
_cuda = None
_host = None


class LokenKernelError(RuntimeError):
    pass


def _load(name: str):
    path = _LIBDIR / name
    if not path.exists():
        from .. import build

        if name == "libloken_cuda.so":
            build.build_cuda()
        else:
            build.build_host()
    if not path.exists():
        raise LokenKernelError(f"{path} is missing and could not be built")
    return C.CDLL(str(path), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else 0)


def cuda_lib():
    global _cuda
    if _cuda is None:
        _cuda = _load("libloken_cuda.so")
        _declare_cuda(_cuda)
    return _cuda


def host_lib():
    global _host
    if _host is None:
        _host = _load("libloken_host.so")
    return _host


vp = C.c_void_p
ll = C.c_longlong


class GemvPre(C.Structure):
    """LkGemvPre of loken_cuda.h: what a quantised GEMV computes its activations from, and a residual
    update it applies on the side."""
    _fields_ = [
        ("mode", C.c_int), ("delta", vp), ("ldd", ll), ("gamma", vp), ("eps", C.c_float), ("glu_mode", C.c_int),
        ("glu_alpha", C.c_float), ("glu_limit", C.c_float), ("upd_x", vp), ("upd_delta", vp), ("upd_ldx", ll),
        ("upd_ldd", ll), ("upd_cols", C.c_int), ("prof", vp),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int), ("A", vp), ("B", vp), ("Ra", C.c_int), ("Rb", C.c_int), ("K", C.c_int),
        ("lda", ll), ("ldb", ll), ("out", vp), ("out_sa", ll), ("out_sb", ll), ("out_fp32", C.c_int),
        ("bias", vp), ("bias_on_a", C.c_int), ("residual", vp), ("a_scale", vp), ("a_mode", C.c_int),
        ("a_ld", ll), ("b_scale", vp), ("b_mode", C.c_int), ("b_ld", ll), ("bn", C.c_int),
        ("splits", C.c_int), ("ws", vp), ("ws_floats", ll), ("counters", vp), ("n_counters", C.c_int),
        ("status", vp), ("symm_view", vp),
        ("aq_fmt", C.c_int), ("aq", vp), ("aq_scale", vp), ("aq_ld", ll), ("aq_sld", ll),
        ("g_rows_per_expert", C.c_int), ("g_max_tiles", C.c_int), ("g_tile_expert", vp), ("g_tile_row0", vp),
        ("g_tile_rows", vp), ("g_ntiles", vp), ("mt", C.c_int), ("rem_mt", C.c_int), ("a_tiled", C.c_int), ("prof", vp),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", vp), ("k_cache", vp), ("v_cache", vp), ("k_scale", vp), ("v_scale", vp),
        ("block_table", vp), ("row_seq", vp), ("seq_lens", vp), ("sinks", vp), ("out", vp),
        ("out_fp8", vp), ("out_scales_t", vp), ("scale_ld", ll), ("ws", vp), ("ws_floats", ll),
        ("counters", vp), ("n_counters", C.c_int), ("status", vp), ("num_slots", ll),
        ("rows", C.c_int), ("n_q", C.c_int), ("n_kv", C.c_int), ("hd", C.c_int), ("max_blocks", C.c_int),
        ("block_size", C.c_int), ("window", C.c_int), ("kv_q8", C.c_int), ("nsplit", C.c_int),
        ("scale", C.c_float), ("parts_out", vp),
    ]


class PrefillArgs(C.Structure):
    _fields_ = [
        ("q", vp), ("k", vp), ("vt", vp), ("out", vp), ("sinks", vp),
        ("tile_seq", vp), ("tile_q0", vp), ("q_start", vp), ("q_len", vp), ("kv_off", vp), ("kv_len", vp),
        ("status", vp),
        ("n_tiles", C.c_int), ("total_q", C.c_int), ("total_kv_pad", ll), ("n_q", C.c_int), ("n_kv", C.c_int),
        ("hd", C.c_int), ("window", C.c_int), ("scale", C.c_float),
    ]


def _declare_cuda(lib):
    lib.lk_launch_count.restype = C.c_ulonglong
    lib.lk_attn_decode_ws_floats.restype = ll
    for name in ("lk_gemm_tc", "lk_attn_decode", "lk_attn_decode_tma", "lk_attn_decode_tc", "lk_attn_prefill"):
        if hasattr(lib, name):
            getattr(lib, name).restype = C.c_int


def ptr(t) -> vp:
    if t is None:
        return vp(None)
    return vp(t.data_ptr())


def stream() -> vp:
    return vp(torch.cuda.current_stream().cuda_stream)


def check(rc: int, what: str):
    if rc != 0:
        if rc > 0:
            raise LokenKernelError(f"{what}: CUDA error {rc}")
        names = {-1: "bad argument", -2: "driver entry point unavailable", -3: "tensor map encode failed",
                 -4: "workspace too small / size beyond maximum"}
        raise LokenKernelError(f"{what}: refused ({names.get(rc, rc)})")


def launch_count() -> int:
    return int(cuda_lib().lk_launch_count())


class Workspace:
    """Per-device scratch shared by kernels that reduce across CTAs (split-K partial tiles,
    split-KV attention partials), their arrival counters, and the device error word.
    Kernels on one stream run one after another, so one workspace per stream is enough."""

    _by_device: dict = {}

    def __init__(self, device, floats: int = 64 << 20, counters: int = 1 << 16):
        self.ws = torch.empty(floats, dtype=torch.float32, device=device)
        self.counters = torch.zeros(counters, dtype=torch.int32, device=device)
        self.status = torch.zeros(4, dtype=torch.int32, device=device)

    @classmethod
    def get(cls, device) -> "Workspace":
        key = (torch.device(device).index or 0) if torch.device(device).index is not None else torch.cuda.current_device()
        w = cls._by_device.get(key)
        if w is None:
            w = cls(torch.device("cuda", key))
            cls._by_device[key] = w
        return w

    def read_status(self) -> int:
        return int(self.status[0].item())

    def clear_status(self):
        self.status.zero_()
