"""Symmetric memory between the ranks of one node and the collectives built on it.

Each rank cudaMallocs one heap through the kernel library, exports it as a CUDA IPC handle,
gathers everybody's handles over torch.distributed and maps them, so this library's kernels can
load and store peer memory directly over NVLink / NVSwitch (csrc/cuda/symm.cuh for the layout
and the signal protocol).  `SymmComm` offers the two calls the decoder makes:

    all_reduce(t, rows)       this library's one-shot push all-reduce kernel for decode-size
                              messages; larger ones go to NCCL
    all_gather_cols(logits)   NCCL all-gather (a few MB once per step)

and hands the mapped view to the GEMM launcher for the fused GEMM -> all-reduce epilogue.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops._lib import Workspace, check, cuda_lib, ptr, stream
from .comm import NcclComm

MAX_RANKS = 8


class SymmViewC(C.Structure):
    _fields_ = [("base", C.c_void_p * MAX_RANKS), ("world", C.c_int), ("rank", C.c_int),
                ("flags_off", C.c_longlong), ("recv_off", C.c_longlong), ("slot_bytes", C.c_longlong),
                ("max_chunks", C.c_int), ("pad", C.c_int),
                ("ll_off", C.c_longlong), ("ll_half_bytes", C.c_longlong), ("ll_hop2_off", C.c_longlong)]


class SymmHeap:
    """One rank's heap plus the mapped heaps of its peers."""

    def __init__(self, slot_bytes: int, max_chunks: int = 256, group=None, ll_hop1_bytes: int = 0,
                 ll_hop2_bytes: int = 0):
        lib = cuda_lib()
        assert lib.lk_symm_view_size() == C.sizeof(SymmViewC), "SymmView layout mismatch"
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert self.world <= MAX_RANKS
        self.slot_bytes = (slot_bytes + 255) // 256 * 256
        self.max_chunks = max_chunks
        self.flags_off = 256
        flags_bytes = 2 * MAX_RANKS * max_chunks * 4
        self.recv_off = (self.flags_off + flags_bytes + 1023) // 1024 * 1024
        # flag-in-data areas (two halves): first-hop region, then second-hop region
        self.ll_off = (self.recv_off + 2 * MAX_RANKS * self.slot_bytes + 1023) // 1024 * 1024
        self.ll_hop2_off = (ll_hop1_bytes + 1023) // 1024 * 1024
        self.ll_half_bytes = self.ll_hop2_off + (ll_hop2_bytes + 1023) // 1024 * 1024
        self.bytes = self.ll_off + 2 * self.ll_half_bytes
        p = C.c_void_p()
        check(lib.lk_symm_alloc(C.c_longlong(self.bytes), C.byref(p)), "lk_symm_alloc")
        self.local = p.value
        self.mapped: List[Optional[int]] = [None] * self.world
        self.mapped[self.rank] = self.local
        if self.world > 1:
            h = (C.c_ubyte * 64)()
            check(lib.lk_ipc_export(C.c_void_p(self.local), h), "lk_ipc_export")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(h), group=group)
            for r, hb in enumerate(handles):
                if r == self.rank:
                    continue
                buf = (C.c_ubyte * 64).from_buffer_copy(hb)
                q = C.c_void_p()
                check(lib.lk_ipc_open(buf, C.byref(q)), "lk_ipc_open")
                self.mapped[r] = q.value
            dist.barrier(group=group)
        v = SymmViewC()
        for r in range(self.world):
            v.base[r] = self.mapped[r]
        v.world, v.rank = self.world, self.rank
        v.flags_off, v.recv_off, v.slot_bytes = self.flags_off, self.recv_off, self.slot_bytes
        v.max_chunks = max_chunks
        v.ll_off, v.ll_half_bytes, v.ll_hop2_off = self.ll_off, self.ll_half_bytes, self.ll_hop2_off
        self.view = v

    def close(self):
        lib = cuda_lib()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        for r, p in enumerate(self.mapped):
            if p is not None and r != self.rank:
                lib.lk_ipc_close(C.c_void_p(p))
        if self.local:
            lib.lk_symm_free(C.c_void_p(self.local))
            self.local = None
        self.mapped = []


class SymmComm:
    def __init__(self, device, max_rows: int, hidden: int, group=None, push_max_bytes: int = 4 << 20,
                 top_k: int = 0):
        self.device = device
        self.group = group
        self.size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        # flag-in-data areas of the fused layer-boundary kernel: partial rows (4 bytes per value, every
        # source's share of this rank's rows) and normalised rows (at most 4 bytes per value + scales)
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.max_rows, self.hidden = max_rows, hidden
        hop1 = (max_rows + world) * hidden * 4
        hop2 = max_rows * (hidden * 4 + hidden // 16 + 16)
        if top_k:
            # expert-parallel dispatch: every (token, choice) pair may land on one rank: a 16-byte header and
            # 4 bytes per value per slot, world * ceil(max_rows / world) * top_k slots (csrc/cuda/ep_moe.cu)
            hop1 = max(hop1, 256 + (max_rows + world) * top_k * (16 + hidden * 4) - hop2)
        self.heap = SymmHeap(max_rows * hidden * 2, group=group, ll_hop1_bytes=hop1, ll_hop2_bytes=hop2)
        self.nccl = NcclComm(group)
        self.push_max_bytes = min(push_max_bytes, self.heap.slot_bytes)
        self.wsp = Workspace.get(device)
        self.collectives = 0
        # True: row-parallel GEMMs sum inside their epilogue; False: GEMM, then `all_reduce`.  Measured on
        # the 70B decode step the second is faster at 2 and at 8 ranks (17.7 / 12.4 against 19.1 / 13.7 ms).
        self.fused_gemm = False
        # True: a row-parallel layer's partial sums go through `sum_norm` (reduce-scatter + residual +
        # RMSNorm + quantise + all-gather in one kernel, residual stream sharded by rows in between)
        self.fused_norm = True

    def can_sum_norm(self, rows: int, hidden: int) -> bool:
        return self.size > 1 and self.fused_norm and rows <= self.max_rows and hidden == self.hidden \
            and hidden % 8 == 0 and self.size in (2, 4, 8)

    def sum_norm(self, partial: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float, rows: int, *,
                 out: Optional[torch.Tensor] = None, out_fp8=None, gather: bool = True, local: bool = False):
        """x[own rows] += sum over ranks of partial[own rows]; normalised rows -> `out` (bf16) or `out_fp8`
        (e4m3 + per-128 scales): every row on every rank when `gather`, else the owned rows only.
        Row r belongs to rank r // ceil(rows / world).  `local`: `partial` already is the complete update of
        the owned rows (the expert-parallel combine's output), nothing is summed over ranks."""
        H = x.shape[1]
        check(cuda_lib().lk_tp_sum_norm(C.byref(self.heap.view), ptr(partial), C.c_longlong(partial.stride(0)),
                                        ptr(x), C.c_longlong(x.stride(0)), ptr(w), C.c_float(eps), rows, H,
                                        ptr(out), C.c_longlong(out.stride(0) if out is not None else 0),
                                        ptr(out_fp8.data) if out_fp8 is not None else None,
                                        ptr(out_fp8.scale_t) if out_fp8 is not None else None,
                                        C.c_longlong(out_fp8.scale_t.stride(0) if out_fp8 is not None else 0),
                                        int(gather), int(local), ptr(self.wsp.status), stream()), "lk_tp_sum_norm")
        self.collectives += 1

    def owned_rows(self, rows: int) -> tuple:
        rpr = (rows + self.size - 1) // self.size
        return min(rows, self.rank * rpr), min(rows, (self.rank + 1) * rpr)

    def all_reduce(self, t: torch.Tensor, rows: int, residual: Optional[torch.Tensor] = None):
        if self.size == 1:
            return
        cols = t.shape[1]
        if rows * cols * 2 > self.push_max_bytes:
            self.nccl.all_reduce(t, rows)
            if residual is not None:
                t[:rows].add_(residual[:rows])
            return
        check(cuda_lib().lk_allreduce_push(C.byref(self.heap.view), ptr(t), rows, cols, C.c_longlong(t.stride(0)),
                                           ptr(residual), ptr(self.wsp.status), stream()), "lk_allreduce_push")
        self.collectives += 1

    @staticmethod
    def set_allreduce_mode(mode: int):
        """0: the library picks (two-shot from four ranks and 256 KiB up), 1: one-shot, 2: two-shot.
        Process-wide; every rank has to set the same value."""
        cuda_lib().lk_allreduce_set_mode(C.c_int(mode))

    def all_gather_cols(self, logits: torch.Tensor) -> torch.Tensor:
        return self.nccl.all_gather_cols(logits)

    def barrier(self):
        self.nccl.barrier()

    def close(self):
        self.heap.close()
