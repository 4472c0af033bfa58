"""Dry planning: what a load will take on the device, without allocating anything, and how an
allocator would lay those blocks out.

`dry_demand(cfg, ...)` walks the same shapes the loader, the KV pool, the decoder's static buffers
and the decode graphs allocate (`models/weights.py`, `models/transformer.py:Buffers`,
`serve/runner.py`) and returns the list of blocks (name, bytes) with their total: the role of the
reference's allocation-free "dry device" that runs the real forward to get the exact peak
(`src/tensor/dry.rs:1-16`, `src/inference/place/dry_plan.rs`).  `HeapReplay` replays such a list
through a first-fit allocator with the CUDA caching allocator's rounding (512-byte small blocks,
2 MiB segments for large ones) to show the fragmentation a plan would meet
(`src/tensor/heap.rs:1-18`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from ..models.config import ModelConfig

MiB = 1 << 20


def _fmt_bits(fmt: str) -> float:
    return {"bf16": 16.0, "fp8_block": 8.0 + 32.0 / (128 * 128), "q8_0": 8.5, "q4_k": 4.5 + 0.125, "q6_k": 8.0 + 0.5625,
            "mxfp4": 4.25}.get(fmt, 16.0)


@dataclass
class Demand:
    blocks: List[Tuple[str, int]] = field(default_factory=list)

    def add(self, name: str, nbytes: float):
        self.blocks.append((name, int(nbytes)))

    @property
    def total(self) -> int:
        return sum(b for _, b in self.blocks)

    def by_group(self) -> Dict[str, int]:
        out: Dict[str, int] = {}
        for n, b in self.blocks:
            g = n.split("/", 1)[0]
            out[g] = out.get(g, 0) + b
        return out


def dry_demand(cfg: ModelConfig, *, tp: int = 1, ep: int = 1, max_seqs: int = 256, max_ctx: int = 8192,
               max_prefill_tokens: int = 8192, num_blocks: Optional[int] = None, block_size: int = 16,
               graph_buckets: Optional[List[int]] = None) -> Demand:
    """Every device block a load of `cfg` at this degree makes, by the constructors' own shapes."""
    from ..models.weights import linear_format

    d = Demand()
    H, hd = cfg.hidden, cfg.head_dim
    nq, nkv = cfg.n_q // tp, max(1, cfg.n_kv // tp)
    vl = cfg.vocab // tp if tp > 1 else cfg.vocab
    d.add("weights/embed", cfg.vocab * H * 2)
    if not cfg.tie_embeddings or tp > 1:
        d.add("weights/lm_head", vl * H * 2)
    for il in range(cfg.n_layers):
        d.add(f"weights/l{il}/qkv", (nq + 2 * nkv) * hd * H * _fmt_bits(linear_format(cfg, "qkv")) / 8)
        d.add(f"weights/l{il}/o", H * nq * hd * _fmt_bits(linear_format(cfg, "o")) / 8)
        if cfg.is_moe:
            e_local = cfg.n_experts // ep
            I = cfg.expert_intermediate
            bits = _fmt_bits(linear_format(cfg, "expert"))
            d.add(f"weights/l{il}/experts_gate_up", e_local * 2 * I * H * bits / 8)
            d.add(f"weights/l{il}/experts_down", e_local * H * I * bits / 8)
            d.add(f"weights/l{il}/router", cfg.n_experts * H * 2)
        else:
            I = cfg.intermediate // tp
            d.add(f"weights/l{il}/gate_up", 2 * I * H * _fmt_bits(linear_format(cfg, "gate_up")) / 8)
            d.add(f"weights/l{il}/down", H * I * _fmt_bits(linear_format(cfg, "down")) / 8)
        d.add(f"weights/l{il}/norms", 2 * H * 4)
    # paged KV pool
    per_tok = (hd + (hd // 32) * 2) if cfg.kv_format == "q8" else hd * 2
    if num_blocks is None:
        num_blocks = (max_seqs * max_ctx) // block_size + 64
    for il in range(cfg.n_layers):
        d.add(f"kv/l{il}", 2 * num_blocks * block_size * nkv * per_tok)
    # static activation buffers of the decoder (sized for the largest step)
    cap = max(max_prefill_tokens, max_seqs)
    act = cap * (3 * H * 2 + (nq + 2 * nkv) * hd * 2 + 2 * nq * hd * 2 + H + nq * hd)
    if not cfg.is_moe:
        I = cfg.intermediate // tp
        act += cap * (2 * I * 2 + I * 2 + I)
    else:
        P = (cap + ep) * cfg.top_k + 256
        act += P * (H * 2 * 2 + cfg.expert_intermediate * 2 * 3 + H + cfg.expert_intermediate)
    d.add("activations/decoder", act)
    d.add("activations/logits", cap * vl * 4 * (2 if tp > 1 else 1))
    d.add("activations/prefill_kv_gather", 2 * max(4096, max_prefill_tokens + max_ctx) * nkv * hd * 2)
    d.add("workspace/splitk+status", (64 << 20) * 4 + (1 << 16) * 4)
    # decode graphs: a captured graph keeps its own copies of the launch parameters, little memory; the
    # staging buffers per bucket are what counts
    for b in (graph_buckets or [1, 2, 4, 8, 16, 32, 64, 128, 256]):
        if b <= max_seqs:
            d.add(f"graphs/bucket{b}", b * (vl * 4 + 64) + (2 << 20))
    if tp > 1 or ep > 1:
        world = max(tp, ep)
        rows = max(max_seqs, 256)
        slot = rows * H * 2
        hop1 = (rows + world) * H * 4
        hop2 = rows * (H * 4 + H // 16 + 16)
        if cfg.is_moe:
            hop1 = max(hop1, 256 + (rows + world) * cfg.top_k * (16 + H * 4) - hop2)
        d.add("symmetric_heap", 2 * 8 * slot + 2 * (hop1 + hop2) + (1 << 20))
    return d


class HeapReplay:
    """First-fit replay of (alloc, free) events with the caching allocator's granularity."""

    SMALL = 1 * MiB          # requests up to this size come from 2 MiB small-pool segments in 512-byte units
    SEGMENT = 2 * MiB        # large requests are rounded up to whole 2 MiB segments (20 MiB+: exact multiples)

    def __init__(self, capacity: int):
        self.capacity = capacity
        self.free_list: List[Tuple[int, int]] = [(0, capacity)]     # (offset, size), sorted by offset
        self.live: Dict[str, Tuple[int, int]] = {}
        self.peak = 0
        self.failed: List[Tuple[str, int]] = []

    @classmethod
    def round(cls, n: int) -> int:
        if n <= cls.SMALL:
            return (n + 511) // 512 * 512
        return (n + cls.SEGMENT - 1) // cls.SEGMENT * cls.SEGMENT

    def alloc(self, name: str, nbytes: int) -> bool:
        n = self.round(max(1, nbytes))
        for i, (off, size) in enumerate(self.free_list):
            if size >= n:
                self.live[name] = (off, n)
                if size == n:
                    self.free_list.pop(i)
                else:
                    self.free_list[i] = (off + n, size - n)
                self.peak = max(self.peak, max(o + s for o, s in self.live.values()))
                return True
        self.failed.append((name, nbytes))
        return False

    def free(self, name: str):
        off, n = self.live.pop(name)
        self.free_list.append((off, n))
        self.free_list.sort()
        merged: List[Tuple[int, int]] = []
        for o, s in self.free_list:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + s)
            else:
                merged.append((o, s))
        self.free_list = merged

    @property
    def used(self) -> int:
        return sum(s for _, s in self.live.values())

    @property
    def largest_free(self) -> int:
        return max((s for _, s in self.free_list), default=0)

    def fragmentation(self) -> float:
        """Share of the free memory that the largest free block does not cover."""
        free = sum(s for _, s in self.free_list)
        return 0.0 if free == 0 else 1.0 - self.largest_free / free


def fits(cfg: ModelConfig, free_bytes: int, **kw) -> Tuple[bool, Demand, HeapReplay]:
    """Would the load fit `free_bytes`, fragmentation included?  (the dry plan of a load admission)"""
    d = dry_demand(cfg, **kw)
    heap = HeapReplay(free_bytes)
    ok = all(heap.alloc(n, b) for n, b in d.blocks)
    return ok, d, heap
