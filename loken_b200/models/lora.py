"""LoRA adapters (PEFT layout) folded into the base weights at load time.

An adapter directory holds `adapter_config.json` (`r`, `lora_alpha`, `target_modules`) and
`adapter_model.safetensors` with `...layers.{i}.{self_attn|mlp}.{proj}.lora_A.weight` [r, in] and
`lora_B.weight` [out, r].  `merge_lora` adds `(lora_alpha / r) * B @ A` to each targeted projection:
bf16 weights are updated in place, block-fp8 weights are expanded, updated and quantised again with
fresh block scales.  Several adapters merge one after the other, each with its own weight.

The reference keeps adapters separate and applies several per batch in one fused kernel
(`src/tensor/lora.rs`, `src/inference/load/lora.rs`); merging costs nothing per token and serves one
adapter mix per loaded model, which is what this module offers.  GGUF block formats are refused
(re-quantising them would change the base model's codes).
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch

from .weights import Linear, ModelWeights, dequant_linear, make_linear

_KEY = re.compile(r"layers\.(\d+)\.(?:self_attn|mlp)\.(q_proj|k_proj|v_proj|o_proj|gate_proj|up_proj|down_proj)"
                  r"\.lora_([AB])(?:\.[^.]+)?\.weight$")


@dataclass
class LoraAdapter:
    r: int
    alpha: float
    # (layer, projection) -> (A [r, in], B [out, r]), fp32 on the CPU
    pairs: Dict[Tuple[int, str], Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)

    @property
    def scale(self) -> float:
        return self.alpha / self.r


def adapter_from_tensors(tensors: Dict[str, torch.Tensor], r: int, alpha: float) -> LoraAdapter:
    halves: Dict[Tuple[int, str], Dict[str, torch.Tensor]] = {}
    for name, t in tensors.items():
        m = _KEY.search(name)
        if not m:
            continue
        halves.setdefault((int(m.group(1)), m.group(2)), {})[m.group(3)] = t.float().cpu()
    ad = LoraAdapter(r, alpha)
    for key, h in halves.items():
        if "A" not in h or "B" not in h:
            raise ValueError(f"adapter tensor pair of layer {key[0]} {key[1]} is incomplete")
        if h["A"].shape[0] != h["B"].shape[1]:
            raise ValueError(f"rank mismatch in layer {key[0]} {key[1]}: A {tuple(h['A'].shape)}, B {tuple(h['B'].shape)}")
        ad.pairs[key] = (h["A"], h["B"])
    if not ad.pairs:
        raise ValueError("no LoRA tensors found (expected ...layers.N.<block>.<proj>.lora_A.weight)")
    return ad


def load_lora(path: str) -> LoraAdapter:
    """Reads a PEFT adapter directory (or its safetensors file, with the config beside it)."""
    from safetensors import safe_open

    d = path if os.path.isdir(path) else os.path.dirname(path)
    cfg_path = os.path.join(d, "adapter_config.json")
    with open(cfg_path) as f:
        cfg = json.load(f)
    r = int(cfg["r"])
    alpha = float(cfg.get("lora_alpha", r))
    file = path if os.path.isfile(path) else os.path.join(d, "adapter_model.safetensors")
    tensors = {}
    with safe_open(file, framework="pt") as sf:
        for k in sf.keys():
            tensors[k] = sf.get_tensor(k)
    return adapter_from_tensors(tensors, r, alpha)


def _row_ranges(mw: ModelWeights) -> Dict[str, Tuple[str, int, int]]:
    """projection -> (fused linear, first row, end row) for an unsharded model."""
    c = mw.cfg
    hd = c.head_dim
    q, kv, I = c.n_q * hd, c.n_kv * hd, c.intermediate
    return {"q_proj": ("wqkv", 0, q), "k_proj": ("wqkv", q, q + kv), "v_proj": ("wqkv", q + kv, q + 2 * kv),
            "o_proj": ("wo", 0, c.hidden), "gate_proj": ("w_gate_up", 0, I), "up_proj": ("w_gate_up", I, 2 * I),
            "down_proj": ("w_down", 0, c.hidden)}


def merge_lora(mw: ModelWeights, adapter: LoraAdapter, weight: float = 1.0) -> int:
    """Adds `weight * (alpha / r) * B @ A` to every targeted projection; returns how many were changed."""
    if mw.tp_size != 1:
        raise ValueError("adapters are merged into an unsharded model; shard after merging")
    ranges = _row_ranges(mw)
    by_linear: Dict[Tuple[int, str], list] = {}
    for (il, proj), (A, B) in adapter.pairs.items():
        if il >= len(mw.layers) or mw.layers[il] is None:
            raise ValueError(f"adapter names layer {il}; the model holds {len(mw.layers)}")
        name, r0, r1 = ranges[proj]
        lin: Optional[Linear] = getattr(mw.layers[il], name)
        if lin is None:
            raise ValueError(f"layer {il} has no dense {proj} (mixture-of-experts layers take no adapter here)")
        if B.shape[0] != r1 - r0 or A.shape[1] != lin.n_in:
            raise ValueError(f"layer {il} {proj}: adapter is {B.shape[0]} x {A.shape[1]}, the model {r1 - r0} x {lin.n_in}")
        by_linear.setdefault((il, name), []).append((r0, r1, A, B))
    for (il, name), parts in by_linear.items():
        lin = getattr(mw.layers[il], name)
        if lin.kind == "gguf":
            raise ValueError("GGUF block weights take no merged adapter; load the bf16 or fp8 checkpoint")
        dev = lin.weight.device if lin.kind == "bf16" else lin.weight.data.device
        full = dequant_linear(lin)
        for r0, r1, A, B in parts:
            full[r0:r1] += (weight * adapter.scale) * (B.to(dev) @ A.to(dev))
        setattr(mw.layers[il], name, make_linear(full, lin.kind, lin.bias))
    return len(adapter.pairs)


class AdapterSet:
    """The adapters of a loaded model, changed in place without a reload (`POST /api/layers/swap`).

    `apply(wanted)` takes the set the model should end up with (path -> weight).  Every projection an old or a
    new adapter touches is rebuilt as base + the sum of the wanted adapters and copied INTO the tensors the
    model already uses, so captured graphs, fused layers and workspaces keep pointing at valid weights.  The
    base of a projection is kept on the host from the first time an adapter touches it (what was merged at
    load counts as base), which makes a detach exact: the bytes return, not an approximation of them."""

    def __init__(self, mw: ModelWeights):
        if mw.tp_size != 1:
            raise ValueError("adapters are swapped on an unsharded model")
        self.mw = mw
        self.base: Dict[Tuple[int, str], Linear] = {}       # host copies, as stored
        self.active: Dict[str, Tuple[LoraAdapter, float]] = {}

    @staticmethod
    def _host_copy(lin: Linear) -> Linear:
        if lin.kind == "bf16":
            return Linear("bf16", lin.weight.detach().to("cpu", copy=True), lin.bias, lin.n_out, lin.n_in)
        w = lin.weight
        return Linear(lin.kind, type(w)(w.data.detach().to("cpu", copy=True), w.scale.detach().to("cpu", copy=True)),
                      lin.bias, lin.n_out, lin.n_in)

    @staticmethod
    def _write(dst: Linear, src: Linear):
        if dst.kind == "bf16":
            dst.weight.copy_(src.weight.to(dst.weight.device))
        else:
            dst.weight.data.copy_(src.weight.data.to(dst.weight.data.device))
            dst.weight.scale.copy_(src.weight.scale.to(dst.weight.scale.device))

    def _targets(self, adapter: LoraAdapter, ranges) -> Dict[Tuple[int, str], list]:
        out: Dict[Tuple[int, str], list] = {}
        for (il, proj), (A, B) in adapter.pairs.items():
            if il >= len(self.mw.layers) or self.mw.layers[il] is None:
                raise ValueError(f"adapter names layer {il}; the model holds {len(self.mw.layers)}")
            name, r0, r1 = ranges[proj]
            lin = getattr(self.mw.layers[il], name)
            if lin is None:
                raise ValueError(f"layer {il} has no dense {proj} (mixture-of-experts layers take no adapter here)")
            if lin.kind == "gguf":
                raise ValueError("GGUF block weights take no merged adapter; load the bf16 or fp8 checkpoint")
            if B.shape[0] != r1 - r0 or A.shape[1] != lin.n_in:
                raise ValueError(f"layer {il} {proj}: adapter is {B.shape[0]} x {A.shape[1]}, the model {r1 - r0} x {lin.n_in}")
            out.setdefault((il, name), []).append((r0, r1, A, B))
        return out

    def apply(self, wanted: Dict[str, float], loader=load_lora) -> dict:
        ranges = _row_ranges(self.mw)
        new_active: Dict[str, Tuple[LoraAdapter, float]] = {}
        for path, wt in wanted.items():
            old = self.active.get(path)
            new_active[path] = (old[0] if old is not None else loader(path), float(wt))
        # everything is checked before anything is written
        plans = {path: self._targets(ad, ranges) for path, (ad, _w) in new_active.items()}
        touched = set()
        for path, (ad, _w) in self.active.items():
            touched |= set(self._targets(ad, ranges))
        for t in plans.values():
            touched |= set(t)
        for key in touched:
            il, name = key
            lin = getattr(self.mw.layers[il], name)
            if key not in self.base:
                self.base[key] = self._host_copy(lin)
            base = self.base[key]
            parts = [(r0, r1, A, B, w * ad.scale) for path, (ad, w) in new_active.items()
                     for (r0, r1, A, B) in plans[path].get(key, [])]
            if not parts:
                self._write(lin, base)                  # no adapter left on it: the stored bytes come back
                continue
            dev = lin.weight.device if lin.kind == "bf16" else lin.weight.data.device
            full = dequant_linear(base).to(dev)
            for r0, r1, A, B, sc in parts:
                full[r0:r1] += sc * (B.to(dev) @ A.to(dev))
            self._write(lin, make_linear(full, lin.kind, lin.bias))
        report = {"attached": sorted(set(new_active) - set(self.active)), "detached": sorted(set(self.active) - set(new_active)),
                  "kept": sorted(set(new_active) & set(self.active)), "projections": len(touched)}
        self.active = new_active
        return report
