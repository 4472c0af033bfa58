"""Per-request figures: queue / prefill / decode times, energy, KV place, prompt-reading progress.

The contract is the reference's (`docs/API.md:448-514`, `src/request_metrics.rs`,
`src/api/request_figures.rs`): a chat answer carries

    "loken": {"queue_ms", "prefill_ms", "decode_ms",
              "energy": {"joules", "gpu_joules", "cpu_joules", "estimated", "share"},
              "kv": {"used_tokens", "capacity_tokens"}}

inside its final usage; a field that is not measured is left out; a stream whose prompt is still
being read after 250 ms reports `: loken-prefill {"done": n, "total": m}` comment lines.

Energy follows the reference's rule: the meter is read at every start and end of a request; each
reading between two of them is split among the requests active over it by the tokens each
computed over it (prompt read and answer generated), evenly when none computed a token.  GPU joules
come from NVML (the total-energy counter where the driver offers it, else integrated power);
CPU package + DRAM joules from RAPL (`/sys/class/powercap`), `null` and `estimated: true` when it is
not readable.  Both readers are injectable, so the accounting is tested without hardware.
"""
from __future__ import annotations

import glob
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


@dataclass
class RequestFigures:
    arrival: float = 0.0
    prefill_start: Optional[float] = None
    first_token: Optional[float] = None
    end: Optional[float] = None
    prompt_done: int = 0           # uncached prompt tokens read so far
    prompt_total: int = 0          # uncached prompt tokens to read
    kv_used: Optional[int] = None
    kv_capacity: Optional[int] = None
    gpu_joules: Optional[float] = None
    cpu_joules: Optional[float] = None
    shared: bool = False           # another request was active at some point of this one
    tokens_since_reading: int = 0  # tokens computed since the last meter reading (ledger's book-keeping)
    accepted_drafts: int = 0
    rejected_drafts: int = 0

    def to_json(self) -> dict:
        """The `loken` object; fields that were not measured are left out."""
        out: dict = {}
        t_start = self.prefill_start if self.prefill_start is not None else self.arrival
        if self.prefill_start is not None:
            out["queue_ms"] = round(max(0.0, self.prefill_start - self.arrival) * 1e3, 3)
        if self.first_token is not None:
            out["prefill_ms"] = round(max(0.0, self.first_token - t_start) * 1e3, 3)
            if self.end is not None:
                out["decode_ms"] = round(max(0.0, self.end - self.first_token) * 1e3, 3)
        if self.gpu_joules is not None or self.cpu_joules is not None:
            e: dict = {"joules": round((self.gpu_joules or 0.0) + (self.cpu_joules or 0.0), 4)}
            if self.gpu_joules is not None:
                e["gpu_joules"] = round(self.gpu_joules, 4)
            e["cpu_joules"] = round(self.cpu_joules, 4) if self.cpu_joules is not None else None
            e["estimated"] = self.cpu_joules is None
            e["share"] = "work" if self.shared else "alone"
            out["energy"] = e
        if self.kv_used is not None and self.kv_capacity is not None:
            out["kv"] = {"used_tokens": int(self.kv_used), "capacity_tokens": int(self.kv_capacity)}
        return out


def sum_figures(parts: List[dict]) -> dict:
    """Figures of an answer that gathers several generations (`n` > 1): times and energy are added,
    `share` is `work` when any part shared, `kv` is the place after the last one."""
    out: dict = {}
    for p in parts:
        for k in ("queue_ms", "prefill_ms", "decode_ms"):
            if k in p:
                out[k] = round(out.get(k, 0.0) + p[k], 3)
        if "energy" in p:
            e = out.setdefault("energy", {"joules": 0.0, "estimated": False, "share": "alone"})
            pe = p["energy"]
            e["joules"] = round(e["joules"] + pe.get("joules", 0.0), 4)
            for k in ("gpu_joules", "cpu_joules"):
                if pe.get(k) is not None:
                    e[k] = round((e.get(k) or 0.0) + pe[k], 4)
                elif k == "cpu_joules":
                    e.setdefault(k, None)
            e["estimated"] = e["estimated"] or bool(pe.get("estimated"))
            if pe.get("share") == "work":
                e["share"] = "work"
        if "kv" in p:
            out["kv"] = p["kv"]
        if p.get("nodes"):                    # a generation a peer answered, or left and this node continued
            out.setdefault("nodes", []).extend(p["nodes"])
        if p.get("taken_back"):
            out["taken_back"] = p["taken_back"]
    return out


def nvml_energy_reader(device_index: int = 0) -> Optional[Callable[[], float]]:
    """Joules since an arbitrary origin from the GPU's total-energy counter, or None."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        pynvml.nvmlDeviceGetTotalEnergyConsumption(h)          # raises where the counter is absent
        return lambda: pynvml.nvmlDeviceGetTotalEnergyConsumption(h) / 1000.0
    except Exception:
        return None


def rapl_energy_reader(root: str = "/sys/class/powercap") -> Optional[Callable[[], float]]:
    """Joules since an arbitrary origin summed over the RAPL package (and DRAM) domains, or None when
    the counters are not readable (containers usually hide them)."""
    files = sorted(glob.glob(f"{root}/intel-rapl:*/energy_uj"))
    try:
        for f in files:
            int(open(f).read())
    except Exception:
        return None
    if not files:
        return None

    def read() -> float:
        return sum(int(open(f).read()) for f in files) / 1e6

    return read


class EnergyLedger:
    """Splits meter readings among the requests that were active between them."""

    def __init__(self, gpu_reader: Optional[Callable[[], float]] = None,
                 cpu_reader: Optional[Callable[[], float]] = None):
        self.gpu, self.cpu = gpu_reader, cpu_reader
        self.lock = threading.Lock()
        self.active: List[RequestFigures] = []
        self.last_gpu: Optional[float] = None
        self.last_cpu: Optional[float] = None

    @classmethod
    def default(cls, device_index: int = 0) -> "EnergyLedger":
        return cls(nvml_energy_reader(device_index), rapl_energy_reader())

    def _reading(self):
        """Reads both meters and books the energy since the previous reading to the active requests."""
        g = self.gpu() if self.gpu else None
        c = self.cpu() if self.cpu else None
        dg = (g - self.last_gpu) if (g is not None and self.last_gpu is not None) else None
        dc = (c - self.last_cpu) if (c is not None and self.last_cpu is not None) else None
        self.last_gpu, self.last_cpu = g, c
        if not self.active:
            return
        tot = sum(f.tokens_since_reading for f in self.active)
        for f in self.active:
            share = (f.tokens_since_reading / tot) if tot > 0 else 1.0 / len(self.active)
            if dg is not None:
                f.gpu_joules = (f.gpu_joules or 0.0) + max(0.0, dg) * share
            if dc is not None:
                f.cpu_joules = (f.cpu_joules or 0.0) + max(0.0, dc) * share
            f.tokens_since_reading = 0

    def open(self, fig: RequestFigures):
        with self.lock:
            self._reading()
            if self.active:
                fig.shared = True
                for f in self.active:
                    f.shared = True
            if self.gpu:
                fig.gpu_joules = 0.0
            if self.cpu:
                fig.cpu_joules = 0.0
            self.active.append(fig)

    def note_tokens(self, fig: RequestFigures, n: int):
        fig.tokens_since_reading += int(n)

    def close(self, fig: RequestFigures):
        with self.lock:
            if fig in self.active:
                self._reading()
                self.active.remove(fig)
