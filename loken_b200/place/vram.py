"""Device-memory authority: the one place that reads GPU memory state and decides what gives way.

What the reference keeps in `src/inference/place/{vram_manager,room,reclaim}.rs`:

  * `probe()`            free / total bytes of a device (injectable; torch.cuda.mem_get_info by default)
  * reclaim registry     components that can give memory back on request (parked KV pools, capture
                         arenas, staging buffers) register a callable; they are asked in priority
                         order, cheapest first, before anything is evicted
  * `ensure_headroom()`  make `need` bytes free: trim the caching allocator's pools first, then the
                         reclaim registry, then evict idle models oldest first; reports what it did
  * `load_admission()`   loads are serialised: one load measures and claims memory at a time
  * `residency_epoch`    bumped whenever something resident was evicted, so a plan made before can tell
                         it is stale

Nothing here changes a device setting; it only reads memory counters and frees this process's own
allocations.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

GiB = 1 << 30


def _torch_probe(device_index: int) -> Tuple[int, int]:
    import torch

    return torch.cuda.mem_get_info(device_index)


def _torch_trim():
    import torch

    if torch.cuda.is_available():
        torch.cuda.empty_cache()


@dataclass
class Reclaimer:
    name: str
    fn: Callable[[int], int]        # asked for `need` bytes, returns the bytes it released
    priority: int = 0               # lower is asked first
    device: Optional[int] = None    # None: any device


@dataclass
class HeadroomReport:
    need: int
    free_before: int
    free_after: int
    trimmed: bool = False
    reclaimed: List[Tuple[str, int]] = field(default_factory=list)
    evicted: List[str] = field(default_factory=list)

    @property
    def ok(self) -> bool:
        return self.free_after >= self.need


class VramAuthority:
    def __init__(self, probe: Optional[Callable[[int], Tuple[int, int]]] = None,
                 trim: Optional[Callable[[], None]] = None, reserve_bytes: int = 1 * GiB):
        self._probe = probe or _torch_probe
        self._trim = trim or _torch_trim
        self.reserve = reserve_bytes         # runtime reserve kept free on every device (contexts, workspaces)
        self._reclaimers: List[Reclaimer] = []
        self._evict_idle: Optional[Callable[[], Optional[str]]] = None
        self._load_lock = threading.Lock()
        self._lock = threading.Lock()
        self.residency_epoch = 0

    # ---- reading ----
    def probe(self, device: int = 0) -> Tuple[int, int]:
        return self._probe(device)

    def free(self, device: int = 0) -> int:
        return max(0, self.probe(device)[0] - self.reserve)

    # ---- registry ----
    def register(self, name: str, fn: Callable[[int], int], priority: int = 0, device: Optional[int] = None):
        with self._lock:
            self._reclaimers = [r for r in self._reclaimers if r.name != name]
            self._reclaimers.append(Reclaimer(name, fn, priority, device))
            self._reclaimers.sort(key=lambda r: r.priority)

    def unregister(self, name: str):
        with self._lock:
            self._reclaimers = [r for r in self._reclaimers if r.name != name]

    def set_evictor(self, evict_idle: Callable[[], Optional[str]]):
        """`evict_idle()` unloads the model that has been idle longest and returns its id, or None."""
        self._evict_idle = evict_idle

    # ---- making room ----
    def ensure_headroom(self, need: int, device: int = 0, allow_evict: bool = True) -> HeadroomReport:
        rep = HeadroomReport(need, self.free(device), 0)
        free = rep.free_before
        if free < need:
            self._trim()                     # cached blocks of the allocator are the cheapest memory there is
            rep.trimmed = True
            free = self.free(device)
        if free < need:
            with self._lock:
                todo = [r for r in self._reclaimers if r.device in (None, device)]
            for r in todo:
                got = 0
                try:
                    got = int(r.fn(need - free) or 0)
                except Exception:
                    got = 0
                if got > 0:
                    rep.reclaimed.append((r.name, got))
                    self._trim()
                    free = self.free(device)
                if free >= need:
                    break
        while free < need and allow_evict and self._evict_idle is not None:
            victim = self._evict_idle()
            if victim is None:
                break
            rep.evicted.append(victim)
            self.residency_epoch += 1
            self._trim()
            free = self.free(device)
        rep.free_after = free
        return rep

    def give_way(self, device: int = 0) -> HeadroomReport:
        """One rung of request-time recovery after an allocation failed: trim the allocator's cache, ask
        every reclaimer once, and if none of that released anything unload ONE idle model (the one
        idle longest).  The caller retries and calls again while the report says something gave way."""
        rep = HeadroomReport(0, self.free(device), 0)
        self._trim()
        rep.trimmed = True
        with self._lock:
            todo = [r for r in self._reclaimers if r.device in (None, device)]
        for r in todo:
            try:
                got = int(r.fn(1 << 62) or 0)
            except Exception:
                got = 0
            if got > 0:
                rep.reclaimed.append((r.name, got))
        if not rep.reclaimed and self._evict_idle is not None:
            victim = self._evict_idle()
            if victim is not None:
                rep.evicted.append(victim)
                self.residency_epoch += 1
        self._trim()
        rep.free_after = self.free(device)
        return rep

    def load_admission(self):
        """Context manager: one load at a time measures memory and claims it."""
        return self._load_lock


_default: Optional[VramAuthority] = None


def authority() -> VramAuthority:
    global _default
    if _default is None:
        _default = VramAuthority()
    return _default


# ---- host memory budget ----------------------------------------------------------------------------
def host_budget_bytes(meminfo_path: str = "/proc/meminfo", cgroup_paths=("/sys/fs/cgroup/memory.max",
                                                                         "/sys/fs/cgroup/memory/memory.limit_in_bytes"),
                      cgroup_usage_paths=("/sys/fs/cgroup/memory.current",
                                          "/sys/fs/cgroup/memory/memory.usage_in_bytes"),
                      headroom: float = 0.25) -> int:
    """Host memory a model may take: what is available minus a quarter as headroom, the process's
    control group taken into account (`layer_executor.rs:9-121` of the reference)."""
    avail = 0
    try:
        for line in open(meminfo_path):
            if line.startswith("MemAvailable:"):
                avail = int(line.split()[1]) * 1024
                break
    except OSError:
        pass
    for lim_p, use_p in zip(cgroup_paths, cgroup_usage_paths):
        try:
            raw = open(lim_p).read().strip()
            if raw and raw != "max":
                limit = int(raw)
                used = int(open(use_p).read().strip())
                if 0 < limit < (1 << 60):
                    avail = min(avail, max(0, limit - used)) if avail else max(0, limit - used)
                break
        except (OSError, ValueError):
            continue
    return int(avail * (1.0 - headroom))
