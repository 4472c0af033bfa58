"""Sleeping models: an idle model gives its device memory back while its files stay warm in host RAM.

When a model's keep-alive ends, and its files fit the host memory budget, the reference does not
unload it outright: it keeps the files read into (and where allowed locked in) host memory,
releases the card memory, and the next request loads it from that memory without touching the disk
(`src/inference/place/sleep.rs:1-12`, `docs/MODELS.md`).  A model that does not fit is unloaded; an
unload by name also frees a sleeping model.

Here a `SleepingModel` holds read-only mappings of the model's files, touched page by page so they
sit in the page cache, and `mlock`ed when the process limit allows it (failure to lock is not an
error: the pages are then merely likely to stay).  `SleepRegistry` decides sleep versus unload from
`host_budget_bytes()` and hands the record back on wake.
"""
from __future__ import annotations

import ctypes
import mmap
import os
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

from .vram import host_budget_bytes


def model_files(path: str) -> List[str]:
    """The files a load reads: a GGUF (and the other parts of a split set), or every weight / JSON file
    of a checkpoint directory."""
    if os.path.isdir(path):
        keep = (".safetensors", ".json", ".gguf", ".model", ".txt")
        return sorted(os.path.join(path, f) for f in os.listdir(path) if f.endswith(keep))
    base = os.path.basename(path)
    if "-of-" in base and base.endswith(".gguf"):            # name-00001-of-00003.gguf
        stem = base.rsplit("-", 3)[0]
        d = os.path.dirname(path) or "."
        return sorted(os.path.join(d, f) for f in os.listdir(d) if f.startswith(stem) and f.endswith(".gguf"))
    return [path]


def _mlock(mm: mmap.mmap) -> bool:
    """Locks the mapping's pages in memory when the process limit (RLIMIT_MEMLOCK) allows it."""
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        view = ctypes.c_char.from_buffer(mm)             # a private (copy-on-write) mapping exports a writable buffer
        addr = ctypes.addressof(view)
        del view                                         # the export must be gone before the map can be closed
        return libc.mlock(ctypes.c_void_p(addr), ctypes.c_size_t(len(mm))) == 0
    except Exception:
        return False


@dataclass
class SleepingModel:
    model_id: str
    path: str
    load_kwargs: dict = field(default_factory=dict)
    files: List[str] = field(default_factory=list)
    host_bytes: int = 0
    locked: bool = False
    since: float = 0.0
    _maps: list = field(default_factory=list, repr=False)

    def warm(self, touch: bool = True, lock: bool = True):
        """Maps the files, reads one byte per page so they are resident, and tries to lock them."""
        self.files = model_files(self.path)
        self.host_bytes = 0
        all_locked = bool(self.files)
        for f in self.files:
            size = os.path.getsize(f)
            if size == 0:
                continue
            fd = os.open(f, os.O_RDONLY)
            try:
                mm = mmap.mmap(fd, size, access=mmap.ACCESS_COPY)      # never written: pages stay shared with the page cache
            finally:
                os.close(fd)
            if touch:
                step = mmap.PAGESIZE
                s = 0
                for off in range(0, size, step * 256):          # one read per MiB pulls read-ahead along
                    s += mm[off]
                del s
                try:
                    mm.madvise(mmap.MADV_WILLNEED)
                except (AttributeError, OSError):
                    pass
            all_locked = all_locked and lock and _mlock(mm)
            self._maps.append(mm)
            self.host_bytes += size
        self.locked = all_locked
        self.since = time.time()
        return self

    def release(self):
        for mm in self._maps:
            try:
                mm.close()
            except Exception:
                pass
        self._maps = []


class SleepRegistry:
    """Models that left the device but stay warm on the host."""

    def __init__(self, budget: Optional[Callable[[], int]] = None):
        self.budget = budget or host_budget_bytes
        self.sleeping: Dict[str, SleepingModel] = {}
        self.lock = threading.Lock()

    def bytes_held(self) -> int:
        return sum(m.host_bytes for m in self.sleeping.values())

    def put_to_sleep(self, model_id: str, path: Optional[str], load_kwargs: Optional[dict] = None,
                     touch: bool = True) -> Optional[SleepingModel]:
        """Called when a model's keep-alive ends, after (or instead of) unloading it from the device.
        Returns the record when the model sleeps, None when it is simply unloaded: no files on disk
        (a random-init shape), or files larger than what the host can spare."""
        if not path or not os.path.exists(path):
            return None
        need = sum(os.path.getsize(f) for f in model_files(path))
        with self.lock:
            if need > self.budget():
                return None
            m = SleepingModel(model_id, path, dict(load_kwargs or {})).warm(touch=touch)
            self.sleeping[model_id] = m
            return m

    def wake(self, model_id: str) -> Optional[SleepingModel]:
        """The record of a sleeping model, removed from the registry: the caller loads from `path` (its
        pages are in memory) and then calls `release()` on the record."""
        with self.lock:
            return self.sleeping.pop(model_id, None)

    def drop(self, model_id: str) -> bool:
        """An unload by name also frees a sleeping model."""
        with self.lock:
            m = self.sleeping.pop(model_id, None)
        if m is None:
            return False
        m.release()
        return True

    def make_room(self, need: int) -> List[str]:
        """Frees sleeping models, longest asleep first, until `need` more bytes fit the host budget."""
        gone = []
        with self.lock:
            order = sorted(self.sleeping.values(), key=lambda m: m.since)
            free = self.budget()
            for m in order:
                if free >= need:
                    break
                self.sleeping.pop(m.model_id, None)
                m.release()
                free += m.host_bytes
                gone.append(m.model_id)
        return gone
