"""Resumable downloads into the model stores (`loken pull`, `/api/pull`).

A file is fetched to `<target>.partial`; an interrupted fetch resumes with an HTTP Range request
from the bytes already on disk, and the finished file is checked against its sha256 before it
takes its name (`src/download/{mod,http,progress}.rs` of the reference).  The transport is
injectable (`opener(url, headers) -> (status, headers, iterator of chunks)`), so the logic is
tested without a network; the default uses `requests`.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Callable, Dict, Iterable, Iterator, Optional, Tuple

from .catalogue import MT_MODEL, OllamaStore, blob_path, split_ollama_name

Opener = Callable[[str, Dict[str, str]], Tuple[int, Dict[str, str], Iterable[bytes]]]


def requests_opener(url: str, headers: Dict[str, str]):
    import requests

    r = requests.get(url, headers=headers, stream=True, timeout=60)
    return r.status_code, dict(r.headers), r.iter_content(chunk_size=1 << 20)


def fetch(url: str, target: str, *, sha256: Optional[str] = None, opener: Opener = requests_opener,
          headers: Optional[Dict[str, str]] = None, progress: Optional[Callable[[int, Optional[int]], None]] = None
          ) -> int:
    """Downloads `url` to `target`, resuming `target.partial` when it exists.  Returns the bytes
    fetched over the wire in this call."""
    os.makedirs(os.path.dirname(target) or ".", exist_ok=True)
    if os.path.exists(target):
        return 0
    part = target + ".partial"
    have = os.path.getsize(part) if os.path.exists(part) else 0
    h = dict(headers or {})
    if have:
        h["Range"] = f"bytes={have}-"
    status, rh, chunks = opener(url, h)
    if status == 416 and have:                # nothing left to fetch: the partial file is the whole file
        chunks = iter(())
    elif status == 200 and have:              # the server ignored the range: start over
        have = 0
        open(part, "wb").close()
    elif status not in (200, 206):
        raise IOError(f"GET {url} answered {status}")
    total = None
    if "Content-Range" in rh or "content-range" in rh:
        total = int((rh.get("Content-Range") or rh.get("content-range")).rsplit("/", 1)[-1])
    elif rh.get("Content-Length") or rh.get("content-length"):
        total = have + int(rh.get("Content-Length") or rh.get("content-length"))
    got = 0
    with open(part, "ab" if have else "wb") as f:
        for c in chunks:
            f.write(c)
            got += len(c)
            if progress:
                progress(have + got, total)
    if total is not None and have + got != total:
        raise IOError(f"GET {url} ended after {have + got} of {total} bytes (resume by calling again)")
    if sha256:
        d = hashlib.sha256()
        with open(part, "rb") as f:
            for b in iter(lambda: f.read(8 << 20), b""):
                d.update(b)
        if d.hexdigest() != sha256.split(":")[-1]:
            os.remove(part)
            raise IOError(f"{url}: sha256 mismatch, the partial file was discarded")
    os.replace(part, target)
    return got


def pull_ollama(store: OllamaStore, name: str, *, opener: Opener = requests_opener,
                base_url: Optional[str] = None, progress=None) -> Iterator[dict]:
    """Fetches an Ollama tag whole: manifest, then every layer into `blobs/` of the directory the
    pull lands on; yields status records shaped like `/api/pull`'s stream."""
    reg, ns, nm, tag = split_ollama_name(name)
    base = base_url or f"https://{reg}"
    yield {"status": "pulling manifest"}
    status, _h, chunks = opener(f"{base}/v2/{ns}/{nm}/manifests/{tag}",
                                {"Accept": "application/vnd.docker.distribution.manifest.v2+json"})
    if status != 200:
        raise IOError(f"manifest of {name}: HTTP {status}")
    raw = b"".join(chunks)
    man = json.loads(raw)
    layers = man.get("layers", [])
    need = sum(int(l.get("size", 0)) for l in layers)
    target = store.pull_target(name, need, [l["digest"] for l in layers])
    for l in layers:
        dg = l["digest"]
        bp = blob_path(target, dg)
        kind = "model" if l.get("mediaType") == MT_MODEL else "layer"
        yield {"status": f"pulling {dg[7:19]}", "digest": dg, "total": int(l.get("size", 0)), "kind": kind}
        fetch(f"{base}/v2/{ns}/{nm}/blobs/{dg}", bp, sha256=dg, opener=opener,
              progress=(lambda done, total, d=dg: progress(d, done, total)) if progress else None)
    yield {"status": "writing manifest"}
    # a pull that replaces a model held elsewhere removes the other directory's manifest (its blobs stay
    # until a delete prunes them)
    for other in store.dirs:
        mp = store.manifest_path(other, name)
        if other != target and os.path.isfile(mp):
            os.remove(mp)
    mp = store.manifest_path(target, name)
    os.makedirs(os.path.dirname(mp), exist_ok=True)
    with open(mp + ".tmp", "wb") as f:
        f.write(raw)
    os.replace(mp + ".tmp", mp)
    yield {"status": "success"}


def pull_huggingface(hf_dir: str, repo: str, files: Iterable[str], *, revision: str = "main",
                     opener: Opener = requests_opener, base_url: str = "https://huggingface.co",
                     token: Optional[str] = None) -> Iterator[dict]:
    """Fetches the named files of a repository into the hub cache layout (snapshot directory per
    revision, `refs/main`)."""
    repo_dir = os.path.join(hf_dir, "models--" + repo.replace("/", "--"))
    snap = os.path.join(repo_dir, "snapshots", revision)
    os.makedirs(snap, exist_ok=True)
    os.makedirs(os.path.join(repo_dir, "refs"), exist_ok=True)
    headers = {"Authorization": f"Bearer {token}"} if token else {}
    for f in files:
        yield {"status": f"pulling {f}"}
        fetch(f"{base_url}/{repo}/resolve/{revision}/{f}", os.path.join(snap, f), opener=opener, headers=headers)
    with open(os.path.join(repo_dir, "refs", "main"), "w") as fh:
        fh.write(revision)
    yield {"status": "success"}


# ---- a model's draft head without the model ------------------------------------------------------------------
def _read_range(url: str, lo: int, hi: int, opener: Opener, headers: Dict[str, str]) -> bytes:
    """Bytes [lo, hi) of `url`.  A server that ignores the Range header is refused: the point is not to fetch
    a whole shard for a few tensors."""
    status, _rh, chunks = opener(url, dict(headers, Range=f"bytes={lo}-{hi - 1}"))
    if status != 206:
        raise IOError(f"GET {url} with a byte range answered {status}; a ranged read was needed")
    data = b"".join(chunks)
    if len(data) != hi - lo:
        raise IOError(f"GET {url} returned {len(data)} bytes for a range of {hi - lo}")
    return data


def fetch_draft_head(repo: str, output: str, *, revision: str = "main", opener: Opener = requests_opener,
                     base_url: str = "https://huggingface.co", token: Optional[str] = None,
                     prefixes: Tuple[str, ...] = ("mtp.", "model.mtp.")) -> dict:
    """Writes `<output>` (a GGUF companion, `general.type = draft-head`) from the `mtp.*` tensors of a hub
    repository, reading only their bytes: the index names the shards, a ranged read of each shard's
    safetensors header names the offsets, and one ranged read per tensor brings its data
    (reference: `src/inference/load/mtp_head.rs`, `loken draft-head`).  Returns a summary with the bytes read."""
    import struct

    import numpy as np

    from ..formats import gguf as G

    headers = {"Authorization": f"Bearer {token}"} if token else {}
    url = lambda f: f"{base_url}/{repo}/resolve/{revision}/{f}"
    status, _rh, chunks = opener(url("model.safetensors.index.json"), dict(headers))
    if status == 200:
        wm = json.loads(b"".join(chunks))["weight_map"]
        shards = sorted({f for k, f in wm.items() if k.startswith(prefixes)})
        if not shards:
            raise ValueError(f"{repo} names no mtp.* tensors in its index")
    elif status == 404:
        shards = ["model.safetensors"]
    else:
        raise IOError(f"GET {url('model.safetensors.index.json')} answered {status}")
    wire = 0
    tensors = {}
    dt = {"F32": ("<f4", 4), "F16": ("<f2", 2), "BF16": ("<u2", 2)}
    for shard in shards:
        (hl,) = struct.unpack("<Q", _read_range(url(shard), 0, 8, opener, headers))
        if hl <= 0 or hl > (256 << 20):
            raise IOError(f"{shard}: implausible safetensors header length {hl}")
        head = json.loads(_read_range(url(shard), 8, 8 + hl, opener, headers))
        wire += 8 + hl
        for name, meta in head.items():
            if name == "__metadata__" or not name.startswith(prefixes):
                continue
            if meta["dtype"] not in dt:
                raise ValueError(f"{name}: dtype {meta['dtype']} is not read for a draft head")
            lo, hi = meta["data_offsets"]
            raw = _read_range(url(shard), 8 + hl + lo, 8 + hl + hi, opener, headers)
            wire += hi - lo
            ndt, _esz = dt[meta["dtype"]]
            a = np.frombuffer(raw, dtype=ndt).reshape(meta["shape"])
            if meta["dtype"] == "BF16":
                a = (a.astype(np.uint32) << 16).view(np.float32)
            short = name[len("model."):] if name.startswith("model.") else name
            tensors[short[len("mtp."):]] = np.ascontiguousarray(a, dtype=np.float32)
    if not tensors:
        raise ValueError(f"{repo} carries no mtp.* tensors")
    os.makedirs(os.path.dirname(os.path.abspath(output)) or ".", exist_ok=True)
    tmp = output + ".partial"
    w = G.GGUFWriter(tmp)
    w.add_meta("general.type", "draft-head")
    w.add_meta("general.name", f"{repo} (mtp)")
    for k, v in tensors.items():
        w.add_tensor(k, v, G.F32 if v.ndim < 2 else G.BF16)
    w.close()
    os.replace(tmp, output)
    return {"repo": repo, "output": output, "tensors": len(tensors), "shards": len(shards), "bytes_read": wire}
