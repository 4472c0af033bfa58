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
