"""Model stores and the catalogue over them.

Three layouts, as the reference reads them (`docs/MODELS.md:5-9`, `docs/CONFIGURATION.md:27-58`,
`src/inference/load/{ollama_manager,huggingface_manager,model_dirs}.rs`):

  Ollama        `manifests/<registry>/<namespace>/<name>/<tag>` (JSON: layers with mediaType, digest,
                size) and `blobs/sha256-<hex>`; the model layer is a GGUF, beside it the template,
                system prompt, parameters and licence layers.  Named `name:tag`.
  Hugging Face  the hub cache: `models--<owner>--<repo>/snapshots/<revision>/...` (+ `refs/main`),
                under the store or its `hub/`.  Named `owner/repo`.
  bare GGUF     a `.gguf` at the root of a Hugging Face store (or its `hub/`), named by its file name
                with or without the extension.

Each store key is a list of directories on possibly several disks; together they form one
catalogue: a model held by several directories is listed once and read from the first in the
list; a pull lands on the directory that already holds the model when it has room, else on the
first with room; a manifest and its blobs stay in one directory; a delete removes every copy.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

MT_MODEL = "application/vnd.ollama.image.model"
MT_TEMPLATE = "application/vnd.ollama.image.template"
MT_SYSTEM = "application/vnd.ollama.image.system"
MT_PARAMS = "application/vnd.ollama.image.params"
MT_LICENSE = "application/vnd.ollama.image.license"
MT_ADAPTER = "application/vnd.ollama.image.adapter"
MT_PROJECTOR = "application/vnd.ollama.image.projector"
DEFAULT_REGISTRY = "registry.ollama.ai"


@dataclass
class ModelEntry:
    name: str                    # `name:tag`, `owner/repo` or a file name
    source: str                  # ollama | huggingface | gguf
    path: str                    # the GGUF file, or the snapshot directory of a checkpoint
    store: str                   # the store directory that holds it
    size: int = 0
    digest: str = ""
    template: Optional[str] = None
    system: Optional[str] = None
    params: Dict[str, object] = field(default_factory=dict)
    license: Optional[str] = None
    adapters: List[str] = field(default_factory=list)
    projector: Optional[str] = None
    modified: float = 0.0


def _as_list(v) -> List[str]:
    if v is None:
        return []
    if isinstance(v, str):
        return [os.path.expanduser(v)]
    return [os.path.expanduser(str(x)) for x in v]


def split_ollama_name(name: str) -> Tuple[str, str, str, str]:
    """`[registry/][namespace/]name[:tag]` -> (registry, namespace, name, tag)."""
    tag = "latest"
    last = name.rsplit("/", 1)[-1]
    if ":" in last:
        name, tag = name.rsplit(":", 1)
    parts = name.split("/")
    if len(parts) == 1:
        return DEFAULT_REGISTRY, "library", parts[0], tag
    if len(parts) == 2:
        return DEFAULT_REGISTRY, parts[0], parts[1], tag
    return parts[0], "/".join(parts[1:-1]), parts[-1], tag


def blob_path(store: str, digest: str) -> str:
    return os.path.join(store, "blobs", digest.replace(":", "-"))


def sha256_file(path: str, chunk: int = 8 << 20) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return "sha256:" + h.hexdigest()


def free_bytes(path: str) -> int:
    p = path
    while p and not os.path.exists(p):
        p = os.path.dirname(p)
    try:
        st = os.statvfs(p or "/")
        return st.f_bavail * st.f_frsize
    except OSError:
        return 0


class OllamaStore:
    def __init__(self, dirs):
        self.dirs = _as_list(dirs)

    def manifest_path(self, store: str, name: str) -> str:
        reg, ns, nm, tag = split_ollama_name(name)
        return os.path.join(store, "manifests", reg, ns, nm, tag)

    @staticmethod
    def short_name(reg: str, ns: str, nm: str, tag: str) -> str:
        base = nm if (reg == DEFAULT_REGISTRY and ns == "library") else (
            f"{ns}/{nm}" if reg == DEFAULT_REGISTRY else f"{reg}/{ns}/{nm}")
        return f"{base}:{tag}"

    def _read_entry(self, store: str, mpath: str, name: str) -> Optional[ModelEntry]:
        try:
            man = json.load(open(mpath))
        except Exception:
            return None
        e = ModelEntry(name, "ollama", "", store, modified=os.path.getmtime(mpath))
        total = 0
        for layer in man.get("layers", []):
            mt, dg = layer.get("mediaType", ""), layer.get("digest", "")
            bp = blob_path(store, dg)
            total += int(layer.get("size", 0))
            if mt == MT_MODEL:
                e.path, e.digest = bp, dg
            elif mt in (MT_TEMPLATE, MT_SYSTEM, MT_LICENSE) and os.path.exists(bp):
                text = open(bp, encoding="utf-8", errors="replace").read()
                setattr(e, {MT_TEMPLATE: "template", MT_SYSTEM: "system", MT_LICENSE: "license"}[mt], text)
            elif mt == MT_PARAMS and os.path.exists(bp):
                try:
                    e.params = json.load(open(bp))
                except Exception:
                    e.params = {}
            elif mt == MT_ADAPTER:
                e.adapters.append(bp)
            elif mt == MT_PROJECTOR:
                e.projector = bp
        e.size = total
        if not e.path or not os.path.exists(e.path):
            return None          # a manifest whose weights blob is missing is not a usable model
        return e

    def list(self) -> List[ModelEntry]:
        seen: Dict[str, ModelEntry] = {}
        for store in self.dirs:
            root = os.path.join(store, "manifests")
            if not os.path.isdir(root):
                continue
            for d, _dirs, files in os.walk(root):
                for f in files:
                    rel = os.path.relpath(os.path.join(d, f), root).split(os.sep)
                    if len(rel) < 4:
                        continue
                    reg, tag, nm, ns = rel[0], rel[-1], rel[-2], "/".join(rel[1:-2])
                    name = self.short_name(reg, ns, nm, tag)
                    if name in seen:
                        continue         # the first directory in the list wins
                    e = self._read_entry(store, os.path.join(d, f), name)
                    if e is not None:
                        seen[name] = e
        return sorted(seen.values(), key=lambda e: e.name)

    def find(self, name: str) -> Optional[ModelEntry]:
        reg, ns, nm, tag = split_ollama_name(name)
        for store in self.dirs:
            mp = os.path.join(store, "manifests", reg, ns, nm, tag)
            if os.path.isfile(mp):
                e = self._read_entry(store, mp, self.short_name(reg, ns, nm, tag))
                if e is not None:
                    return e
        return None

    # ---- writing ----
    def write_blob(self, store: str, data_or_path, digest: Optional[str] = None) -> Tuple[str, int]:
        """Stores bytes (or moves a finished file) under its sha256; returns (digest, size)."""
        os.makedirs(os.path.join(store, "blobs"), exist_ok=True)
        if isinstance(data_or_path, (bytes, bytearray)):
            dg = "sha256:" + hashlib.sha256(data_or_path).hexdigest()
            if digest and digest != dg:
                raise ValueError(f"blob digest mismatch: got {dg}, expected {digest}")
            bp = blob_path(store, dg)
            if not os.path.exists(bp):
                tmp = bp + ".partial"
                with open(tmp, "wb") as f:
                    f.write(data_or_path)
                os.replace(tmp, bp)
            return dg, len(data_or_path)
        dg = sha256_file(data_or_path)
        if digest and digest != dg:
            raise ValueError(f"blob digest mismatch: got {dg}, expected {digest}")
        bp = blob_path(store, dg)
        size = os.path.getsize(data_or_path)
        if not os.path.exists(bp):
            shutil.move(data_or_path, bp)
        return dg, size

    def create(self, name: str, gguf_path: str, *, template: Optional[str] = None, system: Optional[str] = None,
               params: Optional[dict] = None, license: Optional[str] = None, link: bool = True) -> ModelEntry:
        """A model built here goes to the first directory listed (the one holding every blob it names)."""
        if not self.dirs:
            raise ValueError("no ollama_models_dir is configured")
        store = self.dirs[0]
        os.makedirs(os.path.join(store, "blobs"), exist_ok=True)
        dg = sha256_file(gguf_path)
        bp = blob_path(store, dg)
        if not os.path.exists(bp):
            if link:
                try:
                    os.link(gguf_path, bp)
                except OSError:
                    shutil.copyfile(gguf_path, bp)
            else:
                shutil.copyfile(gguf_path, bp)
        layers = [{"mediaType": MT_MODEL, "digest": dg, "size": os.path.getsize(bp)}]
        for mt, val in ((MT_TEMPLATE, template), (MT_SYSTEM, system), (MT_LICENSE, license),
                        (MT_PARAMS, json.dumps(params) if params else None)):
            if val:
                d2, n2 = self.write_blob(store, val.encode())
                layers.append({"mediaType": mt, "digest": d2, "size": n2})
        mp = self.manifest_path(store, name)
        os.makedirs(os.path.dirname(mp), exist_ok=True)
        with open(mp + ".tmp", "w") as f:
            json.dump({"schemaVersion": 2, "mediaType": "application/vnd.docker.distribution.manifest.v2+json",
                       "layers": layers}, f)
        os.replace(mp + ".tmp", mp)
        return self.find(name)

    def copy(self, source: str, dest: str) -> ModelEntry:
        """A copy stays in the directory of its source, beside the blobs it shares."""
        e = self.find(source)
        if e is None:
            raise FileNotFoundError(source)
        src = self.manifest_path(e.store, source)
        dst = self.manifest_path(e.store, dest)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(src, dst)
        return self.find(dest)

    def delete(self, name: str) -> int:
        """Removes every copy of the manifest, then the blobs no remaining manifest names."""
        n = 0
        for store in self.dirs:
            mp = self.manifest_path(store, name)
            if os.path.isfile(mp):
                os.remove(mp)
                n += 1
                self.prune(store)
        return n

    def prune(self, store: str) -> int:
        used = set()
        root = os.path.join(store, "manifests")
        for d, _dirs, files in os.walk(root):
            for f in files:
                try:
                    for layer in json.load(open(os.path.join(d, f))).get("layers", []):
                        used.add(layer.get("digest", "").replace(":", "-"))
                except Exception:
                    pass
        gone = 0
        bdir = os.path.join(store, "blobs")
        if os.path.isdir(bdir):
            for f in os.listdir(bdir):
                if f.endswith(".partial") or f in used:
                    continue
                os.remove(os.path.join(bdir, f))
                gone += 1
        return gone

    def pull_target(self, name: str, need_bytes: int, have_digests: Iterable[str] = ()) -> str:
        """The directory a pull lands on: the one already holding the model (manifest or blob) when it
        has room for the bytes it lacks, otherwise the first with room for the whole model."""
        have = list(have_digests)
        for store in self.dirs:
            holds = os.path.isfile(self.manifest_path(store, name)) or any(
                os.path.exists(blob_path(store, d)) for d in have)
            if holds:
                lacking = need_bytes - sum(os.path.getsize(blob_path(store, d)) for d in have
                                           if os.path.exists(blob_path(store, d)))
                if free_bytes(store) >= lacking:
                    return store
        for store in self.dirs:
            if free_bytes(store) >= need_bytes:
                return store
        report = ", ".join(f"{s}: {free_bytes(s) >> 20} MiB free" for s in self.dirs)
        raise OSError(f"no model directory has room for {need_bytes >> 20} MiB ({report})")


class HuggingFaceStore:
    def __init__(self, dirs):
        self.dirs = _as_list(dirs)

    def _roots(self) -> List[str]:
        out = []
        for d in self.dirs:
            out.append(d)
            if os.path.isdir(os.path.join(d, "hub")):
                out.append(os.path.join(d, "hub"))
        return out

    @staticmethod
    def _snapshot(repo_dir: str) -> Optional[str]:
        snaps = os.path.join(repo_dir, "snapshots")
        if not os.path.isdir(snaps):
            return None
        ref = os.path.join(repo_dir, "refs", "main")
        if os.path.isfile(ref):
            rev = open(ref).read().strip()
            if os.path.isdir(os.path.join(snaps, rev)):
                return os.path.join(snaps, rev)
        revs = sorted((os.path.getmtime(os.path.join(snaps, r)), r) for r in os.listdir(snaps))
        return os.path.join(snaps, revs[-1][1]) if revs else None

    @staticmethod
    def _dir_size(p: str) -> int:
        n = 0
        for d, _dirs, files in os.walk(p):
            for f in files:
                try:
                    n += os.path.getsize(os.path.join(d, f))     # follows the cache's symlinks into blobs/
                except OSError:
                    pass
        return n

    def list(self) -> List[ModelEntry]:
        seen: Dict[str, ModelEntry] = {}
        for root in self._roots():
            if not os.path.isdir(root):
                continue
            for name in sorted(os.listdir(root)):
                p = os.path.join(root, name)
                if name.startswith("models--") and os.path.isdir(p):
                    repo = name[len("models--"):].replace("--", "/")
                    snap = self._snapshot(p)
                    if snap and repo not in seen and os.path.exists(os.path.join(snap, "config.json")):
                        seen[repo] = ModelEntry(repo, "huggingface", snap, root, self._dir_size(snap),
                                                modified=os.path.getmtime(snap))
                elif name.endswith(".gguf") and os.path.isfile(p):
                    if name not in seen:
                        seen[name] = ModelEntry(name, "gguf", p, root, os.path.getsize(p), modified=os.path.getmtime(p))
        return sorted(seen.values(), key=lambda e: e.name)

    def find(self, name: str) -> Optional[ModelEntry]:
        want = {name, name + ".gguf", name.split(":")[0] + ".gguf"}
        for e in self.list():
            if e.name == name or (e.source == "gguf" and e.name in want):
                return e
        return None

    def delete(self, name: str) -> int:
        n = 0
        for root in self._roots():
            p = os.path.join(root, "models--" + name.replace("/", "--"))
            if os.path.isdir(p):
                shutil.rmtree(p)
                n += 1
            for cand in (name, name + ".gguf"):
                f = os.path.join(root, cand)
                if cand.endswith(".gguf") and os.path.isfile(f):
                    os.remove(f)
                    n += 1
        return n


class Catalogue:
    """The models of every store, under one roof: what listings show and what a load resolves."""

    def __init__(self, ollama_dirs=None, huggingface_dirs=None):
        self.ollama = OllamaStore(ollama_dirs if ollama_dirs is not None else "~/.ollama/models")
        self.hf = HuggingFaceStore(huggingface_dirs if huggingface_dirs is not None else "~/.cache/huggingface/hub")

    def list(self) -> List[ModelEntry]:
        return self.ollama.list() + self.hf.list()

    def resolve(self, name: str) -> Optional[ModelEntry]:
        """`name:tag` looks in the Ollama stores first, `owner/repo` and file names in the Hugging Face
        stores; a path that exists is taken as it is."""
        if os.path.exists(name):
            src = "huggingface" if os.path.isdir(name) else "gguf"
            return ModelEntry(os.path.basename(os.path.normpath(name)), src, name, os.path.dirname(name) or ".",
                              os.path.getsize(name) if os.path.isfile(name) else 0)
        return self.ollama.find(name) or self.hf.find(name)

    def delete(self, name: str) -> int:
        return self.ollama.delete(name) + self.hf.delete(name)
