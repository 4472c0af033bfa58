"""Sampling randomness as a function of (seed, position), so a generation can be resumed elsewhere.

When a node dies in the middle of an answer the router can send `prompt + tokens already emitted` with the
same seed to another node; the client sees a pause and the cost is one prefill.  That reproduces the
answer only if the draw for token N depends on the seed and N and nothing else.  A sequential generator
carries history (how many draws came before), and under continuous batching or speculation that history
is not a fixed number per token.  Here the uniform for position N is a hash of (seed, N): no state to
advance, so a resumed request, a request that lost its speculative rows, and a request decoded in another
batch all land on the same stream (reference: `src/distributed/replay.rs:1-41`, `:44-78`).

The engine draws one uniform per sampled token (`ops/sampling.py`: the device sampler takes one per row), so
`PositionRng` offers exactly that plus the get / set of its position that speculative verification uses to
give back the draws of rejected rows.  Samplers that need several draws for one token use `uniform_at`
with a draw index.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

_M = (1 << 64) - 1


def _mix(seed: int, position: int, draw: int = 0) -> int:
    """SplitMix64's finaliser over a combination of the three inputs.  Mixed, not added: `seed + position`
    would give two requests whose seeds differ by one the same draws at shifted positions."""
    z = (seed + 0x9E3779B97F4A7C15 + position * 0xBF58476D1CE4E5B9 + draw * 0xD6E8FEB86659FD93) & _M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


def uniform_at(seed: int, position: int, draw: int = 0) -> float:
    """In [0, 1), 53 bits, a pure function of its arguments."""
    return (_mix(seed & _M, position, draw) >> 11) * (1.0 / (1 << 53))


class PositionRng:
    """The generator of one request.  `random()` is the uniform of the current position and moves on by one;
    the state is the position alone."""

    __slots__ = ("seed", "position")

    def __init__(self, seed: int, position: int = 0):
        self.seed = int(seed) & _M
        self.position = int(position)

    def random(self) -> float:
        u = uniform_at(self.seed, self.position)
        self.position += 1
        return u

    def getstate(self) -> int:
        return self.position

    def setstate(self, position: int):
        self.position = int(position)


def _names_nothing(digest: str) -> bool:
    """Empty, or all zeros under any prefix: what a catalogue writes when it has no hash of the bytes (a
    directory of shards has no single file hash).  Neither is evidence that two nodes hold the same weights."""
    h = (digest or "").split(":", 1)[-1].strip()
    return not h or set(h) == {"0"}


@dataclass
class ResumePoint:
    """Where a resumed generation picks up: the emitted tokens are replayed as prompt, sampling goes on at
    the position they ended on."""
    seed: int
    prompt: List[int]
    emitted: List[int] = field(default_factory=list)
    weights_digest: str = ""

    @property
    def tokens(self) -> List[int]:
        return list(self.prompt) + list(self.emitted)

    @property
    def position(self) -> int:
        return len(self.emitted)

    def may_resume_on(self, node_digest: str) -> bool:
        """Only a node that holds the same bytes may continue.  An unknown digest is refused on either side:
        two unrelated checkpoints would otherwise compare equal under a placeholder."""
        return (not _names_nothing(self.weights_digest) and not _names_nothing(node_digest)
                and self.weights_digest == node_digest)

    def to_json(self) -> dict:
        return {"seed": self.seed, "prompt": list(self.prompt), "emitted": list(self.emitted),
                "position": self.position, "weights_digest": self.weights_digest}

    @staticmethod
    def from_json(d: dict) -> "ResumePoint":
        return ResumePoint(int(d["seed"]), list(d["prompt"]), list(d.get("emitted", [])), str(d.get("weights_digest", "")))


def path_fingerprint(path: str, sample: int = 1 << 20, probes: int = 32, probe_bytes: int = 64 << 10) -> str:
    """Identity of a model file or checkpoint directory without reading all of it: sha256 over, per file, its
    name, its size, its first and last `sample` bytes (a GGUF's header and tensor table sit at the front,
    safetensors headers too) and `probes` evenly spaced pieces of its body, so a fine-tune that kept the
    shapes and the embedding table still differs.  Prefixed `fp256:`: a fingerprint, not a hash of the whole
    content."""
    import hashlib
    import os

    if os.path.isdir(path):
        files = sorted(f for f in os.listdir(path)
                       if f.endswith((".safetensors", ".gguf", ".json")) and os.path.isfile(os.path.join(path, f)))
        files = [os.path.join(path, f) for f in files]
    else:
        files = [path]
    if not files:
        return ""
    h = hashlib.sha256()
    for f in files:
        size = os.path.getsize(f)
        h.update(os.path.basename(f).encode() + b"\0" + str(size).encode() + b"\0")
        with open(f, "rb") as fh:
            h.update(fh.read(sample))
            if size > 2 * sample:
                body = size - 2 * sample
                for i in range(probes if body > probes * probe_bytes else 0):
                    fh.seek(sample + (body - probe_bytes) * i // max(1, probes - 1))
                    h.update(fh.read(probe_bytes))
                fh.seek(size - sample)
                h.update(fh.read(sample))
    return "fp256:" + h.hexdigest()
