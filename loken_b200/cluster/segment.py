"""One segment of a pipeline across nodes, backed by a model: layers [lo, hi) with their own paged
cache, driven by the frames of `cluster/pipeline.py`.

`SegmentRunner.run(request_id, hidden[T, H], pos0)` is what a `SegmentServer` calls: the rows are the
residual stream of positions pos0 .. pos0 + T of that request as the previous segment left it.  The
runner grows (or, after a rejected draft or a re-read prompt, trims) the request's cache to pos0,
writes K/V for the new rows, and answers the residual stream after its last layer, or, on the last
segment, the logits of the LAST row (the only one a head samples from).  `cut(request_id, new_len)`
trims a request's cache, `new_len <= 0` drops it.  Requests that stay silent for `idle_s` lose their
cache, so a head that died does not pin a tail's memory.

The reference's tail is `src/inference/serve/pipeline_segment.rs:126-340`; `POST /api/pipeline/tail`
(`api/server.py`) starts one of these on a node and answers the wire port the upstream connects to.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, Optional

import numpy as np
import torch

from ..serve.kv_manager import PagedKvAllocator


class _Req:
    __slots__ = ("seq_id", "last_used")

    def __init__(self, seq_id: int):
        self.seq_id = seq_id
        self.last_used = time.monotonic()


class SegmentRunner:
    def __init__(self, cfg, weights, lo: int, hi: int, *, last: bool, device=None, max_ctx: int = 8192,
                 max_requests: int = 16, max_rows: int = 8192, block_size: int = 16, idle_s: float = 600.0):
        from ..serve.runner import ModelRunner

        self.cfg, self.lo, self.hi, self.last = cfg, lo, hi, last
        self.max_ctx, self.idle_s = max_ctx, idle_s
        blocks = max_requests * ((max_ctx + block_size - 1) // block_size + 1) + 8
        self.alloc = PagedKvAllocator(blocks, block_size, enable_prefix_cache=False)
        self.runner = ModelRunner(cfg, weights, num_blocks=blocks, block_size=block_size, max_seqs=max_requests,
                                  max_tokens=max_rows, max_ctx=max_ctx, use_graphs=False, device=device)
        self.reqs: Dict[int, _Req] = {}
        self.lock = threading.Lock()        # one forward at a time: the runner's staging buffers are shared
        self.rows_done = 0

    # ---- cache bookkeeping ----
    def _reap(self, now: float):
        for rid in [r for r, q in self.reqs.items() if now - q.last_used > self.idle_s]:
            self.cut(rid, 0)

    def cut(self, request_id: int, new_len: int):
        with self.lock:
            q = self.reqs.get(request_id)
            if q is None:
                return
            if new_len <= 0:
                self.alloc.free(q.seq_id)
                del self.reqs[request_id]
            elif new_len < self.alloc.length(q.seq_id):
                self.alloc.trim(q.seq_id, new_len)

    def _prepare(self, request_id: int, pos0: int, T: int) -> _Req:
        if pos0 < 0 or T <= 0 or pos0 + T > self.max_ctx:
            raise ValueError(f"rows {pos0}..{pos0 + T} do not fit this segment's window of {self.max_ctx}")
        now = time.monotonic()
        self._reap(now)
        q = self.reqs.get(request_id)
        if q is None:
            if pos0 != 0:
                raise ValueError(f"request {request_id} is unknown here but its rows start at position {pos0}")
            if len(self.reqs) >= self.runner.max_seqs:
                raise RuntimeError("this segment holds as many requests as it was sized for")
            q = _Req(request_id)
            if not self.alloc.allocate(q.seq_id, T):
                raise MemoryError("no cache blocks left on this segment")
            self.reqs[request_id] = q
        else:
            have = self.alloc.length(q.seq_id)
            if pos0 > have:
                raise ValueError(f"request {request_id}: rows start at {pos0} but the cache ends at {have}")
            if pos0 < have:
                self.alloc.trim(q.seq_id, pos0)       # the head re-sends from an earlier position
            if not self.alloc.append(q.seq_id, T):
                raise MemoryError("no cache blocks left on this segment")
        q.last_used = now
        return q

    # ---- the frame handler ----
    def run(self, request_id: int, hidden: np.ndarray, pos0: int) -> np.ndarray:
        H = self.cfg.hidden
        hidden = np.asarray(hidden)
        if hidden.ndim != 2 or hidden.shape[1] != H:
            raise ValueError(f"expected rows of width {H}, got an array of shape {hidden.shape}")
        T = hidden.shape[0]
        with self.lock:
            q = self._prepare(request_id, int(pos0), T)
            x = torch.from_numpy(np.ascontiguousarray(hidden, dtype=np.float32)).to(self.runner.device).bfloat16()
            out = self.runner.forward_hidden(q.seq_id, x, int(pos0), self.alloc, self.lo, self.hi, self.last)
            self.rows_done += T
            return out.float().cpu().numpy()

    def status(self) -> dict:
        return {"layers": [self.lo, self.hi], "last": self.last, "requests": len(self.reqs), "rows": self.rows_done,
                "free_blocks": self.alloc.free_blocks()}


class PipelineHead:
    """The first segment: embeds the tokens, runs layers [0, cut) on this node and relays the residual
    stream to the following segments over a `SegmentLink`; the last segment's answer is the logits of
    the final row.  One request at a time per call; requests are independent (each has its own cache
    on every segment).  `plan_cut` asks the tail node to start its segment (`POST /api/pipeline/tail`)
    the way the reference's head does (`docs/CLUSTER.md:110-157`)."""

    def __init__(self, cfg, weights, cut: int, link, *, device=None, max_ctx: int = 8192, max_requests: int = 16):
        self.seg = SegmentRunner(cfg, weights, 0, cut, last=False, device=device, max_ctx=max_ctx,
                                 max_requests=max_requests)
        self.cfg, self.w, self.link, self.cut_at = cfg, weights, link, cut

    def forward(self, request_id: int, tokens, pos0: int) -> np.ndarray:
        """Feeds `tokens` at positions pos0.. of the request; returns the logits after the last of them."""
        seg = self.seg
        dev = seg.runner.device
        ids = torch.tensor(list(tokens), dtype=torch.long, device=dev)
        with seg.lock:
            q = seg._prepare(request_id, int(pos0), len(ids))
            from ..models.weights import embed_lookup

            x = (embed_lookup(self.w, ids) * self.cfg.embedding_scale).bfloat16()
            h = seg.runner.forward_hidden(q.seq_id, x, int(pos0), seg.alloc, 0, self.cut_at, False)
            out = h.float().cpu().numpy()
        return np.asarray(self.link.boundary(request_id, out, int(pos0)))

    def generate(self, request_id: int, prompt, max_tokens: int, eos=()) -> list:
        """Greedy decoding through the pipeline (the sampling of a served request lives in the engine;
        this is the segment-level loop the tests and the measuring route use)."""
        logits = self.forward(request_id, prompt, 0)
        out, pos = [], len(prompt)
        for _ in range(max_tokens):
            tok = int(np.argmax(logits.reshape(-1)))
            out.append(tok)
            if tok in eos:
                break
            logits = self.forward(request_id, [tok], pos)
            pos += 1
        self.release(request_id)
        return out

    def release(self, request_id: int):
        self.seg.cut(request_id, 0)
        self.link.cut(request_id, 0)


def plan_cut(tail_url: str, model: str, lo: int, hi: int, post=None, **kw) -> tuple:
    """Asks the node at `tail_url` to run layers [lo, hi) of `model`; returns (host, port) of its wire
    listener."""
    import json
    import urllib.parse
    import urllib.request

    body = dict(kw, model=model, **{"from": lo, "to": hi})
    if post is not None:
        rep = post(tail_url.rstrip("/") + "/api/pipeline/tail", body)
    else:
        req = urllib.request.Request(tail_url.rstrip("/") + "/api/pipeline/tail", data=json.dumps(body).encode(),
                                     headers={"content-type": "application/json"}, method="POST")
        with urllib.request.urlopen(req, timeout=600) as r:
            rep = json.loads(r.read())
    host = urllib.parse.urlparse(tail_url).hostname or "127.0.0.1"
    return host, int(rep["port"])
