"""A request answered by a peer token by token, and taken back when the peer leaves.

When the router predicts that a peer finishes a request sooner (`cluster/routing.py`), the node that
received it keeps the text layer (detokeniser, stop strings, the API dialect, the client's connection) and
asks the peer only for tokens: `POST /api/cluster/generate` streams the peer engine's raw step outputs as
JSON lines.  They are fed into a ticket that looks like a local one, so everything downstream of
`LLM.events_of` is unchanged.

If the peer fails (cannot be reached, answers an error, or its stream ends before the answer does) the
request is taken back: the tokens already received become part of the prompt and generation continues on
this node at the position they ended on.  Because the draw for token N depends on (seed, N) alone
(`serve/replay.py`) the continuation is the stream the peer would have produced; the client sees a pause.
A continuation of a partly sampled answer is refused unless both nodes are known to hold the same bytes
(`ResumePoint.may_resume_on`; reference: `src/distributed/replay.rs:44-78`), or the operator allowed
unverified resumes.  A request that had produced nothing yet simply runs here.

Failures are made on the host in the tests (a transport that raises after k lines); nothing here touches a GPU.
"""
from __future__ import annotations

import dataclasses
import json
import queue
import threading
import time
from typing import Callable, Iterable, Iterator, List, Optional, Tuple

from ..serve.engine import StepOutput
from ..serve.replay import ResumePoint

# sampling fields a peer needs; stop strings, echo and the other text-level options stay with the asking node
WIRE_FIELDS = ("temperature", "top_k", "top_p", "min_p", "repeat_penalty", "repeat_last_n", "max_tokens", "seed",
               "stop_token_ids", "ignore_eos", "logprobs", "top_logprobs", "allowed_token_ids", "bad_words_ids",
               "min_tokens", "context_shift", "num_keep", "resume_position", "cache_salt")


class PeerFailed(RuntimeError):
    pass


def params_to_wire(params) -> dict:
    d = {k: getattr(params, k) for k in WIRE_FIELDS if hasattr(params, k)}
    d["logit_bias"] = {str(k): float(v) for k, v in (params.logit_bias or {}).items()}
    return d


def params_from_wire(d: dict):
    from ..engine.llm import GenerationParams

    kw = {k: d[k] for k in WIRE_FIELDS if k in d and d[k] is not None}
    p = GenerationParams(**kw)
    p.logit_bias = {int(k): float(v) for k, v in (d.get("logit_bias") or {}).items()}
    return p.validate()


def forwardable(ids, params) -> bool:
    """Plain token requests travel; a grammar's matcher state, prompt rows given as embeddings and
    several samples of one prompt stay on the node that holds them."""
    return params.grammar is None and not hasattr(ids, "embeds") and getattr(params, "n", 1) == 1


# ---- the answering side -----------------------------------------------------------------------------------
def serve_raw(llm, ids: List[int], params, *, node_id: str = "", timeout_s: float = 600.0) -> Iterator[bytes]:
    """JSON lines: first {"node", "digest"}, then one line per engine step of the request
    ({"t": tokens, "fin", "reason", "lp", "cached", "fig"}), or {"error"}.  Closing the generator aborts."""
    ticket = llm.submit(ids, params)
    done = False
    try:
        yield (json.dumps({"node": node_id, "digest": getattr(llm, "weights_digest", "") or ""}) + "\n").encode()
        while True:
            try:
                ev = ticket.events.get(timeout=timeout_s)
            except queue.Empty:
                yield (json.dumps({"error": "generation timed out"}) + "\n").encode()
                return
            if isinstance(ev, Exception):
                done = True
                yield (json.dumps({"error": str(ev)}) + "\n").encode()
                return
            line = {"t": [int(t) for t in ev.new_tokens], "fin": bool(ev.finished)}
            if ev.finish_reason:
                line["reason"] = ev.finish_reason
            if ev.logprobs:
                line["lp"] = [[float(lp), [[int(t), float(l)] for t, l in top]] for lp, top in ev.logprobs]
            if ev.finished:
                done = True
                line["cached"] = int(getattr(ev, "cached_tokens", 0) or 0)
                if getattr(ev, "figures", None):
                    line["fig"] = ev.figures
            yield (json.dumps(line) + "\n").encode()
            if ev.finished:
                return
    finally:
        if not done:
            llm.abort(ticket)


def http_stream(peer: str, body: dict, timeout_s: float = 600.0) -> Tuple[Iterable[dict], Callable[[], None]]:
    """The default transport: (lines as dicts, a close function that may be called from another thread)."""
    import requests

    r = requests.post(peer.rstrip("/") + "/api/cluster/generate", json=body, stream=True, timeout=(5.0, timeout_s))
    if r.status_code != 200:
        text = r.text[:200]
        r.close()
        raise PeerFailed(f"the peer answered {r.status_code}: {text}")
    return (json.loads(l) for l in r.iter_lines() if l), r.close


# ---- the asking side ----------------------------------------------------------------------------------------
class RemoteTicket:
    """Stands where a local ticket stands (`events`, `fig`, `prompt_ids`, `params`, `seq_id`) while a thread fills
    `events` from the peer's stream, or from this node's engine after a take-back."""

    def __init__(self, llm, ids: List[int], params, peer: str, *, open_stream=http_stream,
                 on_peer_failed: Optional[Callable[[str], None]] = None, resume_unverified: bool = False,
                 timeout_s: float = 600.0):
        from ..utils.figures import RequestFigures

        if params.seed is None:                 # a seed chosen here is what makes the answer resumable
            import random

            params = dataclasses.replace(params, seed=random.SystemRandom().getrandbits(63))
        self.llm, self.prompt_ids, self.params, self.peer = llm, list(ids), params, peer
        self.salt = 0
        self.events: "queue.Queue" = queue.Queue()
        self.seq_id = None
        self.t0 = time.perf_counter()
        self.on_event = None
        self.fig = RequestFigures(arrival=self.t0)
        self.emitted: List[int] = []
        self.peer_node, self.peer_digest = "", ""
        self.local = None                       # this node's ticket once the request was taken back
        self.taken_back: Optional[str] = None   # why
        self._open, self._failed, self._unverified, self._timeout = open_stream, on_peer_failed, resume_unverified, timeout_s
        self._close: Optional[Callable[[], None]] = None
        self._cancelled = False
        self._lock = threading.Lock()
        self.thread = threading.Thread(target=self._run, daemon=True, name="loken-forward")
        self.thread.start()

    # -- called by LLM.abort (a stop string was hit, the client went away)
    def cancel(self):
        with self._lock:
            self._cancelled = True
            close, local = self._close, self.local
        if local is not None:
            self.llm.abort(local)
        if close is not None:
            try:
                close()
            except Exception:
                pass

    def _run(self):
        body = {"model": self.llm.model_id, "prompt": self.prompt_ids, "params": params_to_wire(self.params)}
        try:
            lines, close = self._open(self.peer, body, self._timeout)
            with self._lock:
                self._close = close
                if self._cancelled:
                    close()
                    return
            for line in lines:
                if "digest" in line and "t" not in line:
                    self.peer_node, self.peer_digest = str(line.get("node", "")), str(line.get("digest", ""))
                    continue
                if line.get("error"):
                    raise PeerFailed(str(line["error"]))
                toks = [int(t) for t in line.get("t", [])]
                lp = [(float(a), [(int(t), float(l)) for t, l in top]) for a, top in line["lp"]] if line.get("lp") else None
                fig = line.get("fig")
                if isinstance(fig, dict):
                    # what a request cost is what every node spent on it: the figures say who answered
                    # (reference: `src/distributed/evidence.rs:1-24`, per-node cost of one request)
                    fig = dict(fig, nodes=[{"node": self.peer_node or self.peer, "role": "answered", "tokens": len(self.emitted) + len(toks)}])
                so = StepOutput(-1, toks, bool(line.get("fin")), line.get("reason"), lp,
                                figures=fig, cached_tokens=int(line.get("cached", 0)))
                self.emitted += toks
                self.events.put(so)
                if so.finished:
                    return
            raise PeerFailed("the peer's stream ended before the answer did")
        except Exception as e:          # transport errors of any kind: the peer is gone as far as this request goes
            if self._cancelled:
                return
            self._take_back(e)

    def _take_back(self, why: Exception):
        self.taken_back = f"{type(why).__name__}: {why}"
        if self._failed is not None:
            try:
                self._failed(self.peer)
            except Exception:
                pass
        p = self.params
        if self.emitted:
            rp = ResumePoint(p.seed, self.prompt_ids, self.emitted, self.peer_digest)
            mine = getattr(self.llm, "weights_digest", "") or ""
            if not (self._unverified or rp.may_resume_on(mine)):
                self.events.put(PeerFailed("the peer left in the middle of the answer and this node is not known to hold "
                                           "the same weights, so the answer cannot be continued here"))
                return
        left = None if p.max_tokens is None else p.max_tokens - len(self.emitted)
        if left is not None and left <= 0:
            self.events.put(StepOutput(-1, [], True, "length"))
            return
        p2 = dataclasses.replace(p, max_tokens=left, resume_position=p.resume_position + len(self.emitted),
                                 min_tokens=max(0, p.min_tokens - len(self.emitted)))
        n_peer = len(self.emitted)

        def relay(ev):
            if not isinstance(ev, Exception):
                self.emitted += list(ev.new_tokens)
            # the last local event carries the figures: they name both nodes and what each wrote
            fig = getattr(ev, "figures", None)
            if isinstance(fig, dict):
                ev.figures = dict(fig, nodes=[{"node": self.peer_node or self.peer, "role": "left", "tokens": n_peer},
                                              {"node": "self", "role": "continued", "tokens": len(self.emitted) - n_peer}],
                                  taken_back=self.taken_back)
            self.events.put(ev)

        with self._lock:
            if self._cancelled:
                return
            try:
                self.local = self.llm.submit(self.prompt_ids + self.emitted, p2, on_event=relay)
            except Exception as e:
                self.events.put(e)
                return
        self.fig = self.local.fig
