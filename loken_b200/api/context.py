"""Server-wide state handed to every route module, and the one helper through which every dialect
runs a generation (gate slot, metrics, cancellation on disconnect)."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Iterator, List, Optional

from ..engine.llm import LLM, GenerationParams, StreamEvent
from ..utils.metrics import Metrics
from .common import ApiError, Auth, ModelRegistry, RateLimiter, RequestGate

VERSION = "0.1.0"


def _ask_prefix(peer: str, model_id: str, ids: List[int], cache_salt=None) -> int:
    import requests

    r = requests.post(peer.rstrip("/") + "/api/cluster/prefix",
                      json={"model": model_id, "prompt": list(ids), "cache_salt": cache_salt}, timeout=2.0)
    r.raise_for_status()
    return int(r.json().get("cached_tokens", 0))


def _fetch_prefill(peer: str, model_id: str, ids: List[int], timeout_s: float) -> bytes:
    import requests

    r = requests.post(peer.rstrip("/") + "/api/cluster/prefill", json={"model": model_id, "prompt_ids": list(ids)},
                      timeout=timeout_s)
    r.raise_for_status()
    return r.content


@dataclass
class ServerSettings:
    host: str = "127.0.0.1"
    port: int = 11434
    api_keys: List[str] = field(default_factory=list)
    require_auth: bool = False
    allowed_origins: List[str] = field(default_factory=list)
    rate_limit_rps: float = 0.0
    rate_limit_burst: int = 0
    max_body_bytes: int = 64 << 20
    request_timeout_s: float = 600.0
    gate_slots: int = 256
    gate_queue: int = 1024
    prefill_peer: Optional[str] = None      # base URL of a node that reads long prompts for this one
    prefill_peer_min_tokens: int = 512
    # requests go to the peer that is predicted to finish them sooner (cluster/routing.py, cluster/forward.py);
    # an answer a peer left unfinished is continued here only when both nodes hold the same bytes, unless
    # `resume_unverified` allows it anyway
    keep_alive_s: float = 300.0             # a model idle this long leaves the device (-1: never); its files stay warm on the host
    route_requests: bool = False
    prefix_ask_min_tokens: int = 512        # prompts at least this long ask the peers how much of them they hold
    resume_unverified: bool = False
    node_id: Optional[str] = None


class ServerContext:
    def __init__(self, registry: ModelRegistry, settings: Optional[ServerSettings] = None):
        self.registry = registry
        self.settings = settings or ServerSettings()
        s = self.settings
        self.auth = Auth(s.api_keys, s.require_auth)
        self.limiter = RateLimiter(s.rate_limit_rps, s.rate_limit_burst)
        self.gate = RequestGate(s.gate_slots, s.gate_queue)
        self.metrics = Metrics()
        self.started = time.time()
        self.inflight = {}
        from ..cluster.handover import HandoverRate

        self.handover = HandoverRate()
        self.fetch_prefill = _fetch_prefill      # replaceable (tests, another transport)
        self.catalogue = None                    # store.catalogue.Catalogue when model stores are configured
        self.opener = None                       # transport of pulls (store.download.Opener); None = requests
        from ..cluster.routing import RateMeter

        from ..place.sleep import SleepRegistry

        self.sleepers = SleepRegistry()          # models whose keep-alive ended: off the device, files warm on the host
        self.asleep = {}                         # model id -> what it was loaded with, for every model the reaper took down
        self.loader = None                       # callable(path, model_id=..., **kw) -> LLM; None = LLM.load
        registry.on_missing = self._wake
        self.rate = RateMeter()                  # this node's decode rate, published by the gossip
        self.prefill_rate = RateMeter()          # and the rate at which it reads prompts
        self.ask_prefix = None                   # callable(addr, model, ids) -> cached tokens on that peer; None = HTTP
        self.layer_cost = {}                     # model -> what a layer costs here (POST /api/cluster/measure), published too
        self.membership = None
        self.router = None                       # cluster.routing.Router once a membership exists and routing is on
        self.open_peer_stream = None             # transport of forwarded requests; None = HTTP (cluster/forward.py)

    # ---- keep-alive: a model that nobody used for a while leaves the device, and comes back when it is named ----
    def reap_idle(self, now: Optional[float] = None) -> List[str]:
        """Takes every model down whose last use is older than the keep-alive and that has no request in flight.
        Its files are kept read into host memory when they fit the host's budget (`place/sleep.py`), so the next
        request that names it loads without touching the disk; otherwise it is simply unloaded.  The last loaded
        model is taken down as well: an idle server holds no device memory.  Returns the ids taken down."""
        ka = self.settings.keep_alive_s
        if ka is None or ka < 0:
            return []
        now = time.time() if now is None else now
        gone = []
        for m in self.registry.list():
            if getattr(m.worker, "tickets", None):
                continue
            last = max(self.registry.last_used.get(m.model_id, 0.0), m.loaded_at)
            if now - last < ka:
                continue
            path, kw = m.path, dict(getattr(m, "load_kwargs", None) or {})
            if not path:
                continue             # random-init weights of a built-in shape: nothing on disk could bring them back
            if not self.registry.drop(m.model_id):
                continue
            rec = self.sleepers.put_to_sleep(m.model_id, path, kw)
            if path:
                self.asleep[m.model_id] = {"path": path, "kwargs": kw, "sleeping": rec is not None}
            self.metrics.count("models_put_to_sleep" if rec is not None else "models_unloaded_idle")
            gone.append(m.model_id)
        return gone

    def _wake(self, name: str):
        """A request names a model the reaper took down: load it again (from warm pages when it sleeps)."""
        if name not in self.asleep and not self.registry.list() and len(self.asleep) == 1:
            name = next(iter(self.asleep))      # the only model this server holds, named loosely or not at all
        info = self.asleep.pop(name, None) if name else None
        if info is None:
            return None
        rec = self.sleepers.wake(name)
        try:
            load = self.loader
            if load is None:
                load = LLM.load
            llm = load(info["path"], model_id=name, **info["kwargs"])
            self.registry.add(llm, default=not self.registry.list())
            self.metrics.count("models_woken")
            return llm
        finally:
            if rec is not None:
                rec.release()

    def _route(self, llm: LLM, ids, params: GenerationParams):
        """The peer that should answer this request, or None for this node."""
        if not self.settings.route_requests or self.membership is None:
            return None
        from ..cluster import forward
        from ..cluster.routing import Router

        if not forward.forwardable(ids, params):
            return None
        if self.router is None or self.router.m is not self.membership:
            self.router = Router(self.membership)
        expected = int(params.max_tokens or 256)
        load = float(len(llm.worker.tickets))
        # a long prompt: who already holds how much of it goes into the estimate (each peer answers for itself)
        prompt_tokens, local_cached, peer_cached = len(ids), 0, {}
        if prompt_tokens >= self.settings.prefix_ask_min_tokens:
            alloc = llm.engine.alloc
            local_cached = len(alloc.match_prefix(list(ids), llm._salt(params))[0]) * alloc.block_size
            for p in self.membership.alive():
                if llm.model_id in p.models and p.tok_per_s > 0:
                    try:
                        peer_cached[p.node_id] = int((self.ask_prefix or _ask_prefix)(p.addr, llm.model_id, list(ids),
                                                                                       params.cache_salt))
                    except Exception:
                        peer_cached[p.node_id] = 0
        try:
            c = self.router.choose(llm.model_id, expected, load, self.rate.rate, local_serves=True,
                                   conversation=params.cache_salt, prompt_tokens=prompt_tokens, local_cached=local_cached,
                                   local_prefill_rate=self.prefill_rate.rate, peer_cached=peer_cached)
        except LookupError:
            return None
        return c if c.addr is not None else None

    def _prefill_on_peer(self, llm: LLM, ids: List[int], params: GenerationParams) -> bool:
        """Disaggregated prefill: a long prompt is read by the configured peer and its cache imported
        here, when the measured hand-over rate beats local prefill (the first long prompt measures
        it).  Any failure falls back to reading the prompt locally."""
        peer = self.settings.prefill_peer
        if hasattr(ids, "embeds"):
            return False             # a prompt given as embedding rows is read here
        if not peer or not self.handover.ask_peer(len(ids), self.settings.prefill_peer_min_tokens):
            return False
        t0 = time.perf_counter()
        try:
            blob = self.fetch_prefill(peer, llm.model_id, ids, self.settings.request_timeout_s)
            salt = llm._salt(params)
            llm.on_engine_thread(lambda eng: eng.import_prefix(blob, salt))
        except Exception:
            self.metrics.count("prefill_peer_failures")
            return False
        self.handover.observe_peer(len(ids), time.perf_counter() - t0)
        self.metrics.count("prefill_peer_handovers")
        return True

    def run(self, llm: LLM, ids: List[int], params: GenerationParams, *, priority: str = "interactive",
            request_id: str = "", scope: Optional[str] = None) -> Iterator[StreamEvent]:
        """Generator of stream events for one request.  Holds a gate slot from the first event to
        the last; closing the generator early (client went away) aborts the request."""
        if len(ids) == 0:
            raise ApiError(400, "the prompt is empty")
        if len(ids) >= llm.engine.max_ctx:
            raise ApiError(400, f"the prompt has {len(ids)} tokens; the context window holds {llm.engine.max_ctx}",
                           code="context_length_exceeded")
        if scope and not params.cache_salt:
            params.cache_salt = "key:" + scope          # per-key prefix-cache scope
        started = self.gate.acquire(priority, timeout=self.settings.request_timeout_s)
        t0 = time.perf_counter()
        first = None
        n_out = 0
        reason = None
        self.inflight[request_id] = {"model": llm.model_id, "prompt_tokens": len(ids), "started": time.time()}
        peer = None
        cached = 0
        try:
            peer = self._route(llm, ids, params)
            if peer is not None:
                from ..cluster import forward

                peered = True
                self.metrics.count("requests_forwarded")
                kw = {"open_stream": self.open_peer_stream} if self.open_peer_stream is not None else {}
                ticket = forward.RemoteTicket(llm, ids, params, peer.addr, on_peer_failed=lambda _a, n=peer.node_id: self._peer_failed(n),
                                              resume_unverified=self.settings.resume_unverified,
                                              timeout_s=self.settings.request_timeout_s, **kw)
            else:
                peered = self._prefill_on_peer(llm, ids, params)
                ticket = llm.submit(ids, params)
            for ev in llm.events_of(ticket, params, self.settings.request_timeout_s):
                if first is None and ev.token_ids:
                    first = time.perf_counter() - t0
                    if not peered and len(ids) >= self.settings.prefill_peer_min_tokens:
                        self.handover.observe_local(len(ids), first)
                n_out += len(ev.token_ids)
                reason = ev.finish_reason or reason
                cached = max(cached, int(ev.cached_tokens or 0))
                yield ev
        finally:
            self.gate.release(started)
            self.inflight.pop(request_id, None)
            total = time.perf_counter() - t0
            if peer is None and first is not None and n_out > 1:
                self.rate.observe(n_out - 1, total - first)         # decode rate of this node: tokens after the first
            if peer is None and first is not None and len(ids) - cached >= 64:
                self.prefill_rate.observe(len(ids) - cached, first)  # and the rate it read this prompt at
            self.metrics.observe_request(llm.model_id, len(ids), n_out, first, total, reason or "disconnect")

    def _peer_failed(self, node_id: str):
        self.metrics.count("requests_taken_back")
        if self.router is not None:
            self.router.failed(node_id)
