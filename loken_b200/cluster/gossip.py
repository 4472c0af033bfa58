"""Gossip over HTTP (`docs/CLUSTER.md:53-63` of the reference: a JSON state poll every gossip
interval): each round this node posts its payload (id, address, models, load, decode rate, free KV
blocks, the peers it believes alive) to every configured and learnt peer's `/api/cluster/gossip`
and folds the answers into its `Membership`.  A peer that stops answering is not removed by hand:
its phi-accrual detector simply stops getting heartbeats and `Membership.alive` drops it.

`post` is injectable (tests drop or delay messages on the host; no GPU is involved).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional

from .membership import Membership


def http_post(url: str, payload: dict, timeout_s: float) -> dict:
    import requests

    r = requests.post(url, json=payload, timeout=timeout_s)
    r.raise_for_status()
    return r.json()


def fold(m: Membership, payload: dict):
    """Takes one node's gossip payload into the membership: the sender is heard from directly, the
    nodes it names are learnt (address only: they have to be heard from themselves to count)."""
    m.observe(payload["id"], payload.get("addr", ""), models=payload.get("models"), load=payload.get("load"),
              tok_per_s=payload.get("tok_per_s"), free_kv_blocks=payload.get("free_kv_blocks"),
              incarnation=int(payload.get("incarnation", 0)), layer_cost=payload.get("layer_cost"),
              card_bytes_free=payload.get("card_bytes_free"), prefill_tok_per_s=payload.get("prefill_tok_per_s"))
    return [k for k in payload.get("known", []) if k.get("id") not in m.peers and k.get("id") != m.self_id]


class GossipLoop:
    def __init__(self, membership: Membership, self_addr: str, seeds: List[str], describe: Callable[[], dict],
                 interval_s: float = 0.5, post: Callable[[str, dict, float], dict] = http_post):
        self.m, self.self_addr, self.describe = membership, self_addr, describe
        self.interval_s, self.post = interval_s, post
        self.addrs: Dict[str, str] = {a: a for a in seeds}       # address -> address (learnt ones are added)
        self.failures: Dict[str, int] = {}
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def payload(self) -> dict:
        d = self.describe()
        return self.m.gossip_payload(self.self_addr, d.get("models", []), d.get("load", 0.0), d.get("tok_per_s", 0.0),
                                     d.get("free_kv_blocks", 0), d.get("layer_cost"), d.get("card_bytes_free", 0),
                                     d.get("prefill_tok_per_s", 0.0))

    def round(self):
        """One gossip round: every known address is told our state and asked for its own."""
        mine = self.payload()
        for addr in list(self.addrs):
            t0 = time.perf_counter()
            try:
                theirs = self.post(addr.rstrip("/") + "/api/cluster/gossip", mine, max(self.interval_s, 0.2))
            except Exception:
                self.failures[addr] = self.failures.get(addr, 0) + 1
                continue
            rtt = (time.perf_counter() - t0) * 1e3
            self.failures[addr] = 0
            for k in fold(self.m, theirs):
                if k.get("addr"):
                    self.addrs.setdefault(k["addr"], k["addr"])
            if theirs.get("id"):
                self.m.timed(theirs["id"], rtt)
        self.m.tick()

    def start(self):
        def run():
            while not self._stop.wait(self.interval_s):
                self.round()

        self._thread = threading.Thread(target=run, name="gossip", daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
