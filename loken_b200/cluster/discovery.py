"""Finding the other nodes of a cluster without a seed list: UDP multicast announcements.

A node sends a small datagram to an administratively scoped multicast group every few seconds and
listens on the same group.  What it hears is ADDED to the configured `[cluster] peers`; multicast
does not cross routers, so seeds stay necessary across subnets.  Two silent hazards are handled the
way the reference handles them (`src/distributed/discovery.rs:13-27`): an announcement that names
another cluster is ignored (two clusters on one switch must not merge), and a node's own
announcement is filtered by node id, not by address (a machine has several addresses).

The datagram is the reference's own, so its nodes and these can see each other:

    loken1 <TAB> cluster <TAB> node_id <TAB> endpoint        (group 239.255.42.99, port 41999)

It is parsed by hand: it arrives unauthenticated from anyone on the network, so the parser does
nothing but split three bounded fields.
"""
from __future__ import annotations

import socket
import struct
import threading
import time
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

DISCOVERY_GROUP = "239.255.42.99"
DISCOVERY_PORT = 41999
MAGIC = "loken1"
MAX_FIELD = 256
MAX_DATAGRAM = 1024


@dataclass(frozen=True)
class Announcement:
    cluster: str
    node_id: str
    endpoint: str           # where the node's HTTP API can be reached

    def encode(self) -> bytes:
        for f in (self.cluster, self.node_id, self.endpoint):
            if "\t" in f or "\n" in f or len(f) > MAX_FIELD:
                raise ValueError("an announcement field holds a separator or is too long")
        return f"{MAGIC}\t{self.cluster}\t{self.node_id}\t{self.endpoint}".encode()

    @staticmethod
    def decode(data: bytes) -> Optional["Announcement"]:
        if len(data) > MAX_DATAGRAM:
            return None
        try:
            parts = data.decode("utf-8").split("\t")
        except UnicodeDecodeError:
            return None
        if len(parts) != 4 or parts[0] != MAGIC:
            return None
        cluster, node, endpoint = parts[1], parts[2], parts[3]
        if not node or not endpoint or any(len(p) > MAX_FIELD or "\n" in p for p in parts[1:]):
            return None
        return Announcement(cluster, node, endpoint)


def accept(mine: Announcement, heard: Optional[Announcement]) -> bool:
    """Is `heard` a peer of `mine`?  Same cluster, another node."""
    return heard is not None and heard.cluster == mine.cluster and heard.node_id != mine.node_id


class Discovery:
    """Announces `me` and collects the peers it hears.  `on_peer(node_id, endpoint)` is called when a
    node is heard for the first time or under a new endpoint; peers that stay silent for `expire_s`
    fall out of `peers()` (the membership detector has the last word on liveness)."""

    def __init__(self, me: Announcement, *, group: str = DISCOVERY_GROUP, port: int = DISCOVERY_PORT,
                 interval_s: float = 5.0, expire_s: float = 30.0, ttl: int = 1, interface: str = "0.0.0.0",
                 on_peer: Optional[Callable[[str, str], None]] = None, loopback: bool = True):
        self.me, self.group, self.port = me, group, port
        self.interval, self.expire = interval_s, expire_s
        self.on_peer = on_peer
        self._seen: Dict[str, Tuple[str, float]] = {}
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._threads = []
        self.rx = socket.socket(socket.AF_INET, socket.SOCK_DGRAM, socket.IPPROTO_UDP)
        self.rx.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        if hasattr(socket, "SO_REUSEPORT"):
            try:
                self.rx.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEPORT, 1)     # several nodes on one machine
            except OSError:
                pass
        self.rx.bind(("", port))
        mreq = struct.pack("4s4s", socket.inet_aton(group), socket.inet_aton(interface))
        self.rx.setsockopt(socket.IPPROTO_IP, socket.IP_ADD_MEMBERSHIP, mreq)
        self.rx.settimeout(0.5)
        self.tx = socket.socket(socket.AF_INET, socket.SOCK_DGRAM, socket.IPPROTO_UDP)
        self.tx.setsockopt(socket.IPPROTO_IP, socket.IP_MULTICAST_TTL, ttl)       # 1: stay on the segment
        self.tx.setsockopt(socket.IPPROTO_IP, socket.IP_MULTICAST_LOOP, 1 if loopback else 0)
        if interface != "0.0.0.0":
            self.tx.setsockopt(socket.IPPROTO_IP, socket.IP_MULTICAST_IF, socket.inet_aton(interface))

    # ---- the two loops ----
    def announce_once(self):
        try:
            self.tx.sendto(self.me.encode(), (self.group, self.port))
        except OSError:
            pass                                  # no route for multicast right now: try again next round

    def handle(self, data: bytes, now: Optional[float] = None) -> Optional[Announcement]:
        """One received datagram (also the entry point of the tests, which need no socket)."""
        a = Announcement.decode(data)
        if not accept(self.me, a):
            return None
        now = time.monotonic() if now is None else now
        with self._lock:
            old = self._seen.get(a.node_id)
            self._seen[a.node_id] = (a.endpoint, now)
        if (old is None or old[0] != a.endpoint) and self.on_peer is not None:
            self.on_peer(a.node_id, a.endpoint)
        return a

    def _listen(self):
        while not self._stop.is_set():
            try:
                data, _ = self.rx.recvfrom(MAX_DATAGRAM + 1)
            except socket.timeout:
                continue
            except OSError:
                return
            self.handle(data)

    def _announce(self):
        while not self._stop.is_set():
            self.announce_once()
            self._stop.wait(self.interval)

    def start(self) -> "Discovery":
        for fn in (self._listen, self._announce):
            t = threading.Thread(target=fn, daemon=True)
            t.start()
            self._threads.append(t)
        return self

    def stop(self):
        self._stop.set()
        for s in (self.rx, self.tx):
            try:
                s.close()
            except OSError:
                pass

    def peers(self, now: Optional[float] = None) -> Dict[str, str]:
        """node id -> endpoint of every node heard within `expire_s`."""
        now = time.monotonic() if now is None else now
        with self._lock:
            for nid in [n for n, (_, t) in self._seen.items() if now - t > self.expire]:
                del self._seen[nid]
            return {n: ep for n, (ep, _) in self._seen.items()}


def union_with_seeds(seeds, discovered: Dict[str, str]):
    """Discovery adds to the seed list, it never replaces it: the endpoints of both, seeds first."""
    out = list(seeds)
    for ep in discovered.values():
        if ep not in out:
            out.append(ep)
    return out
