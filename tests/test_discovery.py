"""Multicast discovery: the datagram format, the two filters (other cluster, own node), expiry, the
union with the seed list; one round over a real socket when the host lets multicast loop back."""
import socket
import time

import pytest

from loken_b200.cluster.discovery import Announcement, Discovery, accept, union_with_seeds


def test_wire_format_is_three_tab_separated_fields():
    a = Announcement("lab", "node-7", "http://10.0.0.7:11434")
    raw = a.encode()
    assert raw == b"loken1\tlab\tnode-7\thttp://10.0.0.7:11434"
    assert Announcement.decode(raw) == a
    for bad in (b"", b"loken2\ta\tb\tc", b"loken1\ta\tb", b"loken1\ta\tb\tc\td", b"loken1\ta\t\tc", b"\xff\xfe",
                b"loken1\ta\tb\t" + b"x" * 2000):
        assert Announcement.decode(bad) is None
    with pytest.raises(ValueError):
        Announcement("a\tb", "n", "e").encode()


def test_other_clusters_and_own_announcements_are_ignored():
    me = Announcement("prod", "n1", "http://a:1")
    assert accept(me, Announcement("prod", "n2", "http://b:1"))
    assert not accept(me, Announcement("dev", "n2", "http://b:1"))         # two clusters on one switch do not merge
    assert not accept(me, Announcement("prod", "n1", "http://other:1"))    # by node id, not by address
    assert not accept(me, None)


def _disco(me, **kw):
    try:
        return Discovery(me, port=0 or 42917, **kw)
    except OSError as e:
        pytest.skip(f"no multicast socket here: {e}")


def test_handle_records_peers_calls_back_once_and_expires():
    heard = []
    d = _disco(Announcement("c", "me", "http://me:1"), expire_s=10.0, on_peer=lambda n, e: heard.append((n, e)))
    try:
        assert d.handle(Announcement("c", "p1", "http://p1:1").encode(), now=100.0) is not None
        d.handle(Announcement("c", "p1", "http://p1:1").encode(), now=101.0)       # same endpoint: no second call
        d.handle(Announcement("c", "p1", "http://p1:2").encode(), now=102.0)       # it moved
        d.handle(Announcement("x", "p2", "http://p2:1").encode(), now=102.0)       # another cluster
        d.handle(d.me.encode(), now=102.0)                                         # ourselves
        assert heard == [("p1", "http://p1:1"), ("p1", "http://p1:2")]
        assert d.peers(now=105.0) == {"p1": "http://p1:2"}
        assert d.peers(now=120.0) == {}
    finally:
        d.stop()


def test_union_keeps_the_seeds_first():
    assert union_with_seeds(["http://s:1"], {"a": "http://a:1", "b": "http://s:1"}) == ["http://s:1", "http://a:1"]


def test_two_nodes_hear_each_other_over_the_group():
    a = _disco(Announcement("t", "a", "http://a:1"), interval_s=0.1)
    try:
        b = Discovery(Announcement("t", "b", "http://b:1"), port=42917, interval_s=0.1)
    except OSError as e:
        a.stop()
        pytest.skip(f"no second multicast socket: {e}")
    try:
        a.start()
        b.start()
        t0 = time.time()
        while time.time() - t0 < 3.0 and not (a.peers() and b.peers()):
            time.sleep(0.05)
        if not (a.peers() and b.peers()):
            pytest.skip("multicast does not loop back on this host")
        assert a.peers() == {"b": "http://b:1"} and b.peers() == {"a": "http://a:1"}
    finally:
        a.stop()
        b.stop()
