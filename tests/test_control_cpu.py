"""Control plane on CPU: prefill quantum controller, operation journal (digest + wire format), framed TCP, roster
liveness with a host-made failure (a member that stops sending heartbeats), disk tier (CRC pages, eviction, adoption).
(Model of the reference's tests: tests/test_prefill_latency.cpp, tests/test_fabric_serve.cpp, tests/test_roster.cpp,
tests/test_nvme_tier.cpp, tests/test_disk_cache.cpp.)"""
import threading
import time

import pytest

from dgpp_b200.runtime import rt


# ------------------------------------------------------------------------------------------------ prefill controller
def test_prefill_quantum_starts_at_256_grows_and_shrinks():
    c = rt.PrefillController()
    assert c.quantum() == 256
    assert c.next(decoding=0, waiting_tokens=5000) == 1024            # idle floor: nobody waits on a decode step
    assert c.next(decoding=2, waiting_tokens=5000) == 256
    assert c.next(decoding=2, waiting_tokens=40) == 48                # never more than what is waiting (granule 16)
    assert c.next(decoding=2, waiting_tokens=0) == 0
    for _ in range(6):
        c.observe(tokens=c.quantum(), pass_ms=100.0, decoding=2)      # well under the 1000 ms gap target
    grown = c.quantum()
    assert grown > 256 and grown % 16 == 0
    c.observe(tokens=grown, pass_ms=1500.0, decoding=2)               # overshoot halves it
    assert c.quantum() == max(64, grown // 2 // 16 * 16)
    for _ in range(20):
        c.observe(tokens=c.quantum(), pass_ms=5000.0, decoding=1)
    assert c.quantum() == 64                                          # floor


def test_prefill_first_token_target_raises_the_quantum_but_respects_the_gap_cap():
    c = rt.PrefillController()
    c.observe(tokens=256, pass_ms=64.0, decoding=1)                   # 4 tokens / ms
    base = c.next(decoding=1, waiting_tokens=6000, oldest_wait_ms=0.0)
    late = c.next(decoding=1, waiting_tokens=6000, oldest_wait_ms=2900.0)
    assert late > base                                                # deadline close: ask for more per pass
    assert late <= 4.0 * 1000.0 + 16                                  # at 4 tok/ms a pass may not exceed the gap target
    assert late <= 8192


# ------------------------------------------------------------------------------------------------ journal
def test_journal_replay_digest_and_divergence():
    lead, follow = rt.Journal(), rt.Journal()
    recs = [lead.append("submit", "req-1", [1, 2, 3], 16), lead.append("tick", arg=12345), lead.append("cancel", "req-1")]
    assert [r["seq"] for r in recs] == [0, 1, 2]
    for r in recs:
        follow.replay_line(r["line"])
    assert follow.digest() == lead.digest() and follow.next_seq() == 3
    # a follower that saw different prompt tokens notices at that record
    other = rt.Journal()
    bad = recs[0]["line"].replace("[1,2,3]", "[1,2,4]")
    assert bad != recs[0]["line"]
    with pytest.raises(RuntimeError, match="digest mismatch"):
        other.replay_line(bad)
    # a gap is an error too
    late = rt.Journal()
    with pytest.raises(RuntimeError, match="expected record 0"):
        late.replay_line(recs[1]["line"])
    # catching up after a reconnect
    assert lead.since(1) == [recs[1]["line"], recs[2]["line"]]
    lead.set_keep(2)
    lead.append("tick", arg=1)
    assert lead.since(0) == []                                        # already dropped: the follower must resync


def test_journal_over_framed_tcp():
    lst = rt.Listener()
    lead = rt.Journal()
    lines = [lead.append("submit", f"r{i}", list(range(i, i + 5)), 8)["line"] for i in range(50)]
    got = {}

    def follower():
        s = rt.FramedSocket.connect("127.0.0.1", lst.port())
        j = rt.Journal()
        while j.next_seq() < 50:
            f = s.recv(2000)
            assert f is not None
            j.replay_line(f.decode())
        s.send(str(j.digest()).encode())
        got["digest"] = j.digest()
        s.close()

    t = threading.Thread(target=follower)
    t.start()
    conn = lst.accept(5000)
    assert conn is not None
    for ln in lines:
        assert conn.send(ln.encode())
    echo = conn.recv(5000)
    t.join(10)
    assert int(echo) == lead.digest() == got["digest"]
    conn.close()


def test_framed_socket_timeout_and_peer_close():
    lst = rt.Listener()
    c = rt.FramedSocket.connect("127.0.0.1", lst.port())
    s = lst.accept(2000)
    t0 = time.time()
    assert s.recv(100) is None                                        # nothing sent: a timeout, not a hang
    assert time.time() - t0 < 2.0
    big = bytes(range(256)) * 4096                                    # 1 MiB frame arrives whole
    assert c.send(big) and s.recv(5000) == big
    c.close()
    with pytest.raises(RuntimeError, match="closed"):
        s.recv(1000)


# ------------------------------------------------------------------------------------------------ roster
def test_roster_forms_and_evicts_a_silent_member():
    srv = rt.RosterServer(world=3, deadline_ms=1000)
    clients = [rt.RosterClient("127.0.0.1", srv.port(), r, 3, f"127.0.0.1:{9000 + r}", heartbeat_ms=50) for r in range(3)]
    try:
        assert all(c.wait_complete(5000) for c in clients)
        v = clients[0].view()
        assert v["members"] == {0: "127.0.0.1:9000", 1: "127.0.0.1:9001", 2: "127.0.0.1:9002"}
        e0 = v["epoch"]
        clients[2].freeze()                                           # rank 2 wedges: no heartbeat, no goodbye
        deadline = time.time() + 10
        while time.time() < deadline and 2 in clients[0].view()["members"]:
            time.sleep(0.02)
        v = clients[0].view()
        assert set(v["members"]) == {0, 1} and v["epoch"] > e0 and not v["complete"]
        assert clients[1].view()["members"] == v["members"]
        assert srv.evictions() == 1
        clients[1].stop(True)                                         # an orderly leave is not an eviction
        deadline = time.time() + 5
        while time.time() < deadline and 1 in clients[0].view()["members"]:
            time.sleep(0.02)
        assert set(clients[0].view()["members"]) == {0} and srv.evictions() == 1
    finally:
        for c in clients:
            c.stop(False)
        srv.stop()


def test_roster_client_sees_a_lost_server():
    srv = rt.RosterServer(world=1, deadline_ms=500)
    c = rt.RosterClient("127.0.0.1", srv.port(), 0, 1, "x", heartbeat_ms=20)
    assert c.wait_complete(3000)
    srv.stop()
    del srv
    deadline = time.time() + 5
    while time.time() < deadline and not c.server_lost():
        time.sleep(0.02)
    assert c.server_lost()
    c.stop(False)


# ------------------------------------------------------------------------------------------------ disk tier
def test_disk_tier_roundtrip_multi_page_crc_and_eviction(tmp_path):
    info = rt.probe_cache_storage(str(tmp_path))
    assert info["exists"] and info["writable"] and info["free_bytes"] > 0
    assert not rt.probe_cache_storage(str(tmp_path / "missing"))["exists"]
    t = rt.DiskTier(str(tmp_path), page_bytes=4096, pages=8)
    per = t.payload_per_page()
    assert per == 4096 - 64
    small, big = b"k" * 100, bytes(i % 251 for i in range(per * 2 + 17))    # 1 page and 3 pages
    assert t.put(1, small) and t.put(2, big)
    assert t.get(1) == small and t.get(2) == big and t.get(3) is None
    assert t.free_pages() == 4 and t.blobs() == 2
    # overwrite frees the old pages
    assert t.put(2, small) and t.free_pages() == 6 and t.get(2) == small
    # a corrupted page is a miss, never wrong bytes
    assert t.corrupt_for_test(1)
    assert t.get(1) is None and not t.contains(1)
    assert t.stats()["crc_failures"] == 1
    # fill up: least recently used blob goes first
    for k in range(10, 17):
        assert t.put(k, bytes([k]) * 10)
    assert t.get(2) == small                                          # touch 2 -> most recent
    assert t.put(99, b"z" * (per + 1))                                # needs 2 pages, slab is full
    assert t.contains(2) and t.contains(99) and not t.contains(10) and not t.contains(11)
    assert t.stats()["evictions"] == 2
    # a blob larger than the slab is refused
    assert not t.put(5, b"x" * (per * 9))


def test_disk_tier_async_commit_and_adoption(tmp_path):
    a = rt.DiskTier(str(tmp_path), page_bytes=4096, pages=16)
    tickets = [a.put_async(k, bytes([k]) * (1000 * k)) for k in range(1, 6)]
    a.wait(tickets[-1])
    d = a.commit_digest()
    a.commit()
    del a
    b = rt.DiskTier(str(tmp_path), page_bytes=4096, pages=16)         # a restarted server adopts the slab
    assert b.blobs() == 5 and b.commit_digest() == d
    for k in range(1, 6):
        assert b.get(k) == bytes([k]) * (1000 * k)
    # same contents written in another order give the same digest (what ranks compare before a commit)
    other = tmp_path / "other"
    other.mkdir()
    c = rt.DiskTier(str(other), page_bytes=4096, pages=16)
    for k in (5, 3, 1, 4, 2):
        c.put(k, bytes([k]) * (1000 * k))
    assert c.commit_digest() == d
    c.put(6, b"x")
    assert c.commit_digest() != d
    # a different geometry does not adopt
    del b
    e = rt.DiskTier(str(tmp_path), page_bytes=8192, pages=8)
    assert e.blobs() == 0
