"""Multi-rank serving over the journal on CPU: rank 0 serves HTTP, a follower rank replays the journal into its own
scheduler + engine; both see identical token streams and digests.  A follower with different state stops with a
divergence error; a vanished leader ends the follower with status 3."""
import http.client
import json
import threading

import pytest

from dgpp_b200.runtime import rt
from dgpp_b200.serve.app import Server
from dgpp_b200.serve.world import WorldLeader, run_follower


def _engine():
    return rt.FakeEngine(slots=4, block_tokens=16, blocks=1024, max_context=2048, vocab=256)


def _post(port, body):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
    c.request("POST", "/v1/completions", json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, json.loads(data)


def test_follower_replays_the_leaders_stream():
    leader = WorldLeader(world=2, config_digest=42)
    seen, result = [], {}

    def follow():
        result["rc"] = run_follower(_engine(), "127.0.0.1", leader.port, config_digest=42, on_events=seen.extend)

    t = threading.Thread(target=follow)
    t.start()
    leader.wait_for_followers()
    tok = rt.Tokenizer.byte_level([], [("<|im_start|>", 256, True), ("<|im_end|>", 257, True)], rt.SplitPattern.Qwen2)
    srv = Server(_engine(), tok, model_name="fake", eos_ids=[257], world_leader=leader)
    port = srv.start()
    try:
        texts = []
        for prompt in ("abc", "hello world", "abc"):
            st, j = _post(port, {"model": "fake", "prompt": prompt, "max_tokens": 6})
            assert st == 200
            texts.append(j["choices"][0]["text"])
        assert texts[0] == texts[2]
    finally:
        srv.stop()                      # sends the shutdown record
    t.join(20)
    assert result["rc"] == 0
    # the follower generated the same tokens for the same requests (3 requests x 6 tokens)
    toks = [e for e in seen if e[0] == "token"]
    assert len(toks) == 18
    by_req = {}
    for kind, rid, a, b in toks:
        by_req.setdefault(rid, []).append(a)
    streams = list(by_req.values())
    assert streams[0] == streams[2]
    assert leader.journal.next_seq() > 3 + 18 // 6


def test_configuration_mismatch_and_divergence_are_errors():
    leader = WorldLeader(world=2, config_digest=1, accept_timeout_s=5)
    err = {}

    def follow():
        try:
            run_follower(_engine(), "127.0.0.1", leader.port, config_digest=2)
        except RuntimeError as e:
            err["e"] = str(e)

    t = threading.Thread(target=follow)
    t.start()
    with pytest.raises(RuntimeError, match="different configuration"):
        leader.wait_for_followers()
    t.join(10)
    assert "different configuration" in err["e"]

    # divergence: the follower's scheduler sees a request the leader's did not
    leader = WorldLeader(world=2, config_digest=0)
    sched = rt.Scheduler(_engine(), rt.SchedulerConfig())
    err = {}

    class Skewed(rt.FakeEngine):
        pass

    def follow2():
        try:
            err["rc"] = run_follower(_engine(), "127.0.0.1", leader.port)
        except RuntimeError as e:
            err["e"] = str(e)

    t = threading.Thread(target=follow2)
    t.start()
    leader.wait_for_followers()
    leader.submit(sched, "r1", [1, 2, 3], 4)
    leader.tick(sched)
    # the leader's scheduler advances without telling the follower: the next tick record carries another digest
    sched.submit("ghost", [9, 9, 9], 2)
    sched.tick()
    try:
        leader.tick(sched)
        leader.tick(sched)
    except RuntimeError:
        pass
    t.join(10)
    assert "diverged" in err.get("e", "")


def test_follower_ends_when_the_leader_vanishes():
    leader = WorldLeader(world=2)
    out = {}
    t = threading.Thread(target=lambda: out.setdefault("rc", run_follower(_engine(), "127.0.0.1", leader.port)))
    t.start()
    leader.wait_for_followers()
    for s in leader.followers:
        s.close()                        # no shutdown record: the connection just goes away
    t.join(10)
    assert out["rc"] == 3


def test_follower_rank_metrics_listener():
    from dgpp_b200.serve.world import RankMetrics
    leader = WorldLeader(world=2)
    m = RankMetrics(rank=1)
    out = {}
    t = threading.Thread(target=lambda: out.setdefault("rc", run_follower(_engine(), "127.0.0.1", leader.port, metrics=m)))
    t.start()
    leader.wait_for_followers()
    sched = rt.Scheduler(_engine(), rt.SchedulerConfig())
    leader.submit(sched, "r", [1, 2, 3, 4], 5)
    while not sched.idle():
        leader.tick(sched)
    leader.shutdown()
    t.join(10)
    c = http.client.HTTPConnection("127.0.0.1", m.port, timeout=10)
    c.request("GET", "/metrics/prometheus")
    text = c.getresponse().read().decode()
    c.close()
    m.stop()
    assert out["rc"] == 0
    assert 'dgpp_rank_up{rank="1"} 1' in text and 'dgpp_rank_tokens_total{rank="1"} 5' in text
    assert 'dgpp_rank_submits_total{rank="1"} 1' in text


def test_configure_records_reach_the_follower_before_the_submit():
    leader = WorldLeader(world=2)
    seen = []
    out = {}

    def follow():
        out["rc"] = run_follower(_engine(), "127.0.0.1", leader.port,
                                 on_configure=lambda rid, params, grammar, ids: seen.append((rid, params, grammar, ids)))

    t = threading.Thread(target=follow)
    t.start()
    leader.wait_for_followers()
    sched = rt.Scheduler(_engine(), rt.SchedulerConfig())
    leader.configure("r1", {"temperature": 0.7, "seed": 3}, ["json", "{}"], [5, 6, 7])
    leader.submit(sched, "r1", [5, 6, 7], 3)
    while not sched.idle():
        leader.tick(sched)
    leader.shutdown()
    t.join(10)
    assert out["rc"] == 0
    assert seen == [("r1", {"seed": 3, "temperature": 0.7}, ["json", "{}"], [5, 6, 7])]
