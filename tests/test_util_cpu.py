"""Runtime services on CPU: logger, trace spans, CRC-32C, watchdogs, deployment config, memory plan."""
import json
import time

import pytest

from dgpp_b200.runtime import rt


def test_logger_levels_and_sink():
    lines = []
    rt.set_log_sink(lines.append)
    rt.set_log_level("warn")
    rt.log("info", "sched", "hidden")
    rt.log("error", "sched", "shown")
    rt.set_log_level("debug")
    rt.log("debug", "kv", "now visible")
    rt.set_log_sink(None)
    rt.set_log_level("info")
    assert len(lines) == 2 and "ERROR [sched] shown" in lines[0] and "DEBUG [kv] now visible" in lines[1]


def test_trace_spans_are_json_lines(tmp_path):
    p = tmp_path / "trace.jsonl"
    assert not rt.trace_enabled()
    rt.trace_open(str(p))
    t0 = rt.trace_now_us()
    rt.trace_emit("prefill", t0, 1234, json.dumps({"tokens": 2048}))
    rt.trace_emit("decode_step", t0 + 2000, 77)
    rt.trace_close()
    rows = [json.loads(l) for l in p.read_text().splitlines()]
    assert [r["name"] for r in rows] == ["prefill", "decode_step"]
    assert rows[0]["dur_us"] == 1234 and rows[0]["args"] == {"tokens": 2048} and rows[1]["args"] == {}


def test_crc32c_known_vectors():
    assert rt.crc32c(b"123456789") == 0xE3069283
    assert rt.crc32c(b"") == 0
    assert rt.crc32c(b"6789", rt.crc32c(b"12345")) == 0xE3069283       # incremental


def test_engine_watchdog_fires_only_on_stall_while_busy():
    fired = []
    w = rt.EngineWatchdog(deadline_ms=150, on_stall=fired.append, poll_ms=20)
    time.sleep(0.3)
    assert not w.fired()                  # idle engine: no deadline
    w.set_busy(True)
    for _ in range(5):
        time.sleep(0.06)
        w.progress()
    assert not w.fired()
    time.sleep(0.4)                       # busy and silent
    assert w.fired() and len(fired) == 1 and fired[0] >= 150
    del w


def test_shutdown_watchdog():
    hit = []
    w = rt.ShutdownWatchdog(limit_ms=100, on_timeout=lambda: hit.append(1))
    time.sleep(0.3)
    assert w.timed_out() and hit == [1]
    w2 = rt.ShutdownWatchdog(limit_ms=200, on_timeout=lambda: hit.append(2))
    w2.disarm()
    time.sleep(0.3)
    assert not w2.timed_out() and hit == [1]


def test_cluster_config_validation_and_digest():
    base = {"model": "acme/tiny", "tensor_parallel": 4, "max_concurrency": 16, "kv_dtype": "fp8"}
    text, d1 = rt.parse_cluster_config(json.dumps(base))
    cfg = json.loads(text)
    assert cfg["tensor_parallel"] == 4 and cfg["prefill_chunk"] == 2048 and cfg["prefix_cache"] is True
    _, d2 = rt.parse_cluster_config(json.dumps({**base, "port": 9000, "host": "0.0.0.0", "log_level": "debug"}))
    assert d1 == d2                                   # per-process settings do not change the digest
    _, d3 = rt.parse_cluster_config(json.dumps({**base, "mtp_depth": 2}))
    assert d3 != d1
    for bad, msg in [({**base, "tensor_paralel": 2}, "unknown key"), ({"port": 1}, "'model' is required"),
                     ({**base, "tensor_parallel": 3}, "tensor_parallel"), ({**base, "kv_dtype": "fp4"}, "kv_dtype"),
                     ({**base, "prefill_chunk": 100}, "prefill_chunk")]:
        with pytest.raises(RuntimeError, match=msg):
            rt.parse_cluster_config(json.dumps(bad))


def test_kv_memory_plan():
    gib = 1 << 30
    blocks, nbytes, tokens = rt.plan_kv(170 * gib, 4 * gib, 8 * gib, 64, 8, 128, 64, True)
    per_block = 64 * 2 * 8 * 64 * (128 + 4)
    assert blocks == (158 * gib) // per_block and nbytes == blocks * per_block and tokens == blocks * 64
    assert rt.plan_kv(2 * gib, 4 * gib, 0, 64, 8, 128, 64) == (0, 0, 0)
    assert rt.plan_kv(170 * gib, 0, 0, 64, 8, 128, 64, True, 1000)[0] == 1000


def test_engine_options_are_config_keys_covered_by_the_digest():
    """Switches that change what the engine computes are `engine_*` keys of the deployment configuration: the
    digest that ranks compare moves with each of them, unknown values are refused, and EngineOptions reads them."""
    from dgpp_b200.engine.options import EngineOptions

    base = {"model": "tiny"}
    text, d0 = rt.parse_cluster_config(json.dumps(base))
    cfg = json.loads(text)
    assert cfg["engine_fp4_splits"] == "auto" and cfg["engine_layer_kernel"] is False
    seen = {d0}
    for k, v in (("engine_decode_splits", 4), ("engine_fuse_combine", False), ("engine_l2_prefetch", True),
                 ("engine_fp4_splits", "resident"), ("engine_cluster_splitk", True), ("engine_fp4_preload", False),
                 ("engine_layer_kernel", True), ("engine_seq_parallel", False), ("engine_moe_prefill_terms", 1),
                 ("engine_mtp_depth", 2), ("engine_pin_split_rows", True)):
        t, d = rt.parse_cluster_config(json.dumps({**base, k: v}))
        assert d not in seen, k
        seen.add(d)
        o = EngineOptions.from_config(json.loads(t))
        assert getattr(o, k[len("engine_"):]) == v
    for bad in ({"engine_fp4_splits": "fast"}, {"engine_decode_splits": -1}, {"engine_unknown": 1}, {"engine_mtp_depth": 4},
                {"engine_moe_prefill_terms": 0}):
        with pytest.raises(Exception):
            rt.parse_cluster_config(json.dumps({**base, **bad}))


def test_process_memory_file_residency_and_prefill_progress(tmp_path):
    from dgpp_b200.runtime import rt

    pm = rt.process_memory()
    assert pm["rss_bytes"] > 1 << 20 and pm["peak_rss_bytes"] >= pm["rss_bytes"] and pm["memlock_limit_bytes"] != 0
    f = tmp_path / "w.bin"
    f.write_bytes(b"x" * (1 << 20))
    frac, size = rt.file_residency(str(f))
    assert size == 1 << 20 and 0.0 <= frac <= 1.0
    assert rt.file_residency(str(tmp_path / "missing"))[0] == -1.0
    p = rt.PrefillProgress()
    p.begin("a", 1000, 0)
    p.begin("b", 50, 10)
    p.advance("a", 256, 40)
    p.advance("a", 100, 90)                 # a smaller count is not an advance
    rows = {r[0]: r for r in p.snapshot(100)}
    assert rows["a"][1:] == (256, 1000, 0, 60) and rows["b"][1:] == (0, 50, 10, 90)
    assert p.most_stalled(100)[0] == "b"
    p.end("b")
    assert p.most_stalled(100)[0] == "a" and len(p.snapshot(100)) == 1
