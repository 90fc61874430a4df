"""Load generator against the fake-engine server: trace shape, streaming measurements, prefix-cache effect."""
from dgpp_b200.bench.load import make_trace, run_load
from dgpp_b200.runtime import rt
from dgpp_b200.serve.app import Server


def test_trace_shapes_are_seeded_and_share_prefixes():
    t1 = make_trace(50, 256, 3, 64, 0.8, 4, 20, seed=5)
    t2 = make_trace(50, 256, 3, 64, 0.8, 4, 20, seed=5)
    assert t1 == t2 and len(t1) == 50
    heads = {tuple(p[:64]) for p in t1 if len(p) >= 68}
    shared = sum(1 for p in t1 if len(p) >= 68)
    assert 1 <= len(heads) <= 3 and 25 <= shared <= 50 and all(max(p) < 256 for p in t1)


def test_load_run_measures_streaming_and_cache_hits():
    tok = rt.Tokenizer.byte_level([], [("<|im_start|>", 256, True), ("<|im_end|>", 257, True)], rt.SplitPattern.Qwen2)
    eng = rt.FakeEngine(slots=4, block_tokens=16, blocks=2048, max_context=4096, vocab=256)
    srv = Server(eng, tok, model_name="fake", eos_ids=[257])
    port = srv.start()
    try:
        trace = make_trace(24, 250, 2, 128, 0.75, 4, 24, seed=1)
        rep = run_load(f"http://127.0.0.1:{port}", trace, concurrency=4, max_tokens=8)
    finally:
        srv.stop()
    assert rep["ok"] == 24 and rep["failed"] == 0 and rep["completion_tokens"] == 24 * 8
    assert rep["prompt_tokens"] == sum(len(p) for p in trace)
    assert rep["cached_tokens"] >= 128 * 8                  # most shared prefixes are served from the block cache
    assert rep["ttft_s"]["p50"] > 0 and rep["completion_tok_s"] > 0 and rep["gap_s"]["p50"] >= 0


def test_suffix_seed_keeps_prefixes_and_changes_the_rest():
    a = make_trace(20, 256, 2, 32, 1.0, 4, 8, seed=3, suffix_seed=10)
    b = make_trace(20, 256, 2, 32, 1.0, 4, 8, seed=3, suffix_seed=11)
    assert {tuple(p[:32]) for p in a} == {tuple(p[:32]) for p in b}
    assert [p[32:] for p in a] != [p[32:] for p in b]


def test_trace_runner_serves_a_child_and_reports_each_concurrency(tmp_path, capsys):
    import json

    from dgpp_b200.bench import trace

    rc = trace.main(["--model", "fake", "--slots", "4", "--port", "8391", "--concurrency", "1,4", "--requests", "10",
                     "--prefix-tokens", "128", "--suffix-tokens", "8,24", "--max-tokens", "6", "--vocab", "250",
                     "--server-log", str(tmp_path / "srv.log"), "--startup-s", "120"])
    assert rc == 0
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert [r["concurrency"] for r in rep["runs"]] == [1, 4]
    assert all(r["ok"] == 10 and r["completion_tokens"] == 60 for r in rep["runs"])
    assert rep["runs"][1]["ttft_prefix_hit_s"]["n"] >= 1      # the second run finds the first run's prefixes resident
