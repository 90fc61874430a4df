import json

from dgpp_b200.tools import transcript_compare as tc


def _write(path, recs):
    with open(path, "w") as f:
        for r in recs:
            f.write(json.dumps(r) + "\n")
    return str(path)


def test_verdicts(tmp_path):
    a = _write(tmp_path / "a.jsonl", [
        {"id": "same", "tokens": [1, 2, 3], "logprobs": [-0.1, -0.2, -0.3]},
        {"id": "tie", "tokens": [5, 6, 7], "logprobs": [-0.5, -0.7, -0.1], "top": [[[5, -0.5]], [[6, -0.7], [9, -0.72]], [[7, -0.1]]]},
        {"id": "far", "tokens": [5, 6, 7], "logprobs": [-0.5, -0.1, -0.1], "top": [[[5, -0.5]], [[6, -0.1], [9, -3.0]], [[7, -0.1]]]},
        {"id": "only_a", "tokens": [1]}])
    b = _write(tmp_path / "b.jsonl", [
        {"id": "same", "tokens": [1, 2, 3], "logprobs": [-0.1, -0.25, -0.3]},
        {"id": "tie", "tokens": [5, 9, 1]},
        {"id": "far", "tokens": [5, 9, 1]}])
    rows = {r["id"]: r for r in tc.compare(tc.load(a), tc.load(b), tie=0.05)}
    assert rows["same"]["verdict"] == "identical" and abs(rows["same"]["logprob_max_delta"] - 0.05) < 1e-9
    assert rows["tie"]["verdict"] == "near_tie" and rows["tie"]["first_difference"] == 1
    assert rows["far"]["verdict"] == "diverged" and rows["far"]["margin"] > 2
    assert rows["only_a"]["verdict"] == "missing"
    assert tc.main([a, b]) == 1
    assert tc.main([a, a]) == 0
    c = _write(tmp_path / "c.jsonl", [{"id": "same", "tokens": [1, 2, 4]}])
    assert tc.main(["--ranks", a, a]) == 0
    rr = tc.cross_rank([b, c])
    assert [r["verdict"] for r in rr if r["id"] == "same"] == ["rank_mismatch"]
