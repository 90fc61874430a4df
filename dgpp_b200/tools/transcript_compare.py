"""Numerics judges for two runs of the same requests: transcript comparison, log-probability comparison and the
cross-rank check.

Input: JSONL files, one record per request: {"id": ..., "tokens": [...], "logprobs": [...]?, "top": [[id, lp], ...]?}
(`logprobs[i]` is the log-probability of `tokens[i]`; `top` the runner-up list of each step, best first).

* transcript: per request the first position where the token streams differ, or "identical".
* near tie: a divergence counts as a near tie when, in the run that has log-probabilities, the margin between the
  two runs' tokens at the first differing position is at most `--tie` nats -- two correct implementations may
  disagree there; any later difference follows from the first and is not judged.
* logprob: over the common prefix, the largest and mean absolute log-probability difference.
* cross-rank (`--ranks a.jsonl b.jsonl c.jsonl ...`): every file must be byte-for-byte the same token streams.

Exit status 0 when every request is identical or diverges only at a near tie (and, with `--max-logprob-delta`, stays
under the bound); 1 otherwise.
(reference counterparts: scripts/fabric_xcript.py, fabric_logprob.py, fabric_xrank.py.)
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, List, Optional


def load(path: str) -> Dict[str, dict]:
    out = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line:
                r = json.loads(line)
                out[str(r["id"])] = r
    return out


def _margin(rec: dict, pos: int, other_token: int) -> Optional[float]:
    """Log-probability gap between this run's token at `pos` and the other run's token, if this run recorded it."""
    lps, top = rec.get("logprobs"), rec.get("top")
    if not lps or pos >= len(lps) or not top or pos >= len(top):
        return None
    for tid, lp in top[pos]:
        if int(tid) == other_token:
            return float(lps[pos]) - float(lp)
    return None


def compare(a: Dict[str, dict], b: Dict[str, dict], tie: float = 0.05) -> List[dict]:
    rows = []
    for rid in sorted(set(a) | set(b)):
        if rid not in a or rid not in b:
            rows.append({"id": rid, "verdict": "missing", "in": "a" if rid in a else "b"})
            continue
        ta, tb = a[rid]["tokens"], b[rid]["tokens"]
        n = min(len(ta), len(tb))
        first = next((i for i in range(n) if ta[i] != tb[i]), None)
        row = {"id": rid, "tokens_a": len(ta), "tokens_b": len(tb)}
        common = n if first is None else first
        la, lb = a[rid].get("logprobs"), b[rid].get("logprobs")
        if la and lb and common:
            d = [abs(float(x) - float(y)) for x, y in zip(la[:common], lb[:common])]
            row["logprob_max_delta"] = max(d)
            row["logprob_mean_delta"] = sum(d) / len(d)
        if first is None:
            row["verdict"] = "identical" if len(ta) == len(tb) else "length"
        else:
            row["first_difference"] = first
            margins = [m for m in (_margin(a[rid], first, tb[first]), _margin(b[rid], first, ta[first])) if m is not None]
            row["margin"] = min(margins) if margins else None
            row["verdict"] = "near_tie" if margins and min(margins) <= tie else "diverged"
        rows.append(row)
    return rows


def cross_rank(paths: List[str]) -> List[dict]:
    runs = [load(p) for p in paths]
    rows = []
    for rid in sorted(set().union(*runs)):
        streams = [r.get(rid, {}).get("tokens") for r in runs]
        same = all(s == streams[0] and s is not None for s in streams)
        row = {"id": rid, "verdict": "identical" if same else "rank_mismatch"}
        if not same:
            row["ranks"] = [i for i, s in enumerate(streams) if s != streams[0]]
        rows.append(row)
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("a", nargs="?")
    ap.add_argument("b", nargs="?")
    ap.add_argument("--ranks", nargs="+", default=[])
    ap.add_argument("--tie", type=float, default=0.05)
    ap.add_argument("--max-logprob-delta", type=float, default=0.0)
    args = ap.parse_args(argv)
    if args.ranks:
        rows = cross_rank(args.ranks)
        bad = [r for r in rows if r["verdict"] != "identical"]
    else:
        if not (args.a and args.b):
            ap.error("two transcript files (or --ranks) are required")
        rows = compare(load(args.a), load(args.b), args.tie)
        bad = [r for r in rows if r["verdict"] not in ("identical", "near_tie") or
               (args.max_logprob_delta and r.get("logprob_max_delta", 0.0) > args.max_logprob_delta)]
    for r in rows:
        print(json.dumps(r))
    print(json.dumps({"requests": len(rows), "failed": len(bad)}))
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
