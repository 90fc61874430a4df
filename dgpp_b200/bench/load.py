"""HTTP load generator for a running server: a seeded synthetic trace of completion requests at a fixed concurrency,
with optional shared prefixes, streamed so that time-to-first-token and inter-token gaps are measured per request.

    python -m dgpp_b200.bench.load --url http://127.0.0.1:8000 --requests 256 --concurrency 8 \
        --prefixes 4 --prefix-tokens 16384 --shared 0.8 --suffix-tokens 64,512 --max-tokens 128 --vocab 4096

Prompts are token-id arrays (the completions endpoint accepts them as is), so the trace does not depend on a
tokenizer: `shared` of the requests start with one of `prefixes` fixed random prefixes of `prefix-tokens` ids followed
by a unique suffix, the rest are entirely unique.  Output: one JSON object with request counts, wall time, prompt /
completion tokens per second, TTFT and inter-token-gap percentiles, and the server's cached-token total (prefix-cache
effect).  (reference counterparts: scripts/serve_campaign.py, scripts/timed_load.py, scripts/bench_stream.py.)
"""
from __future__ import annotations

import argparse
import http.client
import json
import random
import threading
import time
import urllib.parse
from typing import Dict, List


def make_trace(n: int, vocab: int, prefixes: int, prefix_tokens: int, shared: float, suffix_lo: int, suffix_hi: int,
               seed: int = 0, suffix_seed: int | None = None) -> List[List[int]]:
    """`seed` fixes the shared prefixes; `suffix_seed` (default: the same stream) the suffixes and the draw of which
    request gets which prefix, so that two traces can share prefixes without sharing anything else."""
    rnd = random.Random(seed)
    fixed = [[rnd.randrange(vocab) for _ in range(prefix_tokens)] for _ in range(prefixes)]
    if suffix_seed is not None:
        rnd = random.Random(suffix_seed)
    out = []
    for _ in range(n):
        suffix = [rnd.randrange(vocab) for _ in range(rnd.randint(suffix_lo, suffix_hi))]
        if fixed and rnd.random() < shared:
            out.append(fixed[rnd.randrange(prefixes)] + suffix)
        else:
            out.append([rnd.randrange(vocab) for _ in range(prefix_tokens)] + suffix if prefix_tokens and not fixed else suffix)
    return out


def _pct(xs: List[float], p: float) -> float:
    if not xs:
        return 0.0
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(p * len(xs)))]


def run_one(host: str, port: int, model: str, prompt: List[int], max_tokens: int, timeout: float) -> Dict:
    body = json.dumps({"model": model, "prompt": prompt, "max_tokens": max_tokens, "stream": True,
                       "stream_options": {"include_usage": True}, "ignore_eos": True})
    t0 = time.perf_counter()
    c = http.client.HTTPConnection(host, port, timeout=timeout)
    c.request("POST", "/v1/completions", body, {"Content-Type": "application/json"})
    r = c.getresponse()
    stamps, usage, buf = [], {}, b""
    if r.status != 200:
        data = r.read()
        c.close()
        return {"ok": False, "status": r.status, "error": data[:200].decode("utf-8", "replace")}
    while True:
        chunk = r.read1(65536) if hasattr(r, "read1") else r.read(4096)
        if not chunk:
            break
        buf += chunk
        while b"\n\n" in buf:
            ev, buf = buf.split(b"\n\n", 1)
            if not ev.startswith(b"data: "):
                continue
            data = ev[6:]
            if data == b"[DONE]":
                continue
            j = json.loads(data)
            if j.get("usage"):
                usage = j["usage"]
            if j.get("choices") and j["choices"][0].get("text"):
                stamps.append(time.perf_counter())
    c.close()
    t1 = time.perf_counter()
    gaps = [b - a for a, b in zip(stamps, stamps[1:])]
    return {"ok": True, "ttft": (stamps[0] - t0) if stamps else t1 - t0, "wall": t1 - t0, "gaps": gaps,
            "prompt_tokens": usage.get("prompt_tokens", len(prompt)), "completion_tokens": usage.get("completion_tokens", 0),
            "cached_tokens": (usage.get("prompt_tokens_details") or {}).get("cached_tokens", 0)}


def run_load(url: str, trace: List[List[int]], concurrency: int, max_tokens: int, model: str = "", timeout: float = 600.0) -> Dict:
    u = urllib.parse.urlparse(url)
    host, port = u.hostname, u.port or 80
    if not model:
        c = http.client.HTTPConnection(host, port, timeout=30)
        c.request("GET", "/v1/models")
        model = json.loads(c.getresponse().read())["data"][0]["id"]
        c.close()
    results: List[Dict] = [None] * len(trace)
    nxt = [0]
    lock = threading.Lock()

    def worker():
        while True:
            with lock:
                i = nxt[0]
                nxt[0] += 1
            if i >= len(trace):
                return
            try:
                results[i] = run_one(host, port, model, trace[i], max_tokens, timeout)
            except Exception as e:  # a dropped connection is a failed request, not a crashed run
                results[i] = {"ok": False, "status": 0, "error": str(e)}

    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker) for _ in range(concurrency)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    good = [r for r in results if r and r["ok"]]
    ttft = [r["ttft"] for r in good]
    hit = [r["ttft"] for r in good if r["cached_tokens"] * 2 >= r["prompt_tokens"]]     # most of the prompt was resident
    gaps = [g for r in good for g in r["gaps"]]
    pt, ct = sum(r["prompt_tokens"] for r in good), sum(r["completion_tokens"] for r in good)
    return {"requests": len(trace), "ok": len(good), "failed": len(trace) - len(good), "concurrency": concurrency,
            "wall_s": round(wall, 3), "prompt_tok_s": round(pt / wall, 1), "completion_tok_s": round(ct / wall, 1),
            "prompt_tokens": pt, "completion_tokens": ct, "cached_tokens": sum(r["cached_tokens"] for r in good),
            "ttft_s": {"p50": round(_pct(ttft, 0.5), 4), "p90": round(_pct(ttft, 0.9), 4), "max": round(max(ttft or [0]), 4)},
            "ttft_prefix_hit_s": {"n": len(hit), "p50": round(_pct(hit, 0.5), 4), "p90": round(_pct(hit, 0.9), 4)},
            "gap_s": {"p50": round(_pct(gaps, 0.5), 5), "p99": round(_pct(gaps, 0.99), 5)},
            "errors": [r["error"] for r in results if r and not r["ok"]][:3]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--prefixes", type=int, default=4)
    ap.add_argument("--prefix-tokens", type=int, default=256)
    ap.add_argument("--shared", type=float, default=0.8)
    ap.add_argument("--suffix-tokens", default="16,128")
    ap.add_argument("--max-tokens", type=int, default=32)
    ap.add_argument("--vocab", type=int, default=4096)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--model", default="")
    a = ap.parse_args(argv)
    lo, hi = (int(x) for x in a.suffix_tokens.split(","))
    trace = make_trace(a.requests, a.vocab, a.prefixes, a.prefix_tokens, a.shared, lo, hi, a.seed)
    print(json.dumps(run_load(a.url, trace, a.concurrency, a.max_tokens, a.model)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
