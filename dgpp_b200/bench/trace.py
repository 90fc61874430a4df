"""Serve a model over HTTP and drive the multi-turn shared-prefix trace against it at several concurrencies.

    python -m dgpp_b200.bench.trace --model hybrid --slots 32 --max-context 24576 --concurrency 1,8,32 \
        --requests 256 --prefixes 4 --prefix-tokens 16384 --shared 0.8 --suffix-tokens 512,4096 --max-tokens 512 \
        --vocab 151936 [--mtp-depth 3]

Starts `python -m dgpp_b200.serve.app` with the given model flags as a child process, waits for its listening line,
runs `dgpp_b200.bench.load` once per concurrency (each on a fresh seed, so a later run does not hit the earlier run's
suffixes; the fixed prefixes stay resident in the prefix cache between runs, and the first run's misses are reported
through its cached-token total), stops the child and prints one JSON object.  (reference counterparts:
scripts/serve_campaign.py, bench/http_trace.)
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time

from .load import make_trace, run_load


def _start(cmd, log_path: str, wait_s: float):
    log = open(log_path, "w")
    proc = subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
    t0 = time.time()
    while time.time() - t0 < wait_s:
        if proc.poll() is not None:
            raise RuntimeError(f"server exited with {proc.returncode}: see {log_path}")
        with open(log_path) as f:
            for line in f:
                if line.startswith("listening on "):
                    return proc, line.split()[-1].strip(), time.time() - t0
        time.sleep(0.5)
    os.killpg(proc.pid, signal.SIGTERM)
    raise RuntimeError(f"server did not come up in {wait_s:.0f} s: see {log_path}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="hybrid-tiny")
    ap.add_argument("--slots", type=int, default=8)
    ap.add_argument("--max-context", type=int, default=4096)
    ap.add_argument("--mtp-depth", type=int, default=0)
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--port", type=int, default=8077)
    ap.add_argument("--concurrency", default="1,8")
    ap.add_argument("--requests", default="64", help="one count, or one per concurrency")
    ap.add_argument("--prefixes", type=int, default=4)
    ap.add_argument("--prefix-tokens", type=int, default=1024)
    ap.add_argument("--shared", type=float, default=0.8)
    ap.add_argument("--suffix-tokens", default="64,512")
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--vocab", type=int, default=4096)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--server-log", default="trace_server.log")
    ap.add_argument("--mixed-pass", action="store_true", help="start the server with mixed reader + decoder passes")
    ap.add_argument("--prefill-budget-busy", type=int, default=0)
    ap.add_argument("--startup-s", type=float, default=600.0)
    ap.add_argument("--request-timeout-s", type=float, default=900.0)
    a = ap.parse_args(argv)
    cmd = [sys.executable, "-m", "dgpp_b200.serve.app", "--model", a.model, "--slots", str(a.slots), "--port", str(a.port),
           "--max-context", str(a.max_context), "--mtp-depth", str(a.mtp_depth), "--layers", str(a.layers)]
    if a.mixed_pass:
        cmd.append("--mixed-pass")
    if a.prefill_budget_busy:
        cmd += ["--prefill-budget-busy", str(a.prefill_budget_busy)]
    proc, url, up_s = _start(cmd, a.server_log, a.startup_s)
    lo, hi = (int(x) for x in a.suffix_tokens.split(","))
    conc = [int(x) for x in a.concurrency.split(",")]
    reqs = [int(x) for x in a.requests.split(",")]
    reqs = reqs * len(conc) if len(reqs) == 1 else reqs
    assert len(reqs) == len(conc), "--requests: one count, or one per concurrency"
    out = {"model": a.model, "mixed_pass": bool(a.mixed_pass), "mtp_depth": a.mtp_depth, "slots": a.slots, "startup_s": round(up_s, 1),
           "trace": {"requests": reqs, "prefixes": a.prefixes, "prefix_tokens": a.prefix_tokens, "shared": a.shared,
                     "suffix_tokens": [lo, hi], "max_tokens": a.max_tokens, "vocab": a.vocab}, "runs": []}
    try:
        run_load(url, [[1, 2, 3, 4]], 1, 2, timeout=a.request_timeout_s)      # first-request costs (lazy imports) stay out of the trace
        for k, c in enumerate(conc):
            trace = make_trace(reqs[k], a.vocab, a.prefixes, a.prefix_tokens, a.shared, lo, hi, a.seed, suffix_seed=a.seed + 1 + k)
            out["runs"].append(run_load(url, trace, c, a.max_tokens, timeout=a.request_timeout_s))
            print(json.dumps(out["runs"][-1]), file=sys.stderr, flush=True)
    finally:
        os.killpg(proc.pid, signal.SIGTERM)          # the child's own process group: nothing else is in it
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
