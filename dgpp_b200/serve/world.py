"""Multi-rank serving: rank 0 owns the HTTP front end and the scheduler's inputs, every other rank replays them.

The scheduler is a pure function of its input stream, so ranks stay in lock step when they see the same submits,
cancels and tick boundaries in the same order.  Rank 0 (``WorldLeader``) appends every such input to the operation
journal and sends the record to each follower over a framed TCP connection BEFORE acting on it; a follower
(``run_follower``) replays the records into its own scheduler + engine.  A `tick` record carries the leader's
scheduler digest from before the tick: a follower whose own digest differs has diverged and stops with an error
instead of entering a collective with different shapes.  A closed connection ends the follower (exit status 3 in
the serving process) and marks the leader's world as failed.
(reference counterparts: src/serve/fabric_serve.cpp JournalWriter / JournalReader / run_journal_peer, the
 settings + warm records, per-tick admission / cancel records with op-stream digests.)
"""
from __future__ import annotations

import json
from typing import List, Optional

from ..runtime import rt

MASK63 = (1 << 63) - 1


class WorldLeader:
    def __init__(self, world: int, port: int = 0, config_digest: int = 0, accept_timeout_s: float = 60.0):
        self.world = world
        self.journal = rt.Journal()
        self.listener = rt.Listener(port, True)
        self.port = self.listener.port()
        self.config_digest = config_digest
        self.followers: List[object] = []
        self.failed: Optional[str] = None
        self._accept_timeout_ms = int(accept_timeout_s * 1000)

    def wait_for_followers(self) -> None:
        """Accept world - 1 followers; each one first receives the settings record (world size, config digest)."""
        while len(self.followers) < self.world - 1:
            s = self.listener.accept(self._accept_timeout_ms)
            if s is None:
                raise RuntimeError(f"only {len(self.followers)} of {self.world - 1} followers connected")
            s.send(json.dumps({"op": "settings", "world": self.world, "config_digest": str(self.config_digest)}).encode())
            hello = s.recv(self._accept_timeout_ms)
            if hello is None or json.loads(hello).get("config_digest") != str(self.config_digest):
                raise RuntimeError("a follower runs a different configuration")
            self.followers.append(s)

    def _send(self, rec: dict) -> None:
        line = rec["line"].encode()
        for s in self.followers:
            if not s.send(line):
                self.failed = "a follower's journal connection is closed"
                raise RuntimeError(self.failed)

    def submit(self, sched, rid: str, ids, max_tokens: int, **kw) -> None:
        extra = json.dumps(kw, sort_keys=True)
        self._send(self.journal.append("submit", rid, list(ids), int(max_tokens), extra))
        sched.submit(rid, list(ids), max_tokens, **kw)

    def configure(self, rid: str, params: Optional[dict], grammar_spec, prompt_ids) -> None:
        """Sampling parameters / grammar of a request, sent ahead of its submit record so that every rank binds the
        same sampler state to the request (grammar_spec: ["json", schema] or ["tools", tools_json, required,
        parallel, only-function] -- each rank compiles its own copy)."""
        extra = json.dumps({"params": params, "grammar": grammar_spec}, sort_keys=True)
        self._send(self.journal.append("configure", rid, list(prompt_ids or []), 0, extra))

    def cancel(self, sched, rid: str) -> None:
        self._send(self.journal.append("cancel", rid))
        sched.cancel(rid)

    def tick(self, sched) -> None:
        self._send(self.journal.append("tick", "", [], sched.op_digest() & MASK63))
        sched.tick()

    def shutdown(self) -> None:
        try:
            self._send(self.journal.append("shutdown"))
        except RuntimeError:
            pass
        for s in self.followers:
            s.close()
        self.followers = []


class RankMetrics:
    """Per-rank Prometheus listener of a follower (`dgpp_rank_*` families): the leader's HTTP endpoint only knows
    rank 0, so every other rank answers GET /metrics/prometheus (and /health) on its own port.
    (reference counterpart: src/serve/rank_metrics.cpp.)"""

    def __init__(self, rank: int, port: int = 0, host: str = "127.0.0.1"):
        import threading
        self.rank = rank
        self.c = {"journal_records_total": 0, "ticks_total": 0, "tokens_total": 0, "submits_total": 0,
                  "cancels_total": 0}
        self.http = rt.HttpServer(host, port)
        self.http.start()
        self.port = self.http.port()
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._loop, daemon=True)
        self._t.start()

    def text(self) -> str:
        lines = [f'dgpp_rank_up{{rank="{self.rank}"}} 1']
        for k, v in self.c.items():
            lines.append(f"# TYPE dgpp_rank_{k} counter")
            lines.append(f'dgpp_rank_{k}{{rank="{self.rank}"}} {v}')
        return "\n".join(lines) + "\n"

    def _loop(self) -> None:
        while not self._stop.is_set():
            for req in self.http.poll(50):
                if req["method"] == "GET" and req["path"] in ("/metrics", "/metrics/prometheus"):
                    self.http.respond(req["conn"], 200, "text/plain; version=0.0.4", self.text().encode())
                elif req["method"] == "GET" and req["path"] == "/health":
                    self.http.respond(req["conn"], 200, "application/json", b'{"status":"ok"}')
                else:
                    self.http.respond(req["conn"], 404, "application/json", b'{"error":"not found"}')

    def stop(self) -> None:
        self._stop.set()
        self._t.join(5)
        self.http.stop()


def run_follower(engine, host: str, port: int, sched_config=None, config_digest: int = 0, on_events=None,
                 idle_timeout_ms: int = 1000, max_idle_s: float = 0.0, metrics: Optional[RankMetrics] = None,
                 on_configure=None) -> int:
    """Replay the leader's journal into a local scheduler + engine until a `shutdown` record (returns 0) or until
    the leader goes away (returns 3).  A digest mismatch raises.  `on_events(list)` receives the scheduler's events
    after every tick (followers normally drop them: rank 0 answers the clients)."""
    sock = rt.FramedSocket.connect(host, port, 30000)
    first = sock.recv(30000)
    if first is None:
        raise RuntimeError("no settings record from the leader")
    settings = json.loads(first)
    if settings.get("config_digest") != str(config_digest):
        sock.send(json.dumps({"config_digest": str(config_digest)}).encode())
        raise RuntimeError("this rank runs a different configuration than the leader")
    sock.send(json.dumps({"config_digest": str(config_digest)}).encode())
    sched = rt.Scheduler(engine, sched_config or rt.SchedulerConfig())
    journal = rt.Journal()
    idle = 0.0
    while True:
        try:
            frame = sock.recv(idle_timeout_ms)
        except RuntimeError:
            return 3                                    # the leader closed the connection
        if frame is None:
            idle += idle_timeout_ms / 1000.0
            if max_idle_s and idle >= max_idle_s:
                return 3
            continue
        idle = 0.0
        rec = journal.replay_line(frame.decode())       # order + running digest are checked here
        op = rec["op"]
        if metrics is not None:
            metrics.c["journal_records_total"] += 1
            if op in ("submit", "cancel", "tick"):
                metrics.c[op + "s_total"] += 1
        if op == "submit":
            kw = json.loads(rec["extra"]) if rec["extra"] else {}
            sched.submit(rec["id"], list(rec["tokens"]), rec["arg"], **kw)
        elif op == "configure":
            if on_configure is not None:
                d = json.loads(rec["extra"])
                on_configure(rec["id"], d.get("params"), d.get("grammar"), list(rec["tokens"]))
        elif op == "cancel":
            sched.cancel(rec["id"])
        elif op == "tick":
            mine = sched.op_digest() & MASK63
            if mine != rec["arg"]:
                raise RuntimeError(f"scheduler digest {mine:x} differs from the leader's {rec['arg']:x} at journal "
                                   f"record {rec['seq']}: this rank has diverged")
            sched.tick()
            ev = sched.events()
            if metrics is not None:
                metrics.c["tokens_total"] += sum(1 for e in ev if e[0] == "token")
            if on_events is not None:
                on_events(ev)
        elif op == "shutdown":
            sock.close()
            return 0
        else:
            raise RuntimeError(f"unknown journal record {op!r}")
