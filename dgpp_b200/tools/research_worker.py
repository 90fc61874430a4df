"""Research worker: an opt-in socket service that exposes a loaded dense model to analysis scripts.

One JSON object per line in, one per line out, over TCP on a loopback address (never bound elsewhere).  Operations:

    {"op": "info"}                                            model shape, adapter state
    {"op": "logits", "tokens": [...], "top_k": 5, "full": false}
                                                              next-token distribution after the prompt: top ids with
                                                              log-probabilities, optionally every logit (base64 fp32)
    {"op": "generate", "tokens": [...], "max_new": 16, "stop": [ids]}
                                                              greedy continuation (ties to the lower id)
    {"op": "likelihood", "tokens": [...], "start": k}         teacher-forced log-probability of tokens[k:] given what
                                                              precedes each (sum and per token)
    {"op": "capture", "tokens": [...], "layers": [0, 3], "rows": "last" | "all"}
                                                              bf16 residual stream entering the listed layers (the
                                                              layer count names the final-norm input), base64 fp32
    {"op": "install_adapter", "dir": path} / {"op": "remove_adapter"}
                                                              low-rank adapter from an adapter directory
    {"op": "shutdown"}

Every reply carries "ok"; failures carry "error" and leave the worker serving.  With `token` set, every request must
carry the same "token".  All arithmetic is the model's PyTorch oracle (the numerics contract of the kernels), so the
worker runs wherever the weights are, CPU included; requests are served one at a time.
(reference counterpart: apps/dgpp_heretic_worker.cpp: logits, greedy generation, activation capture, teacher-forced
 likelihood, adapter install over a research socket.)
"""
from __future__ import annotations

import argparse
import base64
import json
import socket
import socketserver
import threading
from typing import Any, Dict, List, Optional

import torch


def _b64(t: torch.Tensor) -> Dict[str, Any]:
    a = t.detach().float().cpu().contiguous()
    return {"shape": list(a.shape), "dtype": "f32", "b64": base64.b64encode(a.numpy().tobytes()).decode()}


class ResearchWorld:
    """The model and the operations on it."""

    MAX_TOKENS = 32768

    def __init__(self, model, adapter=None):
        self.model, self.adapter = model, adapter
        self.lock = threading.Lock()

    def _tokens(self, req: dict, need: int = 1) -> torch.Tensor:
        toks = req.get("tokens")
        v = self.model.cfg.vocab
        if not isinstance(toks, list) or len(toks) < need or len(toks) > self.MAX_TOKENS or \
                not all(isinstance(t, int) and not isinstance(t, bool) and 0 <= t < v for t in toks):
            raise ValueError(f"tokens must be a list of {need}..{self.MAX_TOKENS} ids in [0, {v})")
        return torch.tensor(toks, dtype=torch.int64)

    def _forward(self, toks: torch.Tensor, start: int = 0, kv=None, capture=None):
        return self.model.forward_reference(toks, start_pos=start, kv=kv, lora=self.adapter, capture=capture)

    def info(self, req: dict) -> dict:
        c = self.model.cfg
        return {"layers": c.layers, "hidden": c.hidden, "vocab": c.vocab, "q_heads": c.q_heads, "kv_heads": c.kv_heads,
                "head_dim": c.head_dim, "adapter": self.adapter is not None, "device": str(self.model.embed.device)}

    def logits(self, req: dict) -> dict:
        lg, _ = self._forward(self._tokens(req))
        last = lg[-1].float()
        lp = torch.log_softmax(last, -1)
        k = max(1, min(int(req.get("top_k", 5)), last.numel()))
        order = torch.argsort(-last, stable=True)[:k]
        out = {"top": [{"id": int(i), "logprob": float(lp[i]), "logit": float(last[i])} for i in order]}
        if req.get("full"):
            out["logits"] = _b64(last)
        return out

    def generate(self, req: dict) -> dict:
        toks = self._tokens(req)
        n = int(req.get("max_new", 16))
        if not 0 < n <= 4096:
            raise ValueError("max_new must be in 1..4096")
        stop = set(req.get("stop") or [])
        lg, kv = self._forward(toks)
        out: List[int] = []
        pos = toks.numel()
        for _ in range(n):
            last = lg[-1].float()
            nxt = int(torch.argsort(-last, stable=True)[0])
            out.append(nxt)
            if nxt in stop:
                break
            lg, kv = self._forward(torch.tensor([nxt]), start=pos, kv=kv)
            pos += 1
        return {"tokens": out}

    def likelihood(self, req: dict) -> dict:
        toks = self._tokens(req, need=2)
        start = int(req.get("start", 1))
        if not 1 <= start < toks.numel():
            raise ValueError("start must be in 1..len(tokens) - 1")
        lg, _ = self._forward(toks[:-1])
        lp = torch.log_softmax(lg.float(), -1)
        per = lp[torch.arange(start - 1, toks.numel() - 1), toks[start:].to(lp.device)]
        return {"logprob": float(per.sum()), "per_token": [float(x) for x in per], "count": int(per.numel())}

    def capture(self, req: dict) -> dict:
        toks = self._tokens(req)
        layers = req.get("layers")
        L = self.model.cfg.layers
        if not isinstance(layers, list) or not layers or not all(isinstance(i, int) and 0 <= i <= L for i in layers):
            raise ValueError(f"layers must list indices in 0..{L}")
        cap = {i: None for i in layers}
        self._forward(toks, capture=cap)
        last = req.get("rows", "last") == "last"
        return {"activations": {str(i): _b64(t[-1:] if last else t) for i, t in cap.items()}}

    def install_adapter(self, req: dict) -> dict:
        from ..adapters.lora import load_adapter

        d = req.get("dir")
        if not isinstance(d, str):
            raise ValueError("dir must be a path")
        self.adapter = load_adapter(d, self.model.cfg, device=self.model.embed.device)
        return {"rank": int(self.adapter.rank), "scale": float(self.adapter.scale)}

    def remove_adapter(self, req: dict) -> dict:
        self.adapter = None
        return {}

    OPS = ("info", "logits", "generate", "likelihood", "capture", "install_adapter", "remove_adapter")

    def handle(self, req: dict) -> dict:
        op = req.get("op")
        if op not in self.OPS:
            raise ValueError(f"unknown op {op!r}; one of {', '.join(self.OPS)}, shutdown")
        with self.lock, torch.no_grad():
            return getattr(self, op)(req)


class FamilyWorld(ResearchWorld):
    """The same operations over a model of the smaller families (anything with `forward_reference(tokens)` and
    `cfg.vocab`): every call recomputes the whole prompt, there is no activation capture and no adapter."""

    OPS = ("info", "logits", "generate", "likelihood")

    def _forward(self, toks, start: int = 0, kv=None, capture=None):
        prev = kv if kv is not None else toks[:0]
        full = torch.cat([prev, toks]) if start else toks
        return self.model.forward_reference(full), full

    def info(self, req: dict) -> dict:
        c = self.model.cfg
        return {"family": type(self.model).__name__, "layers": c.layers, "hidden": c.hidden, "vocab": c.vocab,
                "adapter": False, "device": str(self.model.embed.device)}


class _Handler(socketserver.StreamRequestHandler):
    def handle(self):
        srv = self.server
        for raw in self.rfile:
            if len(raw) > srv.max_line:
                reply = {"ok": False, "error": "request line too long"}
            else:
                try:
                    req = json.loads(raw)
                    if not isinstance(req, dict):
                        raise ValueError("a request is one JSON object")
                    if srv.token and req.get("token") != srv.token:
                        raise PermissionError("bad token")
                    if req.get("op") == "shutdown":
                        self.wfile.write(b'{"ok": true}\n')
                        threading.Thread(target=srv.shutdown, daemon=True).start()
                        return
                    reply = {"ok": True, **srv.world.handle(req)}
                except Exception as e:  # the worker keeps serving: the caller gets the reason
                    reply = {"ok": False, "error": f"{type(e).__name__}: {e}"}
            self.wfile.write((json.dumps(reply) + "\n").encode())
            self.wfile.flush()


class ResearchServer(socketserver.ThreadingTCPServer):
    allow_reuse_address = True
    daemon_threads = True

    def __init__(self, world: ResearchWorld, port: int = 0, token: str = "", host: str = "127.0.0.1", max_line: int = 1 << 22):
        if host not in ("127.0.0.1", "::1", "localhost"):
            raise ValueError("the research worker binds loopback addresses only")
        super().__init__((host, port), _Handler)
        self.world, self.token, self.max_line = world, token, max_line

    @property
    def port(self) -> int:
        return self.server_address[1]


def request(port: int, obj: dict, host: str = "127.0.0.1", timeout: float = 120.0) -> dict:
    """One request, one reply (client side, for scripts and tests)."""
    with socket.create_connection((host, port), timeout=timeout) as s:
        s.sendall((json.dumps(obj) + "\n").encode())
        buf = b""
        while not buf.endswith(b"\n"):
            part = s.recv(1 << 16)
            if not part:
                break
            buf += part
    return json.loads(buf)


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="research socket worker over a dense checkpoint (loopback only)")
    ap.add_argument("--model-dir", default="", help="dense safetensors checkpoint; empty: the tiny random-init model")
    ap.add_argument("--family-dir", default="", help="a native family checkpoint (loaders.family_io) instead")
    ap.add_argument("--port", type=int, default=8791)
    ap.add_argument("--token", default="")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    if a.family_dir:
        from ..loaders.family_io import load_family
        srv = ResearchServer(FamilyWorld(load_family(a.family_dir, a.device)), a.port, a.token)
        print(json.dumps({"research_worker": "listening", "port": srv.port}), flush=True)
        srv.serve_forever()
        return 0
    if a.model_dir:
        from ..loaders.checkpoint import load_dense
        model = load_dense(a.model_dir, device=a.device)
    else:
        from ..models.dense import DenseConfig, DenseModel
        model = DenseModel.random_init(DenseConfig.tiny(weight_fmt="bf16"), device=a.device, seed=0, std=0.05)
    srv = ResearchServer(ResearchWorld(model), a.port, a.token)
    print(json.dumps({"research_worker": "listening", "port": srv.port}), flush=True)
    srv.serve_forever()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
