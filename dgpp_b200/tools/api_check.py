"""API contract check against a running server: one request per documented behaviour of the OpenAI surface, each
judged on status code and response shape.  Prints one line per check and a JSON summary; exit status 1 if any fails.

    python -m dgpp_b200.tools.api_check --url http://127.0.0.1:8000

(reference counterparts: scripts/serve_api_check.py, docs/openai-compatibility.md.)
"""
from __future__ import annotations

import argparse
import http.client
import json
import urllib.parse
from typing import Callable, List, Tuple


class Client:
    def __init__(self, url: str, timeout: float = 120.0):
        u = urllib.parse.urlparse(url)
        self.host, self.port, self.timeout = u.hostname, u.port or 80, timeout

    def call(self, method: str, path: str, body=None, raw: bool = False):
        c = http.client.HTTPConnection(self.host, self.port, timeout=self.timeout)
        data = None if body is None else (body if isinstance(body, (bytes, str)) else json.dumps(body))
        c.request(method, path, data, {"Content-Type": "application/json"} if body is not None else {})
        r = c.getresponse()
        payload = r.read()
        c.close()
        if raw:
            return r.status, payload
        try:
            return r.status, json.loads(payload)
        except ValueError:
            return r.status, payload


def _sse(payload: bytes) -> List[dict]:
    out = []
    for ev in payload.split(b"\n\n"):
        if ev.startswith(b"data: ") and ev[6:] != b"[DONE]":
            out.append(json.loads(ev[6:]))
    return out


def checks(c: Client, model: str) -> List[Tuple[str, Callable[[], bool]]]:
    chat = lambda **kw: c.call("POST", "/v1/chat/completions",
                               {"model": model, "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, **kw})

    def is_error(resp, status, param=None):
        st, j = resp
        return st == status and isinstance(j, dict) and "error" in j and (param is None or j["error"].get("param") == param)

    def stream_ok():
        st, payload = c.call("POST", "/v1/chat/completions", {
            "model": model, "messages": [{"role": "user", "content": "hi"}], "max_tokens": 5, "stream": True,
            "stream_options": {"include_usage": True}}, raw=True)
        ev = _sse(payload)
        return (st == 200 and payload.rstrip().endswith(b"data: [DONE]") and ev and
                ev[0]["object"] == "chat.completion.chunk" and any(e.get("usage") for e in ev) and
                any(e["choices"] and e["choices"][0].get("finish_reason") for e in ev if e.get("choices")))

    def n_choices():
        st, j = chat(n=2, seed=1, temperature=0.8)
        return st == 200 and [ch["index"] for ch in j["choices"]] == [0, 1]

    def usage_adds_up():
        st, j = chat()
        u = j.get("usage", {})
        return st == 200 and u.get("total_tokens") == u.get("prompt_tokens", -1) + u.get("completion_tokens", -1)

    def deterministic():
        a, b = chat(temperature=0), chat(temperature=0)
        return a[0] == b[0] == 200 and a[1]["choices"][0]["message"] == b[1]["choices"][0]["message"]

    def logprobs():
        st, j = chat(logprobs=True, top_logprobs=2)
        lp = j["choices"][0].get("logprobs") if st == 200 else None
        return bool(lp and lp["content"] and "logprob" in lp["content"][0] and len(lp["content"][0]["top_logprobs"]) <= 2)

    def json_mode():
        st, j = chat(response_format={"type": "json_object"}, max_tokens=24)
        if st != 200:
            return False
        text = j["choices"][0]["message"]["content"]
        if j["choices"][0]["finish_reason"] == "length":
            return text.lstrip()[:1] in ("{", "")            # cut off mid-object is still a constrained prefix
        try:
            return isinstance(json.loads(text), dict)
        except ValueError:
            return False

    def completions_ids():
        st, j = c.call("POST", "/v1/completions", {"model": model, "prompt": [1, 2, 3, 4], "max_tokens": 3})
        return st == 200 and j["object"] == "text_completion" and j["usage"]["prompt_tokens"] == 4

    return [
        ("GET /health", lambda: c.call("GET", "/health") == (200, {"status": "ok"})),
        ("GET /v1/models lists the model", lambda: c.call("GET", "/v1/models")[1]["data"][0]["id"] == model),
        ("GET /v1/models/<other> is 404", lambda: c.call("GET", "/v1/models/not-this-model")[0] == 404),
        ("unknown route is 404", lambda: c.call("GET", "/v1/nope")[0] == 404),
        ("wrong method is 405", lambda: c.call("GET", "/v1/chat/completions")[0] == 405),
        ("malformed JSON is 400", lambda: is_error(c.call("POST", "/v1/chat/completions", "{not json"), 400)),
        ("missing messages names the field", lambda: is_error(c.call("POST", "/v1/chat/completions", {"model": model}), 400, "messages")),
        ("bad role names the field", lambda: is_error(c.call("POST", "/v1/chat/completions", {
            "model": model, "messages": [{"role": "wizard", "content": "x"}]}), 400, "messages[0].role")),
        ("temperature out of range is 400", lambda: is_error(chat(temperature=9.0), 400, "temperature")),
        ("max_tokens beyond the context is 400", lambda: is_error(chat(max_tokens=10 ** 7), 400, "max_tokens")),
        ("chat completion shape and usage", usage_adds_up),
        ("greedy is deterministic", deterministic),
        ("n = 2 returns two indexed choices", n_choices),
        ("streaming: chunks, finish_reason, usage, [DONE]", stream_ok),
        ("logprobs with top_logprobs", logprobs),
        ("response_format json_object", json_mode),
        ("completions with a token-id prompt", completions_ids),
        ("metrics JSON and Prometheus", lambda: c.call("GET", "/metrics")[0] == 200 and
         b"# TYPE" in c.call("GET", "/metrics/prometheus", raw=True)[1]),
        ("files: list", lambda: c.call("GET", "/v1/files")[1].get("object") == "list"),
    ]


def run(url: str, model: str = "") -> dict:
    c = Client(url)
    if not model:
        model = c.call("GET", "/v1/models")[1]["data"][0]["id"]
    results = []
    for name, fn in checks(c, model):
        try:
            ok = bool(fn())
            err = ""
        except Exception as e:  # a check that cannot even read the answer has failed
            ok, err = False, f"{type(e).__name__}: {e}"
        results.append({"check": name, "ok": ok, "error": err})
    return {"url": url, "model": model, "passed": sum(r["ok"] for r in results), "failed": sum(not r["ok"] for r in results),
            "results": results}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="")
    a = ap.parse_args(argv)
    out = run(a.url, a.model)
    for r in out["results"]:
        print(f"{'ok  ' if r['ok'] else 'FAIL'} {r['check']}" + (f"   ({r['error']})" if r["error"] else ""))
    print(json.dumps({k: out[k] for k in ("url", "model", "passed", "failed")}))
    return 0 if out["failed"] == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
