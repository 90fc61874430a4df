"""HTTP serving end to end on CPU: native HTTP/SSE server + OpenAI layer + scheduler + deterministic fake engine.
(Model of the reference's serving tests: tests/test_openai_compat.cpp, tests/test_http_server.cpp.)"""
import http.client
import json

import pytest

from dgpp_b200.runtime import rt
from dgpp_b200.serve.app import Server


@pytest.fixture()
def server():
    tok = rt.Tokenizer.byte_level([], [("<|im_start|>", 256, True), ("<|im_end|>", 257, True)], rt.SplitPattern.Qwen2)
    eng = rt.FakeEngine(slots=4, block_tokens=16, blocks=1024, max_context=2048, vocab=256)
    srv = Server(eng, tok, model_name="fake", eos_ids=[257])
    port = srv.start()
    yield srv, port
    srv.stop()


def _req(port, method, path, body=None):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=20)
    c.request(method, path, body, {"Content-Type": "application/json"} if body is not None else {})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, data


def test_health_models_and_unknown_route(server):
    _, port = server
    assert _req(port, "GET", "/health") == (200, b'{"status":"ok"}')
    st, body = _req(port, "GET", "/v1/models")
    assert st == 200 and json.loads(body)["data"][0]["id"] == "fake"
    assert _req(port, "GET", "/v1/models/fake")[0] == 200
    assert _req(port, "GET", "/v1/models/other")[0] == 404
    assert _req(port, "GET", "/nope")[0] == 404
    assert _req(port, "GET", "/v1/chat/completions")[0] == 405


def test_chat_completion_matches_fake_engine_and_usage(server):
    _, port = server
    body = json.dumps({"model": "fake", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 8})
    st, a = _req(port, "POST", "/v1/chat/completions", body)
    st2, b = _req(port, "POST", "/v1/chat/completions", body)
    assert st == 200 and st2 == 200
    ja, jb = json.loads(a), json.loads(b)
    assert ja["object"] == "chat.completion"
    assert ja["choices"][0]["finish_reason"] == "length"
    assert ja["choices"][0]["message"]["content"] == jb["choices"][0]["message"]["content"]     # deterministic
    assert ja["usage"]["completion_tokens"] == 8
    assert ja["usage"]["total_tokens"] == ja["usage"]["prompt_tokens"] + 8
    # the second identical request hits the 16-token block prefix cache
    assert jb["usage"]["prompt_tokens_details"]["cached_tokens"] >= 16


def test_streaming_chunks_usage_and_done(server):
    _, port = server
    body = json.dumps({"model": "fake", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "stream": True,
                       "stream_options": {"include_usage": True}})
    st, data = _req(port, "POST", "/v1/chat/completions", body)
    assert st == 200
    events = [e[len("data: "):] for e in data.decode("utf-8", "replace").split("\n\n") if e.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    finals = [c for c in chunks if c["choices"] and c["choices"][0]["finish_reason"]]
    assert len(finals) == 1 and finals[0]["choices"][0]["finish_reason"] == "length"
    usage = [c for c in chunks if c.get("usage")]
    assert len(usage) == 1 and usage[0]["usage"]["completion_tokens"] == 6
    # streamed text == non-streamed text
    st, whole = _req(port, "POST", "/v1/chat/completions",
                     json.dumps({"model": "fake", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 6}))
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"])
    assert text == json.loads(whole)["choices"][0]["message"]["content"]


def test_completions_n_and_token_prompt(server):
    _, port = server
    st, data = _req(port, "POST", "/v1/completions", json.dumps({"model": "fake", "prompt": "abc", "max_tokens": 5, "n": 2}))
    j = json.loads(data)
    assert st == 200 and [c["index"] for c in j["choices"]] == [0, 1]
    assert j["choices"][0]["text"] == j["choices"][1]["text"]
    assert j["usage"]["completion_tokens"] == 10
    st, data = _req(port, "POST", "/v1/completions", json.dumps({"model": "fake", "prompt": [97, 98, 99], "max_tokens": 5}))
    assert st == 200 and json.loads(data)["choices"][0]["text"] == j["choices"][0]["text"]


def test_bad_requests(server):
    _, port = server
    st, data = _req(port, "POST", "/v1/completions", "{bad")
    assert st == 400 and json.loads(data)["error"]["type"] == "invalid_request_error"
    st, data = _req(port, "POST", "/v1/chat/completions", json.dumps({"model": "fake", "messages": []}))
    assert st == 400
    st, data = _req(port, "POST", "/v1/completions", json.dumps({"model": "fake", "prompt": "x" * 3000, "max_tokens": 10}))
    assert st == 400 and json.loads(data)["error"]["code"] == "context_length_exceeded"


def test_stop_sequence_truncates(server):
    _, port = server
    st, data = _req(port, "POST", "/v1/completions", json.dumps({"model": "fake", "prompt": "abc", "max_tokens": 16}))
    full = json.loads(data)["choices"][0]["text"]
    # choose an ASCII character from the middle of the output as the stop string
    cut = next((i for i in range(1, len(full)) if full[i].isascii() and full[i] not in full[:i]), None)
    if cut is None:
        pytest.skip("fake engine output has no usable ASCII stop character")
    st, data = _req(port, "POST", "/v1/completions",
                    json.dumps({"model": "fake", "prompt": "abc", "max_tokens": 16, "stop": [full[cut]]}))
    j = json.loads(data)
    assert j["choices"][0]["text"] == full[:cut]
    assert j["choices"][0]["finish_reason"] == "stop"


def test_metrics(server):
    _, port = server
    _req(port, "POST", "/v1/completions", json.dumps({"model": "fake", "prompt": "abc", "max_tokens": 4}))
    st, data = _req(port, "GET", "/metrics")
    j = json.loads(data)
    assert st == 200 and j["counters"]["requests_total"] == 1 and j["counters"]["completion_tokens_total"] == 4
    st, data = _req(port, "GET", "/metrics/prometheus")
    text = data.decode()
    assert "dgpp_b200_requests_total 1" in text and "time_to_first_token_seconds_count 1" in text


def test_tool_calls_are_parsed_from_generated_text():
    """An engine that 'generates' a fixed text with a tool call: the server must return it as tool_calls."""
    tok = rt.Tokenizer.byte_level([], [("<|im_start|>", 256, True), ("<|im_end|>", 257, True)], rt.SplitPattern.Qwen2)
    script = b'Checking.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Oslo"}}\n</tool_call>'
    script_ids = list(script) + [257]

    class Engine(rt.SchedulerEngine):
        def __init__(self):
            super().__init__()
            self.pos = {}
            self.blocks = {}
        def max_concurrent(self): return 2
        def block_tokens(self): return 16
        def total_blocks(self): return 512
        def free_blocks(self): return 512 - sum(len(b) for b in self.blocks.values())
        def max_context(self): return 4096
        def reserve(self, slot, tokens):
            need = (tokens + 15) // 16
            cur = self.blocks.setdefault(slot, [])
            while len(cur) < need:
                cur.append(len(cur) + slot * 256)
            return True
        def attach_prefix(self, slot, blocks): self.blocks[slot] = list(blocks)
        def prefill(self, slot, tokens, pos, last):
            self.pos[slot] = 0
            return script_ids[0] if last else -1
        def step_batch(self, slots):
            out = []
            for s in slots:
                self.pos[s] += 1
                out.append([script_ids[min(self.pos[s], len(script_ids) - 1)]])
            return out
        def slot_blocks(self, slot): return list(self.blocks.get(slot, []))
        def retain_block(self, b): pass
        def release_block(self, b): pass
        def block_refcount(self, b): return 1
        def close(self, slot): self.blocks.pop(slot, None)

    srv = Server(Engine(), tok, model_name="scripted", eos_ids=[257])
    port = srv.start()
    try:
        req = {"model": "scripted", "messages": [{"role": "user", "content": "weather?"}], "max_tokens": 200,
               "tools": [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object"}}}]}
        st, data = _req(port, "POST", "/v1/chat/completions", json.dumps(req))
        j = json.loads(data)
        ch = j["choices"][0]
        assert st == 200 and ch["finish_reason"] == "tool_calls"
        assert ch["message"]["content"] == "Checking.\n"
        call = ch["message"]["tool_calls"][0]
        assert call["function"]["name"] == "get_weather" and json.loads(call["function"]["arguments"]) == {"city": "Oslo"}
        # streaming: the call arrives as one tool_calls delta, then finish_reason tool_calls
        st, data = _req(port, "POST", "/v1/chat/completions", json.dumps({**req, "stream": True}))
        events = [json.loads(e[6:]) for e in data.decode().split("\n\n") if e.startswith("data: {")]
        deltas = [c["choices"][0]["delta"] for c in events if c["choices"]]
        calls = [d["tool_calls"][0] for d in deltas if d.get("tool_calls")]
        assert len(calls) == 1 and calls[0]["function"]["name"] == "get_weather" and calls[0]["index"] == 0
        assert "".join(d.get("content") or "" for d in deltas) == "Checking.\n"
        assert [c["choices"][0]["finish_reason"] for c in events if c["choices"]][-1] == "tool_calls"
        # without tools in the request the same text is plain content
        st, data = _req(port, "POST", "/v1/chat/completions", json.dumps({k: v for k, v in req.items() if k != "tools"}))
        assert "<tool_call>" in json.loads(data)["choices"][0]["message"]["content"]
    finally:
        srv.stop()


def test_tool_choice_naming_an_unknown_function_is_rejected(server):
    _, port = server
    req = {"model": "fake", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
           "tools": [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}}],
           "tool_choice": {"type": "function", "function": {"name": "g"}}}
    st, data = _req(port, "POST", "/v1/chat/completions", json.dumps(req))
    assert st == 400 and json.loads(data)["error"]["param"] == "tool_choice"
    req["tool_choice"] = {"type": "function", "function": {"name": "f"}}
    assert _req(port, "POST", "/v1/chat/completions", json.dumps(req))[0] == 200


def _failing_engine(ok_steps):
    """A CPU reference engine that, after `ok_steps` decode passes, raises what KernelEngine raises when the device
    status block reports a failed bounded wait (made on the host: nothing faults or hangs)."""
    from dgpp_b200.engine.adapters import EngineFailure, ReferenceEngine
    from dgpp_b200.models.dense import DenseConfig, DenseModel

    class FailsAfter(ReferenceEngine):
        left = ok_steps

        def step_batch(self, slots):
            if self.left <= 0:
                raise EngineFailure("device status code=4 count=1 detail=1 (a bounded device wait gave up)")
            self.left -= 1
            return super().step_batch(slots)

    model = DenseModel.random_init(DenseConfig.plumbing_fp32(vocab=256), device="cpu", seed=0)
    return FailsAfter(model, slots=2, num_blocks=64, block_tokens=16, max_context=256)


def test_engine_failure_reaches_open_streams_and_stops_the_server():
    tok = rt.Tokenizer.byte_level([], [("<|im_start|>", 256, True), ("<|im_end|>", 257, True)], rt.SplitPattern.Qwen2)
    eng = _failing_engine(ok_steps=3)
    srv = Server(eng, tok, model_name="fake", eos_ids=[257])
    port = srv.start()
    try:
        body = json.dumps({"model": "fake", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 50, "stream": True})
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=20)
        c.request("POST", "/v1/chat/completions", body, {"Content-Type": "application/json"})
        data = c.getresponse().read().decode()
        c.close()
        events = [json.loads(l[6:]) for l in data.splitlines() if l.startswith("data: {")]
        assert any("choices" in e for e in events)                                   # some tokens were streamed
        err = [e for e in events if "error" in e]
        assert err and err[-1]["error"]["type"] == "engine_failure" and "device status" in err[-1]["error"]["message"]
        assert srv.failed_event.wait(5.0)                                            # what main() turns into exit status 2
        st, b = _req(port, "GET", "/health")
        assert st == 503 and json.loads(b)["error"]["type"] == "engine_failure"
    finally:
        srv.stop()
