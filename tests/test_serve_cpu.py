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
