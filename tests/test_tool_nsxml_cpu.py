"""Namespace-XML tool calls (MiniMax style) through the streaming parser: several invokes per block, nested values,
schema-typed scalars, arbitrary chunking, malformed blocks returned as content."""
import json

from dgpp_b200.runtime import rt

NS = "]<]minimax[>["


def _block(*invokes):
    return NS + "<tool_call>\n" + "\n".join(invokes) + "\n" + NS + "</tool_call>"


def _invoke(name, body):
    return f'{NS}<invoke name="{name}">{body}{NS}</invoke>'


def _run(text, step, tools=None):
    p = rt.ToolParser(rt.ToolFormat.NsXml, "c_")
    if tools is not None:
        p.set_tools(json.dumps(tools))
    ev = []
    data = text.encode()
    for i in range(0, len(data), step):
        ev += p.feed(data[i:i + step])
    ev += p.finish()
    content = b"".join(e[1] for e in ev if e[0] == "content").decode()
    calls = [(e[3], json.loads(e[4])) for e in ev if e[0] == "tool_call"]
    return content, calls, p.calls()


TOOLS = [{"type": "function", "function": {"name": "search", "parameters": {"type": "object", "properties": {
    "query": {"type": "string"}, "limit": {"type": "integer"}, "exact": {"type": "boolean"},
    "filters": {"type": "object", "properties": {"lang": {"type": "string"}, "years": {"type": "array", "items": {"type": "integer"}}}},
    "code": {"type": "string"}}}}},
    {"type": "function", "function": {"name": "noop", "parameters": {"type": "object", "properties": {}}}}]


def test_two_invokes_nested_values_and_schema_types():
    body = (f"{NS}<query>a < b & c{NS}</query>{NS}<limit>5{NS}</limit>{NS}<exact>true{NS}</exact>"
            f"{NS}<filters>{NS}<lang>en{NS}</lang>{NS}<years>{NS}<item>2020{NS}</item>{NS}<item>2021{NS}</item>{NS}</years>{NS}</filters>"
            f"{NS}<code>42{NS}</code>")
    text = "Let me look.\n" + _block(_invoke("search", body), _invoke("noop", "")) + "\nDone."
    want = [("search", {"query": "a < b & c", "limit": 5, "exact": True, "filters": {"lang": "en", "years": [2020, 2021]},
                        "code": "42"}), ("noop", {})]
    for step in (1, 3, 7, 64, 10000):
        content, calls, n = _run(text, step, TOOLS)
        assert calls == want and n == 2, step
        assert content == "Let me look.\nDone.", (step, content)


def test_without_schemas_scalars_read_as_literals_or_strings():
    body = f"{NS}<n>3.5{NS}</n>{NS}<flag>false{NS}</flag>{NS}<none>null{NS}</none>{NS}<s>hello world{NS}</s>" \
           f"{NS}<list>{NS}<item>x{NS}</item>{NS}<item>{NS}<k>1{NS}</k>{NS}</item>{NS}</list>{NS}<text>{{\"a\": 1}}{NS}</text>"
    _, calls, _ = _run(_block(_invoke("f", body)), 5)
    assert calls == [("f", {"n": 3.5, "flag": False, "none": None, "s": "hello world", "list": ["x", {"k": 1}],
                            "text": '{"a": 1}'})]


def test_malformed_blocks_come_back_as_content_and_ids_count_up():
    bad = _block(f'{NS}<invoke name="f">{NS}<a>1{NS}</b>{NS}</invoke>')                 # mismatched closing tag
    content, calls, _ = _run("x" + bad + "y", 4)
    assert calls == [] and content == "x" + bad + "y"
    dup = _block(_invoke("f", f"{NS}<a>1{NS}</a>{NS}<a>2{NS}</a>"))                        # a key twice
    assert _run(dup, 9)[1] == []
    p = rt.ToolParser(rt.ToolFormat.NsXml, "id")
    ev = p.feed((_block(_invoke("a", "")) + _block(_invoke("b", ""))).encode()) + p.finish()
    assert [(e[1], e[2], e[3]) for e in ev if e[0] == "tool_call"] == [(0, "id0", "a"), (1, "id1", "b")]
    # an unterminated block is content at the end of the stream
    content, calls, _ = _run("hi " + NS + "<tool_call>" + _invoke("f", ""), 6)
    assert calls == [] and content.startswith("hi " + NS + "<tool_call>")
    # another namespace marker
    q = rt.ToolParser(rt.ToolFormat.NsXml, "c")
    q.set_namespace("@@")
    ev = q.feed(b'@@<tool_call>@@<invoke name="g">@@<v>7@@</v>@@</invoke>@@</tool_call>') + q.finish()
    assert [(e[3], e[4]) for e in ev if e[0] == "tool_call"] == [("g", '{"v":7}')] or \
        [(e[3], json.loads(e[4])) for e in ev if e[0] == "tool_call"] == [("g", {"v": 7})]


def test_dsml_spaced_dialect_and_namespaced_names():
    M = "｜DSML｜"
    text = (f"Checking.\n\n<{M} calls>\n<{M} invoke name=\"weather::get_forecast\">\n"
            f"<{M} parameter name=\"city\" string=\"true\">Paris</{M} parameter>\n"
            f"<{M} parameter name=\"days\" string=\"false\">3</{M} parameter>\n</{M} invoke>\n</{M} calls>")
    for step in (1, 5, 4096):
        p = rt.ToolParser(rt.ToolFormat.Dsml, "c")
        p.set_dsml_spaced(True)
        ev, data = [], text.encode()
        for i in range(0, len(data), step):
            ev += p.feed(data[i:i + step])
        ev += p.finish()
        calls = [(e[3], json.loads(e[4])) for e in ev if e[0] == "tool_call"]
        content = b"".join(e[1] for e in ev if e[0] == "content").decode()
        assert calls == [("get_forecast", {"city": "Paris", "days": 3})], step
        assert content == "Checking.", (step, content)
    # the unspaced dialect does not take the spaced tags for calls
    p = rt.ToolParser(rt.ToolFormat.Dsml, "c")
    ev = p.feed(text.encode()) + p.finish()
    assert not [e for e in ev if e[0] == "tool_call"]
