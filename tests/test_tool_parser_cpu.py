"""Streaming tool-call parser: arbitrary chunking, both formats, malformed bodies fall back to content."""
import json
import random

from dgpp_b200.runtime import rt


def run(fmt, text: bytes, cuts):
    p = rt.ToolParser(fmt)
    ev = []
    last = 0
    for c in list(cuts) + [len(text)]:
        ev += p.feed(text[last:c])
        last = c
    ev += p.finish()
    content = b"".join(e[1] for e in ev if e[0] == "content")
    calls = [e[1:] for e in ev if e[0] == "tool_call"]
    return content, calls


JSON_TEXT = (b'Let me check.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris", "days": 3}}\n</tool_call>\n'
             b'<tool_call>{"name": "noop"}</tool_call> done <tool_ca not a tag')


def test_json_tags_any_chunking():
    want_calls = [(0, "call_0", "get_weather", '{"city":"Paris","days":3}'), (1, "call_1", "noop", "{}")]
    rnd = random.Random(0)
    for trial in range(50):
        cuts = sorted(rnd.sample(range(1, len(JSON_TEXT)), rnd.randint(0, 30)))
        content, calls = run(rt.ToolFormat.JsonTags, JSON_TEXT, cuts)
        assert calls == want_calls, (trial, calls)
        assert content == b"Let me check.\n done <tool_ca not a tag"
    # byte-at-a-time
    content, calls = run(rt.ToolFormat.JsonTags, JSON_TEXT, range(1, len(JSON_TEXT)))
    assert calls == want_calls


def test_content_is_released_early():
    p = rt.ToolParser(rt.ToolFormat.JsonTags)
    assert p.feed(b"hello <to") == [("content", b"hello ")]          # "<to" could start a tag: held back
    assert p.feed(b"day>") == [("content", b"<today>")]
    assert p.feed(b"<tool_call>{") == []
    assert p.feed(b'"name":"f","arguments":"{\\"a\\":1}"}</tool_call>') == [("tool_call", 0, "call_0", "f", '{"a":1}')]


def test_malformed_call_becomes_content():
    text = b'<tool_call>{"nam": 1}</tool_call> tail <tool_call>{"name": "x"'
    content, calls = run(rt.ToolFormat.JsonTags, text, [5, 17])
    assert calls == [] and content == text


def test_arg_tags_format():
    text = (b"ok <tool_call>search\n<arg_key>query</arg_key>\n<arg_value>red pandas</arg_value>\n"
            b"<arg_key>limit</arg_key><arg_value>5</arg_value>\n<arg_key>opts</arg_key><arg_value>{\"a\": [1, 2]}</arg_value>"
            b"</tool_call>")
    for cuts in ([], [10, 40, 41, 90], range(1, len(text))):
        content, calls = run(rt.ToolFormat.ArgTags, text, cuts)
        assert content == b"ok "
        assert len(calls) == 1 and calls[0][2] == "search"
        assert json.loads(calls[0][3]) == {"query": "red pandas", "limit": 5, "opts": {"a": [1, 2]}}


def test_tools_block():
    s = rt.render_tools_block(json.dumps([{"type": "function", "function": {"name": "f"}}]))
    assert s.startswith("<tools>\n") and s.endswith("</tools>") and '"name":"f"' in s


def test_dsml_calls_in_any_chunking():
    text = ('I will look.\n\n<｜DSML｜tool_calls>\n<｜DSML｜invoke name="get_weather">\n'
            '<｜DSML｜parameter name="city" string="true">Oslo</｜DSML｜parameter>\n'
            '<｜DSML｜parameter name="days" string="false">3</｜DSML｜parameter>\n</｜DSML｜invoke>\n'
            '<｜DSML｜invoke name="now">\n</｜DSML｜invoke>\n</｜DSML｜tool_calls>').encode()
    rnd = random.Random(1)
    for trial in range(40):
        cuts = sorted(rnd.sample(range(1, len(text)), rnd.randint(0, 40)))
        content, calls = run(rt.ToolFormat.Dsml, text, cuts)
        assert content == b"I will look.", (cuts, content)
        assert [(c[0], c[2], json.loads(c[3])) for c in calls] == [(0, "get_weather", {"city": "Oslo", "days": 3}),
                                                                    (1, "now", {})], cuts
