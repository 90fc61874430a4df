"""Constrained decoding of tool calls: the byte machine behind the vocabulary masks.
(Model of the reference's tests/test_tool_grammar.cpp.)"""
import json

import numpy as np
import pytest

from dgpp_b200.runtime import rt

TOOLS = json.dumps([
    {"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}},
        "required": ["city"], "additionalProperties": False}}},
    {"type": "function", "function": {"name": "get_time", "parameters": {"type": "object", "properties": {}}}},
])
# vocabulary: the 256 bytes, a few merged tokens, end of sequence
EXTRA = [b"<tool_call>", b"</tool_call>", b'{"name": "', b"get_", b'", "arguments": ', b"weather", b"Oslo", b"<tool"]
VOCAB = [bytes([i]) for i in range(256)] + EXTRA + [b""]
EOS = len(VOCAB) - 1


def allowed(g):
    m = np.asarray(g.mask())
    return {i for i in range(len(VOCAB)) if m[i >> 5] >> (i & 31) & 1}


def feed_bytes(g, text: bytes):
    for b in text:
        assert b in allowed(g), (bytes([b]), text)
        assert g.accept(b)


def test_required_choice_forces_a_valid_call():
    g = rt.ToolGrammar(TOOLS, True, True, VOCAB, [EOS])
    a = allowed(g)
    assert EOS not in a and ord("<") in a and 256 in a and 256 + 7 in a        # "<", "<tool_call>", "<tool"
    assert ord("H") not in a                                                    # no free text when a call is required
    feed_bytes(g, b'<tool_call>\n{"name": "get_')
    assert allowed(g) == {ord("w"), ord("t"), 256 + 5}                          # weather | time
    feed_bytes(g, b"weather")
    assert allowed(g) == {ord('"'), 256 + 4}
    feed_bytes(g, b'", "arguments": {"')
    a = allowed(g)
    assert ord("c") in a and ord("d") in a and ord("x") not in a                # only declared properties
    feed_bytes(g, b'days": ')
    a = allowed(g)
    assert ord("7") in a and ord("-") in a and ord('"') not in a                # integer
    feed_bytes(g, b'3, "city": "Oslo"}')
    assert allowed(g) == {ord("}")}                                             # required done -> closing literal
    assert g.in_call() and not g.complete()
    feed_bytes(g, b"}\n</tool_call>")
    assert g.complete() and g.calls() == 1 and not g.in_call()
    assert allowed(g) == {EOS, ord("\n")}                                       # stop, or a parallel call
    feed_bytes(g, b'\n<tool_call>\n{"name": "get_time", "arguments": {}}\n</tool_call>')
    assert g.calls() == 2 and g.accept(EOS)


def test_required_property_must_be_present_before_the_object_closes():
    g = rt.ToolGrammar(TOOLS, True, False, VOCAB, [EOS])
    feed_bytes(g, b'<tool_call>\n{"name": "get_weather", "arguments": {')
    assert ord("}") not in allowed(g)                                           # "city" is required
    feed_bytes(g, b'"city": "x"}}\n</tool_call>')
    assert allowed(g) == {EOS}                                                  # parallel calls off


def test_auto_choice_leaves_text_free_until_a_call_opens():
    g = rt.ToolGrammar(TOOLS, False, True, VOCAB, [EOS])
    a = allowed(g)
    assert EOS in a and len(a) == len(VOCAB)                                    # everything, stop included
    feed_bytes(g, b"Let me check <b> that.\n<tool")
    a = allowed(g)
    assert ord("_") in a and ord("x") in a and EOS in a                         # "<tool" may still be plain text
    feed_bytes(g, b"_call>")
    a = allowed(g)
    assert a == {ord("\n")} and not g.complete()                                # inside a call: the forced layout
    feed_bytes(g, b'\n{"name": "get_time", "arguments": {}}\n</tool_call>')
    assert g.complete() and g.calls() == 1


def test_named_function_restricts_the_name_and_multibyte_tokens_are_checked_whole():
    g = rt.ToolGrammar(TOOLS, True, True, VOCAB, [EOS], "get_time")
    feed_bytes(g, b'<tool_call>\n{"name": "get_')
    assert allowed(g) == {ord("t")}                                             # "weather" token is not allowed
    g2 = rt.ToolGrammar(TOOLS, True, True, VOCAB, [EOS])
    assert g2.accept(256) and g2.accept(ord("\n")) and g2.accept(256 + 2) and g2.accept(256 + 3) and g2.accept(256 + 5)
    assert g2.accept(256 + 4)                                                   # '", "arguments": ' in one token
    assert not g2.accept(ord("["))                                              # arguments are an object
    with pytest.raises(ValueError):
        rt.ToolGrammar(TOOLS, True, True, VOCAB, [EOS], "nope")
