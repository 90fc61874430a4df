"""Template-less prompt renderer (DeepSeek-V4 style layout): turn structure, merging, tools, DSML calls, modes."""
import json

import pytest

from dgpp_b200.runtime import rt

BOS, EOS = "<｜begin▁of▁sentence｜>", "<｜end▁of▁sentence｜>"
U, A = "<｜User｜>", "<｜Assistant｜>"


def render(**g):
    return rt.deepseek_prompt(json.dumps(g))


def test_basic_turns_and_generation_header():
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "Hi"}]
    assert render(messages=msgs) == f"{BOS}Be brief.{U}Hi{A}<think>"
    assert render(messages=msgs, enable_thinking=False) == f"{BOS}Be brief.{U}Hi{A}</think>"
    assert render(messages=msgs, add_generation_prompt=False) == f"{BOS}Be brief.{U}Hi"
    # a conversation ending in a system message gets no header
    assert render(messages=msgs + [{"role": "system", "content": "Stop."}]) == f"{BOS}Be brief.{U}HiStop."


def test_history_reasoning_is_dropped_except_for_the_last_assistant_turn():
    msgs = [{"role": "user", "content": "a"},
            {"role": "assistant", "content": "A1", "reasoning_content": "r1"},
            {"role": "user", "content": "b"},
            {"role": "assistant", "content": "A2", "reasoning_content": "r2"},
            {"role": "user", "content": "c"}]
    got = render(messages=msgs)
    assert got == f"{BOS}{U}a{A}<think></think>A1{EOS}{U}b{A}<think>r2</think>A2{EOS}{U}c{A}<think>"
    keep = render(messages=msgs, clear_thinking=False)
    assert "<think>r1</think>A1" in keep
    chat = render(messages=msgs, enable_thinking=False)
    assert chat == f"{BOS}{U}a{A}</think>A1{EOS}{U}b{A}</think>A2{EOS}{U}c{A}</think>"


def test_user_merge_tool_results_and_tools_block():
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}}]
    msgs = [{"role": "user", "content": "one"}, {"role": "user", "content": [{"type": "text", "text": "two"}]},
            {"role": "assistant", "content": "", "reasoning_content": "why",
             "tool_calls": [{"id": "1", "type": "function", "function": {"name": "f", "arguments": "{\"x\": 1, \"s\": \"v\"}"}}]},
            {"role": "tool", "tool_call_id": "1", "content": "42"},
            {"role": "user", "content": "and?"}]
    got = render(messages=msgs, tools=tools)
    assert got.startswith(f'{BOS}## Tools\n{{"name":"f","parameters":{{"type":"object"}}}}\n{U}one\n\ntwo{A}')
    # tools present -> earlier reasoning is kept
    assert "<think>why</think>" in got
    assert ('<｜DSML｜tool_calls>\n<｜DSML｜invoke name="f">\n<｜DSML｜parameter name="x" string="false">1</｜DSML｜parameter>\n'
            '<｜DSML｜parameter name="s" string="true">v</｜DSML｜parameter>\n</｜DSML｜invoke>\n</｜DSML｜tool_calls>' + EOS) in got
    assert got.endswith(f"{U}<tool_result>42</tool_result>\n\nand?{A}<think>")


def test_effort_and_errors():
    msgs = [{"role": "user", "content": "q"}]
    low = render(messages=msgs, reasoning_effort="medium")
    high = render(messages=msgs, reasoning_effort="high")
    mx = render(messages=msgs, reasoning_effort="max")
    assert low == f"{BOS}{U}q{A}<think>" and high.startswith(BOS + "Reasoning effort: high") and mx != high
    assert render(messages=msgs, reasoning_effort="high", enable_thinking=False) == f"{BOS}{U}q{A}</think>"
    with pytest.raises(ValueError):
        render(messages=msgs, reasoning_effort="extreme")
    with pytest.raises(ValueError):
        render(messages=[{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "x"}}]}])
    with pytest.raises(ValueError):
        render(messages=[{"role": "narrator", "content": "x"}])
