import json

import pytest

from mllm_b200.parsers import ReasoningParser, ToolCallParser


def test_reasoning_non_stream():
    assert ReasoningParser("qwen3").parse_non_stream("<think>plan</think>\nanswer") == ("plan", "answer")
    assert ReasoningParser("qwen3").parse_non_stream("just text") == (None, "just text")
    assert ReasoningParser("deepseek-r1").parse_non_stream("hidden thoughts</think>ok") == ("hidden thoughts", "ok")
    assert ReasoningParser("deepseek-r1").parse_non_stream("never closes") == ("never closes", "")
    with pytest.raises(ValueError):
        ReasoningParser("nope")


@pytest.mark.parametrize("family,text,want_r,want_a", [
    ("qwen3", "<think>a b c</think>\n\nfinal answer", "a b c", "final answer"),
    ("qwen3", "no reasoning here", "", "no reasoning here"),
    ("deepseek-r1", "thinking...</think>done", "thinking...", "done"),
    ("qwen3-thinking", "<think>x</think>y", "x", "y"),
])
def test_reasoning_stream_any_chunking(family, text, want_r, want_a):
    for step in (1, 2, 3, 5, 100):
        p = ReasoningParser(family)
        r = a = ""
        for i in range(0, len(text), step):
            dr, da = p.parse_stream_chunk(text[i:i + step])
            r, a = r + dr, a + da
        assert (r, a) == (want_r, want_a), step


def test_tool_calls_non_stream():
    text = 'Let me check.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>'
    plain, calls = ToolCallParser("qwen25").parse_non_stream(text)
    assert plain == "Let me check." and len(calls) == 1 and calls[0].name == "get_weather"
    assert json.loads(calls[0].parameters) == {"city": "Paris"}
    d = calls[0].to_openai_dict(streaming=False)
    assert d["type"] == "function" and d["function"]["name"] == "get_weather" and d["id"].startswith("call_")
    plain, calls = ToolCallParser("llama3").parse_non_stream('<|python_tag|>{"name": "f", "parameters": {"x": 1}}')
    assert calls[0].name == "f" and json.loads(calls[0].parameters) == {"x": 1}
    xml = "<tool_call><function=search><parameter=q>cats</parameter><parameter=n>3</parameter></function></tool_call>"
    _, calls = ToolCallParser("qwen3_coder").parse_non_stream(xml)
    assert calls[0].name == "search" and json.loads(calls[0].parameters) == {"q": "cats", "n": 3}
    assert ToolCallParser("hermes").parse_non_stream("plain") == ("plain", [])


@pytest.mark.parametrize("step", [1, 3, 7, 1000])
def test_tool_calls_stream_reassemble(step):
    text = 'Hi <tool_call>\n{"name": "add", "arguments": {"a": 1, "b": [2, 3]}}\n</tool_call> bye'
    p = ToolCallParser("qwen25")
    plain, name, args = "", None, ""
    for i in range(0, len(text), step):
        t, items = p.parse_stream_chunk(text[i:i + step])
        plain += t
        for it in items:
            if it.name:
                name = it.name
            args += it.parameters
    assert name == "add" and json.loads(args) == {"a": 1, "b": [2, 3]} and plain.replace(" ", "") == "Hibye"
