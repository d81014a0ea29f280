"""Tool-call and reasoning parsers: whole texts and streams cut at arbitrary places give the same result."""
import json
import os

import pytest

from lightllm_b200.server.function_call_parser import FunctionCallParser
from lightllm_b200.server.reasoning_parser import ReasoningParser

TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {}}},
         {"type": "function", "function": {"name": "add", "parameters": {}}}]


def _stream(parser, text, step):
    normal, calls = "", []
    for i in range(0, len(text), step):
        n, c = parser.parse_stream_chunk(text[i:i + step])
        normal += n
        calls += c
    return normal, calls


@pytest.mark.parametrize("step", [1, 3, 7, 1000])
def test_qwen_tool_calls_whole_and_streamed(step):
    text = ('I will check.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>\n'
            '<tool_call>\n{"name": "add", "arguments": {"a": 1, "b": 2}}\n</tool_call>')
    normal, calls = FunctionCallParser(TOOLS, "qwen25").parse_non_stream(text)
    assert normal == "I will check." and [c.name for c in calls] == ["get_weather", "add"]
    assert json.loads(calls[0].parameters) == {"city": "Paris"} and [c.tool_index for c in calls] == [0, 1]
    s_normal, s_calls = _stream(FunctionCallParser(TOOLS, "qwen25"), text, step)
    assert s_normal.strip() == "I will check."
    assert _assemble(s_calls) == [(c.name, json.loads(c.parameters)) for c in calls]


def _assemble(deltas):
    """What an OpenAI client builds from the deltas: the first delta of a tool index names the function, the
    argument pieces are concatenated."""
    by = {}
    for d in deltas:
        slot = by.setdefault(d.tool_index, {"name": None, "args": ""})
        if d.name is not None:
            assert slot["name"] is None, "the function name is sent once per call"
            slot["name"] = d.name
        else:
            assert slot["name"] is not None, "argument pieces only follow the delta that names the function"
        slot["args"] += d.parameters
    return [(by[i]["name"], json.loads(by[i]["args"])) for i in sorted(by)]


@pytest.mark.parametrize("step", [1, 2, 5, 11])
def test_json_arguments_stream_piece_by_piece(step):
    text = ('<tool_call>{"name": "get_weather", "arguments": {"city": "Pa\\"ris}", "days": [1, {"k": "]"}], '
            '"note": "x"}}</tool_call> done <tool_call>{"name":"add","arguments":{"a":1,"b":2}}</tool_call>')
    normal, deltas = _stream(FunctionCallParser(TOOLS, "qwen25"), text, step)
    assert normal.strip() == "done"
    assert _assemble(deltas) == [("get_weather", {"city": 'Pa"ris}', "days": [1, {"k": "]"}], "note": "x"}),
                                 ("add", {"a": 1, "b": 2})]
    first = [d for d in deltas if d.tool_index == 0]
    assert first[0].name == "get_weather" and first[0].parameters == ""      # name first, empty arguments
    if step <= 5:
        assert len(first) > 4                                                # the arguments came in several pieces
    # the closing brace of the call object and the end marker never leak into the arguments
    assert "".join(d.parameters for d in first).endswith('"note": "x"}')


@pytest.mark.parametrize("step", [1, 3, 1000])
def test_bodies_that_cannot_be_streamed_are_emitted_whole(step, monkeypatch):
    monkeypatch.setenv("LIGHTLLM_ENABLE_TOOL_NAME_CHECK", "1")
    cases = [("mistral", '[TOOL_CALLS][{"name":"add","arguments":{"a":1}},{"name":"get_weather","arguments":{"city":"x"}}]',
              [("add", {"a": 1}), ("get_weather", {"city": "x"})]),
             ("qwen25", '<tool_call>{"name":"add","arguments":"{\\"a\\": 1}"}</tool_call>', [("add", {"a": 1})]),
             ("qwen25", '<tool_call>{"arguments":{"a": 1},"name":"add"}</tool_call>', [("add", {"a": 1})]),
             ("llama3", '<|python_tag|>{"name": "add", "parameters": {"a": 5, "b": 7}} trailing', [("add", {"a": 5, "b": 7})]),
             ("qwen25", '<tool_call>{"name":"rm_rf","arguments":{"a":1}}</tool_call>tail', [])]
    for fmt, text, want in cases:
        normal, deltas = _stream(FunctionCallParser(TOOLS, fmt), text, step)
        assert _assemble(deltas) == want, (fmt, text)


def test_other_call_syntaxes_and_unknown_tools():
    p = FunctionCallParser(TOOLS, "llama3")
    normal, calls = p.parse_non_stream('<|python_tag|>{"name": "add", "parameters": {"a": 2, "b": 3}}')
    assert normal == "" and calls[0].name == "add" and json.loads(calls[0].parameters) == {"a": 2, "b": 3}
    p = FunctionCallParser(TOOLS, "mistral")
    _, calls = p.parse_non_stream('[TOOL_CALLS][{"name": "get_weather", "arguments": {"city": "Rome"}}]')
    assert calls[0].name == "get_weather"
    p = FunctionCallParser(TOOLS, "deepseekv3")
    body = ("<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>add\n```json\n{\"a\": 1, \"b\": 1}\n```"
            "<｜tool▁call▁end｜><｜tool▁calls▁end｜>")
    _, calls = p.parse_non_stream("ok " + body)
    assert calls[0].name == "add" and json.loads(calls[0].parameters) == {"a": 1, "b": 1}
    # a call to a function that was not offered passes, unless the name check is switched on
    undeclared = '<tool_call>{"name": "rm_rf", "arguments": {}}</tool_call>'
    _, calls = FunctionCallParser(TOOLS, "qwen25").parse_non_stream(undeclared)
    assert [c.name for c in calls] == ["rm_rf"]
    os.environ["LIGHTLLM_ENABLE_TOOL_NAME_CHECK"] = "1"
    try:
        _, calls = FunctionCallParser(TOOLS, "qwen25").parse_non_stream(undeclared)
    finally:
        del os.environ["LIGHTLLM_ENABLE_TOOL_NAME_CHECK"]
    assert calls == []
    assert not FunctionCallParser(TOOLS, "qwen25").has_tool_call("plain text")
    with pytest.raises(ValueError):
        FunctionCallParser(TOOLS, "nope")


@pytest.mark.parametrize("step", [1, 4, 1000])
def test_reasoning_split(step):
    text = "<think>first I add\nthen I check</think>The answer is 4."
    r, a = ReasoningParser("qwen3").parse_non_stream(text)
    assert r.strip() == "first I add\nthen I check" and a.strip() == "The answer is 4."
    p = ReasoningParser("qwen3")
    rs, ans = "", ""
    for i in range(0, len(text), step):
        r1, a1 = p.parse_stream_chunk(text[i:i + step])
        rs += r1 or ""
        ans += a1
    assert rs.strip() == "first I add\nthen I check" and ans.strip() == "The answer is 4."
    # a model whose template already opened the block
    r, a = ReasoningParser("deepseek-r1").parse_non_stream("thinking...</think>done")
    assert r.strip() == "thinking..." and a.strip() == "done"
    # no reasoning at all
    r, a = ReasoningParser("qwen3").parse_non_stream("just an answer")
    assert not r and a == "just an answer"
