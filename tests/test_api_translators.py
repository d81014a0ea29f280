"""Anthropic Messages and OpenAI Responses routes as translations of the chat-completions route: request mapping,
answer mapping and the re-cut event streams, on hand-made chat responses / chunks (a random-weight model emits no
tool calls, so the mappings are tested directly).  Reference: lightllm/server/api_anthropic.py,
lightllm/server/api_responses.py."""
import asyncio
import json

from lightllm_b200.server import api_anthropic as an


def _events(raw_list):
    out = []
    for raw in raw_list:
        head, data = raw.decode().strip().split("\n", 1)
        assert head.startswith("event: ") and data.startswith("data: ")
        d = json.loads(data[6:])
        assert d["type"] == head[7:]
        out.append(d)
    return out


async def _collect(agen):
    return [x async for x in agen]


async def _aiter(items):
    for i in items:
        yield i


def test_anthropic_request_mapping():
    body = {"model": "m", "max_tokens": 64, "system": [{"type": "text", "text": "be brief"}], "temperature": 0,
            "stop_sequences": ["END"], "top_k": 5,
            "tools": [{"name": "get_weather", "description": "d", "input_schema": {"type": "object"}}],
            "tool_choice": {"type": "tool", "name": "get_weather", "disable_parallel_tool_use": True},
            "thinking": {"type": "enabled", "budget_tokens": 100},
            "messages": [
                {"role": "user", "content": "weather in Paris?"},
                {"role": "assistant", "content": [{"type": "thinking", "thinking": "need the tool"},
                                                  {"type": "text", "text": "let me check"},
                                                  {"type": "tool_use", "id": "toolu_1", "name": "get_weather",
                                                   "input": {"city": "Paris"}}]},
                {"role": "user", "content": [{"type": "tool_result", "tool_use_id": "toolu_1",
                                              "content": [{"type": "text", "text": "12 C"}]},
                                             {"type": "text", "text": "and Rome?"}]}]}
    chat = an.to_chat_request(body)
    assert chat["messages"][0] == {"role": "system", "content": "be brief"}
    assert chat["messages"][1] == {"role": "user", "content": "weather in Paris?"}
    a = chat["messages"][2]
    assert a["role"] == "assistant" and a["content"] == "let me check" and a["reasoning_content"] == "need the tool"
    assert a["tool_calls"][0]["id"] == "toolu_1" and json.loads(a["tool_calls"][0]["function"]["arguments"]) == \
        {"city": "Paris"}
    assert chat["messages"][3] == {"role": "tool", "tool_call_id": "toolu_1", "content": "12 C"}
    assert chat["messages"][4] == {"role": "user", "content": "and Rome?"}
    assert chat["do_sample"] is False and chat["stop"] == ["END"] and chat["top_k"] == 5 and chat["max_tokens"] == 64
    assert chat["tools"][0]["function"]["parameters"] == {"type": "object"}
    assert chat["tool_choice"] == {"type": "function", "function": {"name": "get_weather"}}
    assert chat["parallel_tool_calls"] is False and chat["chat_template_kwargs"]["enable_thinking"] is True
    assert an.to_chat_request({"messages": [{"role": "user", "content": "x"}], "tools": [{"name": "f"}],
                               "tool_choice": {"type": "any"}})["tool_choice"] == "required"
    from lightllm_b200.server.api_models import ChatCompletionRequest

    ChatCompletionRequest(**chat)             # the dict is a valid chat request


def test_anthropic_answer_mapping():
    resp = {"choices": [{"finish_reason": "tool_calls", "message": {
        "role": "assistant", "content": "checking", "reasoning_content": "hmm",
        "tool_calls": [{"id": "call_abc", "type": "function",
                        "function": {"name": "get_weather", "arguments": "{\"city\": \"Rome\"}"}}]}}],
        "usage": {"prompt_tokens": 30, "completion_tokens": 9, "prompt_tokens_details": {"cached_tokens": 16}}}
    m = an.chat_response_to_message(resp, "m", "msg_1")
    assert [b["type"] for b in m["content"]] == ["thinking", "text", "tool_use"]
    assert m["content"][2] == {"type": "tool_use", "id": "toolu_abc", "name": "get_weather", "input": {"city": "Rome"}}
    assert m["stop_reason"] == "tool_use" and m["usage"]["input_tokens"] == 30 and m["usage"]["output_tokens"] == 9
    assert m["usage"]["cache_read_input_tokens"] == 16 and m["id"] == "msg_1" and m["role"] == "assistant"
    m = an.chat_response_to_message({"choices": [{"finish_reason": "length", "message": {"content": ""}}]}, "m")
    assert m["content"] == [{"type": "text", "text": ""}] and m["stop_reason"] == "max_tokens"


def test_anthropic_event_stream():
    def ch(delta=None, finish=None, usage=None):
        c = {"id": "x", "choices": [] if delta is None and finish is None else
             [{"index": 0, "delta": delta or {}, "finish_reason": finish}]}
        if usage:
            c["usage"] = usage
        return c

    chunks = [ch({"role": "assistant", "reasoning_content": "let "}), ch({"reasoning_content": "me think"}),
              ch({"content": "I will "}), ch({"content": "look it up"}),
              ch({"tool_calls": [{"index": 0, "id": "call_1", "function": {"name": "get_weather", "arguments": ""}}]}),
              ch({"tool_calls": [{"index": 0, "function": {"arguments": "{\"city\": "}}]}),
              ch({"tool_calls": [{"index": 0, "function": {"arguments": "\"Rome\"}"}}]}),
              ch({"tool_calls": [{"index": 1, "id": "call_2", "function": {"name": "get_time", "arguments": "{}"}}]}),
              ch({}, finish="tool_calls"), ch(usage={"prompt_tokens": 21, "completion_tokens": 14})]
    ev = _events(asyncio.run(_collect(an.chat_chunks_to_events(_aiter(chunks), "m", "msg_9"))))
    kinds = [e["type"] for e in ev]
    assert kinds[0] == "message_start" and kinds[-2:] == ["message_delta", "message_stop"]
    starts = [e for e in ev if e["type"] == "content_block_start"]
    assert [s["content_block"]["type"] for s in starts] == ["thinking", "text", "tool_use", "tool_use"]
    assert [s["index"] for s in starts] == [0, 1, 2, 3]
    assert starts[2]["content_block"]["id"] == "toolu_1" and starts[3]["content_block"]["name"] == "get_time"
    stops = [e["index"] for e in ev if e["type"] == "content_block_stop"]
    assert stops == [0, 1, 2, 3]
    # every block is closed before the next one opens
    order = [(e["type"], e["index"]) for e in ev if e["type"] in ("content_block_start", "content_block_stop")]
    assert order == [("content_block_start", 0), ("content_block_stop", 0), ("content_block_start", 1),
                     ("content_block_stop", 1), ("content_block_start", 2), ("content_block_stop", 2),
                     ("content_block_start", 3), ("content_block_stop", 3)]
    deltas = [e for e in ev if e["type"] == "content_block_delta"]
    assert "".join(d["delta"]["thinking"] for d in deltas if d["delta"]["type"] == "thinking_delta") == "let me think"
    assert "".join(d["delta"]["text"] for d in deltas if d["delta"]["type"] == "text_delta") == "I will look it up"
    args2 = "".join(d["delta"]["partial_json"] for d in deltas if d["index"] == 2)
    assert json.loads(args2) == {"city": "Rome"}
    md = ev[-2]
    assert md["delta"]["stop_reason"] == "tool_use" and md["usage"] == {"input_tokens": 21, "output_tokens": 14}
    # nothing produced at all: still a well-formed message with one empty text block
    ev = _events(asyncio.run(_collect(an.chat_chunks_to_events(_aiter([ch({}, finish="stop")]), "m"))))
    assert [e["type"] for e in ev] == ["message_start", "content_block_start", "content_block_stop", "message_delta",
                                       "message_stop"]


def test_sse_reader():
    parts = [b'data: {"a": 1}\n\nda', b'ta: {"b": 2}\n\n', b": keep-alive\n\n", b"data: [DONE]\n\ndata: {\"c\": 3}\n\n"]
    got = asyncio.run(_collect(an.sse_to_chunks(_aiter(parts))))
    assert got == [{"a": 1}, {"b": 2}]


def test_responses_request_mapping():
    from lightllm_b200.server import api_responses as rs
    from lightllm_b200.server.api_models import ChatCompletionRequest

    body = {"model": "m", "instructions": "be brief", "max_output_tokens": 32, "temperature": 0.5,
            "tools": [{"type": "function", "name": "get_weather", "description": "d", "parameters": {"type": "object"}},
                      {"type": "web_search"}],
            "tool_choice": {"type": "function", "name": "get_weather"},
            "text": {"format": {"type": "json_schema", "name": "out", "schema": {"type": "object"}, "strict": True}},
            "reasoning": {"effort": "high"},
            "input": [
                {"role": "user", "content": [{"type": "input_text", "text": "weather "}, {"type": "input_text", "text": "in Paris?"}]},
                {"type": "reasoning", "summary": [{"type": "summary_text", "text": "need the tool"}]},
                {"type": "function_call", "call_id": "call_1", "name": "get_weather", "arguments": "{\"city\": \"Paris\"}"},
                {"type": "function_call_output", "call_id": "call_1", "output": "12 C"},
                {"type": "message", "role": "developer", "content": "answer in French"}]}
    chat = rs.to_chat_request(body)
    m = chat["messages"]
    assert m[0] == {"role": "system", "content": "be brief"} and m[1] == {"role": "user", "content": "weather in Paris?"}
    assert m[2]["role"] == "assistant" and m[2]["reasoning_content"] == "need the tool"
    assert m[2]["tool_calls"][0]["id"] == "call_1" and m[2]["tool_calls"][0]["function"]["name"] == "get_weather"
    assert m[3] == {"role": "tool", "tool_call_id": "call_1", "content": "12 C"}
    assert m[4] == {"role": "system", "content": "answer in French"}
    assert len(chat["tools"]) == 1 and chat["tool_choice"]["function"]["name"] == "get_weather"
    assert chat["response_format"]["json_schema"]["schema"] == {"type": "object"} and chat["max_tokens"] == 32
    assert chat["chat_template_kwargs"]["enable_thinking"] is True and chat["do_sample"] is True
    ChatCompletionRequest(**chat)
    assert rs.to_chat_request({"input": "hi"})["messages"] == [{"role": "user", "content": "hi"}]


def test_responses_answer_and_event_stream():
    from lightllm_b200.server import api_responses as rs

    body = {"model": "m", "input": "x", "max_output_tokens": 8}
    resp = {"created": 5, "choices": [{"finish_reason": "tool_calls", "message": {
        "content": "", "reasoning_content": "hmm",
        "tool_calls": [{"id": "call_7", "function": {"name": "f", "arguments": "{\"a\": 1}"}}]}}],
        "usage": {"prompt_tokens": 10, "completion_tokens": 4}}
    r = rs.chat_response_to_response(resp, body, "resp_1")
    assert [o["type"] for o in r["output"]] == ["reasoning", "function_call"] and r["status"] == "completed"
    assert r["output"][1]["call_id"] == "call_7" and r["output"][1]["arguments"] == "{\"a\": 1}"
    assert r["usage"]["total_tokens"] == 14 and r["id"] == "resp_1" and r["created_at"] == 5
    cut = rs.chat_response_to_response({"choices": [{"finish_reason": "length", "message": {"content": "abc"}}]}, body)
    assert cut["status"] == "incomplete" and cut["incomplete_details"] == {"reason": "max_output_tokens"}
    assert cut["output"][0]["content"][0]["text"] == "abc" and cut["output"][0]["status"] == "incomplete"

    def ch(delta=None, finish=None, usage=None):
        c = {"choices": [] if delta is None and finish is None else [{"delta": delta or {}, "finish_reason": finish}]}
        if usage:
            c["usage"] = usage
        return c

    chunks = [ch({"reasoning_content": "think"}), ch({"content": "Hel"}), ch({"content": "lo"}),
              ch({"tool_calls": [{"index": 0, "id": "call_1", "function": {"name": "f", "arguments": ""}}]}),
              ch({"tool_calls": [{"index": 0, "function": {"arguments": "{\"a\":"}}]}),
              ch({"tool_calls": [{"index": 0, "function": {"arguments": " 1}"}}]}),
              ch({}, finish="tool_calls"), ch(usage={"prompt_tokens": 3, "completion_tokens": 9})]
    ev = _events(asyncio.run(_collect(rs.chat_chunks_to_events(_aiter(chunks), body, "resp_2"))))
    kinds = [e["type"] for e in ev]
    assert kinds[:2] == ["response.created", "response.in_progress"] and kinds[-1] == "response.completed"
    assert [e["sequence_number"] for e in ev] == list(range(len(ev)))
    added = [e for e in ev if e["type"] == "response.output_item.added"]
    assert [a["item"]["type"] for a in added] == ["reasoning", "message", "function_call"]
    assert [a["output_index"] for a in added] == [0, 1, 2]
    done = [e for e in ev if e["type"] == "response.output_item.done"]
    assert done[1]["item"]["content"][0]["text"] == "Hello" and done[2]["item"]["arguments"] == "{\"a\": 1}"
    assert "".join(e["delta"] for e in ev if e["type"] == "response.output_text.delta") == "Hello"
    assert [e["text"] for e in ev if e["type"] == "response.output_text.done"] == ["Hello"]
    final = ev[-1]["response"]
    assert final["status"] == "completed" and [o["type"] for o in final["output"]] == ["reasoning", "message",
                                                                                      "function_call"]
    assert final["usage"]["input_tokens"] == 3 and final["usage"]["output_tokens"] == 9
    # items are closed in order: every added item is done before the next is added
    order = [(e["type"].rsplit(".", 1)[1], e["output_index"]) for e in ev
             if e["type"] in ("response.output_item.added", "response.output_item.done")]
    assert order == [("added", 0), ("done", 0), ("added", 1), ("done", 1), ("added", 2), ("done", 2)]
    ev = _events(asyncio.run(_collect(rs.chat_chunks_to_events(_aiter([ch({"content": "x"}, finish="length")]), body))))
    assert ev[-1]["type"] == "response.incomplete" and ev[-1]["response"]["status"] == "incomplete"
