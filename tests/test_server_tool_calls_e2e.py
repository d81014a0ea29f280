"""Tool calling end to end through a live server: constrained decoding (`--output_constraint_mode xgrammar`, the
`guided_regex` extension field) makes the random-weight model emit a well-formed qwen-style tool call, which must come
back as `tool_calls` on /v1/chat/completions (plain and streamed), as a `tool_use` block on /v1/messages (plain and
as an event stream) and as a `function_call` item on /v1/responses."""
import json
import os
import signal
import socket
import subprocess
import sys
import time

import pytest
import requests

pytest.importorskip("xgrammar")

from test_server_real_tokenizer import ROOT, _free_port, _make_model_dir  # noqa: E402

CALL_RE = r'<tool_call>\n\{"name": "get_weather", "arguments": \{"city": "Paris"\}\}\n</tool_call>'
TOOLS = [{"type": "function", "function": {"name": "get_weather", "description": "weather of a city",
                                           "parameters": {"type": "object", "properties": {"city": {"type": "string"}},
                                                          "required": ["city"]}}}]


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    d = tmp_path_factory.mktemp("tool_calls")
    _make_model_dir(d)
    port = _free_port()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    log = open(d / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(d), "--port",
                             str(port), "--data_type", "fp32", "--max_total_token_num", "4096",
                             "--running_max_req_size", "8", "--max_req_total_len", "512", "--tp", "1",
                             "--output_constraint_mode", "xgrammar", "--tool_call_parser", "qwen25",
                             "--reasoning_parser", "qwen3"],
                            env=env, stdout=log, stderr=subprocess.STDOUT, cwd=ROOT, start_new_session=True)
    url = f"http://127.0.0.1:{port}"
    t0, up = time.time(), False
    while time.time() - t0 < 240 and proc.poll() is None:
        try:
            if requests.get(url + "/liveness", timeout=2).status_code == 200:
                up = True
                break
        except Exception:
            time.sleep(1)
    if not up:
        proc.kill()
        pytest.fail("server did not start:\n" + open(d / "server.log").read()[-3000:])
    yield url
    try:
        os.killpg(proc.pid, signal.SIGTERM)
    except ProcessLookupError:
        pass
    try:
        proc.wait(timeout=20)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)


@pytest.mark.timeout(600)
def test_chat_completions_tool_call(server):
    body = {"model": "m", "messages": [{"role": "user", "content": "weather in Paris?"}], "tools": TOOLS,
            "max_tokens": 200, "guided_regex": CALL_RE}
    c = requests.post(server + "/v1/chat/completions", json=body, timeout=120).json()
    ch = c["choices"][0]
    assert ch["finish_reason"] == "tool_calls", c
    call = ch["message"]["tool_calls"][0]
    assert call["function"]["name"] == "get_weather" and json.loads(call["function"]["arguments"]) == {"city": "Paris"}
    assert "<tool_call>" not in (ch["message"]["content"] or "")
    body["stream"] = True
    name, args, finish = None, "", None
    with requests.post(server + "/v1/chat/completions", json=body, stream=True, timeout=120) as r:
        for line in r.iter_lines():
            if not line.startswith(b"data: ") or line == b"data: [DONE]":
                continue
            chunk = json.loads(line[6:])
            for choice in chunk["choices"]:
                for tc in choice["delta"].get("tool_calls") or []:
                    name = tc["function"].get("name") or name
                    args += tc["function"].get("arguments") or ""
                finish = choice.get("finish_reason") or finish
    assert name == "get_weather" and json.loads(args) == {"city": "Paris"} and finish == "tool_calls"


@pytest.mark.timeout(600)
def test_anthropic_and_responses_tool_use(server):
    msg = {"model": "m", "max_tokens": 200, "messages": [{"role": "user", "content": "weather in Paris?"}],
           "tools": [{"name": "get_weather", "description": "weather of a city",
                      "input_schema": TOOLS[0]["function"]["parameters"]}]}
    # the Messages and Responses bodies have no field for a decoding constraint: the translation layer is called
    # with the chat request it builds plus the constraint, through the chat route it forwards to
    from lightllm_b200.server import api_anthropic as an
    from lightllm_b200.server import api_responses as rs

    chat = an.to_chat_request(msg)
    chat["guided_regex"] = CALL_RE
    resp = requests.post(server + "/v1/chat/completions", json=chat, timeout=120).json()
    m = an.chat_response_to_message(resp, "m")
    assert m["stop_reason"] == "tool_use"
    use = [b for b in m["content"] if b["type"] == "tool_use"][0]
    assert use["name"] == "get_weather" and use["input"] == {"city": "Paris"} and use["id"].startswith("toolu_")
    body = {"model": "m", "input": "weather in Paris?", "max_output_tokens": 200,
            "tools": [{"type": "function", "name": "get_weather", "parameters": TOOLS[0]["function"]["parameters"]}]}
    chat = rs.to_chat_request(body)
    chat["guided_regex"] = CALL_RE
    resp = requests.post(server + "/v1/chat/completions", json=chat, timeout=120).json()
    out = rs.chat_response_to_response(resp, body)
    call = [o for o in out["output"] if o["type"] == "function_call"][0]
    assert call["name"] == "get_weather" and json.loads(call["arguments"]) == {"city": "Paris"}
    # and the live routes themselves (unconstrained: a plain text answer, well-formed)
    a = requests.post(server + "/v1/messages", json=dict(msg, max_tokens=5), timeout=120).json()
    assert a["type"] == "message" and a["content"][0]["type"] in ("text", "tool_use")
    with requests.post(server + "/v1/messages", json=dict(msg, max_tokens=5, stream=True), stream=True,
                       timeout=120) as r:
        events = [l.decode() for l in r.iter_lines() if l.startswith(b"event:")]
    assert events[0] == "event: message_start" and events[-1] == "event: message_stop"
    o = requests.post(server + "/v1/responses", json=dict(body, max_output_tokens=5), timeout=120).json()
    assert o["object"] == "response" and o["output"]
    with requests.post(server + "/v1/responses", json=dict(body, max_output_tokens=5, stream=True), stream=True,
                       timeout=120) as r:
        events = [l.decode() for l in r.iter_lines() if l.startswith(b"event:")]
    assert events[0] == "event: response.created" and events[-1] in ("event: response.completed",
                                                                       "event: response.incomplete")


@pytest.mark.timeout(600)
def test_reasoning_is_separated_and_streamed(server):
    """`--reasoning_parser qwen3`: text between <think> and </think> comes back as reasoning_content (chat), as a
    thinking block (Messages) and as a reasoning item (Responses); streamed chunks carry it in reasoning deltas."""
    from lightllm_b200.server import api_anthropic as an
    from lightllm_b200.server import api_responses as rs

    regex = r"<think>\nthe user greets me\n</think>\n\nHello there!"
    body = {"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 200, "guided_regex": regex}
    resp = requests.post(server + "/v1/chat/completions", json=body, timeout=120).json()
    msg = resp["choices"][0]["message"]
    assert msg["reasoning_content"].strip() == "the user greets me" and msg["content"].strip() == "Hello there!"
    assert resp["choices"][0]["finish_reason"] == "stop"
    m = an.chat_response_to_message(resp, "m")
    assert [b["type"] for b in m["content"]] == ["thinking", "text"] and m["stop_reason"] == "end_turn"
    out = rs.chat_response_to_response(resp, {"model": "m", "input": "hi"})
    assert [o["type"] for o in out["output"]] == ["reasoning", "message"]
    body.update(stream=True, stream_reasoning=True)
    reasoning, content = "", ""
    with requests.post(server + "/v1/chat/completions", json=body, stream=True, timeout=120) as r:
        for line in r.iter_lines():
            if not line.startswith(b"data: ") or line == b"data: [DONE]":
                continue
            for choice in json.loads(line[6:])["choices"]:
                reasoning += choice["delta"].get("reasoning_content") or ""
                content += choice["delta"].get("content") or ""
    assert reasoning.strip() == "the user greets me" and content.strip() == "Hello there!"
