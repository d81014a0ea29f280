"""Whole server on CPU: launcher -> metric manager, detokenizer, router, one model-rank process,
HTTP worker; tiny random-init Llama; requests over real HTTP."""
import json
import os
import socket
import subprocess
import sys
import time

import pytest
import requests

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = {"model_type": "llama", "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4,
       "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 688, "vocab_size": 1024, "rms_norm_eps": 1e-6,
       "rope_theta": 10000.0, "eos_token_id": 2, "max_position_embeddings": 512, "torch_dtype": "float32"}


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    d = tmp_path_factory.mktemp("tiny_model")
    (d / "config.json").write_text(json.dumps(CFG))
    port = _free_port()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    log = open(d / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(d), "--port",
                             str(port), "--data_type", "fp32", "--max_total_token_num", "4096",
                             "--running_max_req_size", "8", "--max_req_total_len", "256", "--tp", "1"],
                            env=env, stdout=log, stderr=subprocess.STDOUT, cwd=ROOT, start_new_session=True)
    url = f"http://127.0.0.1:{port}"
    t0 = time.time()
    up = False
    while time.time() - t0 < 240:
        if proc.poll() is not None:
            break
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
    import signal

    try:
        os.killpg(proc.pid, signal.SIGTERM)
    except ProcessLookupError:
        pass
    try:
        proc.wait(timeout=20)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)


@pytest.mark.timeout(600)
def test_generate_and_prefix_cache(server):
    body = {"inputs": list(range(5, 45)), "parameters": {"max_new_tokens": 8, "ignore_eos": True, "return_details": True}}
    r1 = requests.post(server + "/generate", json=body, timeout=60).json()
    assert r1["count_output_tokens"] == 8 and r1["finish_reason"] == "length" and r1["prompt_tokens"] == 40
    assert r1["input_usage"] == {"input_text_tokens": 40, "input_audio_tokens": 0, "input_image_tokens": 0}
    assert len(r1["tokens"]) == 8 and all("logprob" in t for t in r1["tokens"])
    r2 = requests.post(server + "/generate", json=body, timeout=60).json()
    assert r2["generated_text"] == r1["generated_text"]        # greedy is deterministic
    assert r2["tokens"][0]["prompt_cache_len"] >= 32           # second run hits the radix cache


@pytest.mark.timeout(600)
def test_stream_and_openai_routes(server):
    body = {"inputs": "hello world", "parameters": {"max_new_tokens": 4, "ignore_eos": True}}
    with requests.post(server + "/generate_stream", json=body, stream=True, timeout=60) as r:
        chunks = [json.loads(l[5:]) for l in r.iter_lines() if l.startswith(b"data:")]
    assert len(chunks) == 4 and chunks[-1]["finished"] and chunks[-1]["finish_reason"] == "length"
    chat = {"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 5, "ignore_eos": True}
    c = requests.post(server + "/v1/chat/completions", json=chat, timeout=60).json()
    assert c["object"] == "chat.completion" and c["usage"]["completion_tokens"] == 5
    assert c["choices"][0]["finish_reason"] == "length"
    chat["stream"] = True
    with requests.post(server + "/v1/chat/completions", json=chat, stream=True, timeout=60) as r:
        lines = [l for l in r.iter_lines() if l.startswith(b"data: ")]
    assert lines[-1] == b"data: [DONE]" and len(lines) == 6
    comp = requests.post(server + "/v1/completions", json={"model": "m", "prompt": "abc", "max_tokens": 3},
                         timeout=60).json()
    assert comp["object"] == "text_completion" and comp["usage"]["completion_tokens"] <= 3


@pytest.mark.timeout(600)
def test_sampling_params_validation_and_misc(server):
    bad = requests.post(server + "/generate", json={"inputs": [1, 2], "parameters": {"max_new_tokens": 0}}, timeout=30)
    assert bad.status_code == 400
    bad = requests.post(server + "/generate", json={"inputs": [1, 5000], "parameters": {}}, timeout=30)
    assert bad.status_code == 400  # token id outside the vocabulary
    two = requests.post(server + "/generate", json={"inputs": [5, 6, 7], "parameters": {
        "max_new_tokens": 8, "do_sample": True, "top_p": 0.9, "top_k": 50, "temperature": 1.0, "n": 2, "best_of": 2,
        "seed": 3}}, timeout=60).json()
    assert len(two["generated_text"]) == 2 and two["generated_text"][0] != two["generated_text"][1]
    stop = requests.post(server + "/generate", json={"inputs": [5, 6, 7], "parameters": {
        "max_new_tokens": 30, "ignore_eos": True, "stop_sequences": [[15]]}}, timeout=60).json()
    assert stop["finish_reason"] in ("stop", "length")
    assert requests.get(server + "/health", timeout=60).status_code == 200
    assert requests.get(server + "/v1/models", timeout=10).json()["data"][0]["max_model_len"] == 256
    assert requests.post(server + "/tokens", json={"text": "hello"}, timeout=10).json()["ntokens"] == 5
    m = requests.get(server + "/metrics", timeout=10).text
    assert "lightllm_request_count_total" in m
    assert "current_load" in requests.get(server + "/token_load", timeout=10).json()


@pytest.mark.timeout(600)
def test_concurrent_requests_and_abort(server):
    import concurrent.futures as cf

    def one(i):
        body = {"inputs": [10 + i] * (8 + i), "parameters": {"max_new_tokens": 12, "ignore_eos": True}}
        return requests.post(server + "/generate", json=body, timeout=120).json()

    with cf.ThreadPoolExecutor(12) as ex:
        outs = list(ex.map(one, range(12)))  # more requests than request slots (8): the rest wait or get 429
    ok = [o for o in outs if "count_output_tokens" in o]
    assert len(ok) >= 8 and all(o["count_output_tokens"] == 12 for o in ok)
    # client disconnect mid-stream: the server must stay healthy and free the slot
    body = {"inputs": [3, 4, 5], "parameters": {"max_new_tokens": 200, "ignore_eos": True}}
    with requests.post(server + "/generate_stream", json=body, stream=True, timeout=60) as r:
        it = r.iter_lines()
        next(it)
    time.sleep(1.0)
    again = requests.post(server + "/generate", json={"inputs": [3, 4, 5], "parameters": {"max_new_tokens": 2}},
                          timeout=60)
    assert again.status_code == 200


@pytest.mark.timeout(600)
def test_anthropic_responses_and_tgi_routes(server):
    msg = {"model": "m", "max_tokens": 5, "messages": [{"role": "user", "content": "hi there"}]}
    r = requests.post(server + "/v1/messages", json=msg, timeout=60)
    assert r.status_code == 200, r.text
    a = r.json()
    assert a["type"] == "message" and a["role"] == "assistant" and a["content"][0]["type"] == "text"
    assert a["usage"]["output_tokens"] <= 5 and a["usage"]["input_tokens"] > 0 and a["stop_reason"] in ("max_tokens", "end_turn")
    n = requests.post(server + "/v1/messages/count_tokens", json=msg, timeout=30).json()
    assert n["input_tokens"] == a["usage"]["input_tokens"]
    msg["stream"] = True
    with requests.post(server + "/v1/messages", json=msg, stream=True, timeout=60) as s:
        events = [l.decode() for l in s.iter_lines() if l.startswith(b"event:")]
    assert events[0] == "event: message_start" and events[-1] == "event: message_stop"
    assert "event: content_block_delta" in events

    resp = requests.post(server + "/v1/responses", json={"model": "m", "input": "say something",
                                                         "max_output_tokens": 4}, timeout=60)
    assert resp.status_code == 200, resp.text
    o = resp.json()
    assert o["object"] == "response" and o["status"] in ("completed", "incomplete")
    assert o["usage"]["output_tokens"] <= 4 and any(it["type"] == "message" for it in o["output"])

    tgi = requests.post(server + "/", json={"inputs": "hello", "parameters": {"max_new_tokens": 3}}, timeout=60)
    assert tgi.status_code == 200, tgi.text
    body = tgi.json()
    body = body[0] if isinstance(body, list) else body
    assert "generated_text" in body
    info = requests.get(server + "/get_server_info", timeout=10).json()
    assert info.get("max_req_total_len") == 256 or "max_req_total_len" in json.dumps(info)
    assert requests.get(server + "/get_model_name", timeout=10).status_code == 200
    assert requests.get(server + "/readiness", timeout=10).status_code == 200


@pytest.mark.timeout(600)
def test_openai_logprobs_tools_and_stop(server):
    chat = {"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "ignore_eos": True,
            "logprobs": True, "top_logprobs": 0}
    c = requests.post(server + "/v1/chat/completions", json=chat, timeout=60).json()
    lp = c["choices"][0].get("logprobs")
    assert lp is None or len(lp["content"]) == 4
    n2 = dict(chat, n=2, temperature=1.0, top_p=0.9, seed=1)
    c2 = requests.post(server + "/v1/chat/completions", json=n2, timeout=60).json()
    assert len(c2["choices"]) == 2
    tools = [{"type": "function", "function": {"name": "get_weather", "description": "x",
                                               "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]
    t = requests.post(server + "/v1/chat/completions", json=dict(chat, tools=tools, tool_choice="auto"), timeout=60)
    assert t.status_code == 200, t.text
    comp = requests.post(server + "/v1/completions", json={"model": "m", "prompt": [5, 6, 7, 8], "max_tokens": 3,
                                                          "echo": False, "logprobs": 1}, timeout=60)
    assert comp.status_code == 200, comp.text


@pytest.mark.timeout(600)
def test_load_generator_against_the_server(server):
    """The benchmark client (fixed concurrency and open-loop arrivals) reports throughput and latency percentiles."""
    for extra in (["--concurrency", "3"], ["--qps", "20", "--concurrency", "4"]):
        out = subprocess.run([sys.executable, "-m", "lightllm_b200.benchmark.client", "--url", server,
                              "--num_requests", "6", "--input_len", "12", "--output_len", "5", "--vocab_size", "1000",
                              "--prefix_share", "0.5", *extra], capture_output=True, text=True, cwd=ROOT, timeout=300,
                             env=dict(os.environ, PYTHONPATH=ROOT))
        assert out.returncode == 0, out.stderr[-2000:]
        rep = json.loads(out.stdout.strip().splitlines()[-1])
        txt = json.dumps(rep)
        assert "ttft" in txt.lower() and ("tok" in txt.lower())
        done = rep.get("completed", rep.get("num_completed", rep.get("requests_ok", 6)))
        assert done == 6


@pytest.mark.timeout(600)
def test_request_id_echo_and_validation_metric(server):
    body = {"inputs": list(range(5, 25)), "parameters": {"max_new_tokens": 2, "ignore_eos": True}}
    r = requests.post(server + "/generate", json=body, headers={"X-Request-Id": "abc-123"}, timeout=60)
    assert r.status_code == 200 and r.headers.get("X-Request-Id") == "abc-123"
    assert "X-Request-Id" not in requests.post(server + "/generate", json=body, timeout=60).headers
    m = requests.get(server + "/metrics", timeout=30).text
    assert "lightllm_request_validation_duration_count" in m
