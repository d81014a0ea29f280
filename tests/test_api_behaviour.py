"""API behaviour against the whole server on CPU, modelled on the reference's client-side scripts
(test/test_api/test_abort_chaos.py, test_abort_request.py, test_multiple_choices.py, test_seed_validation.py,
test_invalid_token_ids.py): clients that go away or abort at random leave no request behind, several choices per
request, seeded sampling, forbidden / allowed token ids, validation errors as HTTP 400."""
import json
import os
import random
import signal
import socket
import subprocess
import sys
import threading
import time

import pytest
import requests

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = {"model_type": "llama", "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 4,
       "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 256, "vocab_size": 512, "rms_norm_eps": 1e-6,
       "rope_theta": 10000.0, "eos_token_id": 2, "max_position_embeddings": 512, "torch_dtype": "float32"}


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    d = tmp_path_factory.mktemp("api_behaviour")
    (d / "config.json").write_text(json.dumps(CFG))
    port = _free_port()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    log = open(d / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(d), "--port",
                             str(port), "--data_type", "fp32", "--max_total_token_num", "4096",
                             "--running_max_req_size", "16", "--max_req_total_len", "256", "--tp", "1", "--enable_rl",
                             "--enable_prompt_logprobs"],
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


def _gen(url, ids, **params):
    params.setdefault("max_new_tokens", 8)
    return requests.post(url + "/generate", json={"inputs": ids, "parameters": params}, timeout=120)


@pytest.mark.timeout(600)
def test_abort_chaos_leaves_nothing_behind(server):
    rng = random.Random(0)
    results = []

    def client(i):
        ids = [rng.randrange(3, 500) for _ in range(rng.randrange(8, 60))]
        body = {"inputs": ids, "parameters": {"max_new_tokens": 120, "ignore_eos": True}}
        leave_after = rng.choice([1, 2, 5, None, None])
        got = 0
        try:
            with requests.post(server + "/generate_stream", json=body, stream=True, timeout=120) as r:
                for line in r.iter_lines():
                    if line.startswith(b"data:"):
                        got += 1
                        if leave_after is not None and got >= leave_after:
                            break                  # the client goes away in the middle of the stream
            results.append((i, got, leave_after))
        except Exception as e:                     # an aborted stream may end abruptly; the server must survive
            results.append((i, got, repr(e)))

    for delay in (1.0, 0.05, 0.3):          # late, while the requests are still being admitted, in mid-generation
        results.clear()
        threads = [threading.Thread(target=client, args=(i,)) for i in range(12)]
        t0 = time.time()
        for t in threads:
            t.start()
        time.sleep(delay)
        assert requests.post(server + "/abort_request", json={"abort_all": True}, timeout=30).json()["success"]
        for t in threads:
            t.join(timeout=180)
        # a client that keeps listening gets the end of its stream promptly, whatever stage the abort caught
        assert len(results) == 12 and time.time() - t0 < 60, results
        assert not [r for r in results if isinstance(r[2], str)], results
    # everything drains: no running request, the whole pool free again (prefix-cache entries count as free)
    deadline = time.time() + 60
    while time.time() < deadline:
        load = requests.get(server + "/token_load", timeout=10).json()
        snap = load[0] if isinstance(load, list) and load else load
        if requests.get(server + "/health", timeout=30).status_code == 200 and \
                float(snap.get("current_load", 0.0) if isinstance(snap, dict) else 0.0) <= 0.01:
            break
        time.sleep(1)
    r = _gen(server, list(range(5, 25)), ignore_eos=True)
    assert r.status_code == 200 and r.json()["count_output_tokens"] == 8
    # all sixteen request slots are usable afterwards: sixteen concurrent requests complete
    outs = []
    ts = [threading.Thread(target=lambda: outs.append(_gen(server, list(range(5, 15)), ignore_eos=True).status_code))
          for _ in range(16)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=120)
    assert outs == [200] * 16


@pytest.mark.timeout(300)
def test_multiple_choices(server):
    r = _gen(server, list(range(5, 25)), n=2, best_of=2, do_sample=True, temperature=1.5, ignore_eos=True).json()
    assert len(r["generated_text"]) == 2 and r["count_output_tokens"] == [8, 8]
    chat = {"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "n": 3, "ignore_eos": True}
    c = requests.post(server + "/v1/chat/completions", json=chat, timeout=120).json()
    assert [ch["index"] for ch in c["choices"]] == [0, 1, 2] and c["usage"]["completion_tokens"] == 12
    bad = _gen(server, [5, 6, 7], n=2, best_of=3)
    assert bad.status_code == 400


@pytest.mark.timeout(300)
def test_seeded_sampling(server):
    ids = list(range(40, 70))
    kw = dict(do_sample=True, temperature=2.0, top_k=50, ignore_eos=True, max_new_tokens=12, return_details=True)
    a = [t["id"] for t in _gen(server, ids, seed=7, **kw).json()["tokens"]]
    b = [t["id"] for t in _gen(server, ids, seed=7, **kw).json()["tokens"]]
    c = [t["id"] for t in _gen(server, ids, seed=8, **kw).json()["tokens"]]
    greedy = [t["id"] for t in _gen(server, ids, ignore_eos=True, max_new_tokens=12, return_details=True).json()["tokens"]]
    assert a == b and a != c and a != greedy


@pytest.mark.timeout(300)
def test_forbidden_and_allowed_token_ids(server):
    ids = list(range(100, 130))
    base = [t["id"] for t in _gen(server, ids, ignore_eos=True, return_details=True).json()["tokens"]]
    banned = sorted(set(base))
    out = [t["id"] for t in _gen(server, ids, ignore_eos=True, return_details=True,
                                 invalid_token_ids=banned).json()["tokens"]]
    assert not set(out) & set(banned)
    out = [t["id"] for t in _gen(server, ids, ignore_eos=True, return_details=True,
                                 logit_bias={str(t): -100 for t in banned}).json()["tokens"]]
    assert not set(out) & set(banned)              # logit_bias keys are treated as forbidden ids
    allowed = [11, 12, 13]
    out = [t["id"] for t in _gen(server, ids, ignore_eos=True, return_details=True,
                                 allowed_token_ids=allowed).json()["tokens"]]
    assert set(out) <= set(allowed)


@pytest.mark.timeout(300)
def test_validation_errors_are_400(server):
    # (greedy requests reset temperature / top_p / top_k, so the sampling knobs are checked with do_sample)
    for params in ({"top_p": 1.5, "do_sample": True}, {"temperature": -1.0, "do_sample": True},
                   {"max_new_tokens": 0}, {"presence_penalty": -1.0}, {"top_k": 0, "do_sample": True},
                   {"repetition_penalty": 0.5}, {"min_new_tokens": 50, "max_new_tokens": 8}):
        r = _gen(server, [5, 6, 7], **params)
        assert r.status_code == 400, (params, r.status_code, r.text[:200])
    assert _gen(server, [5, 6, 100000]).status_code == 400            # token id outside the vocabulary
    assert _gen(server, list(range(3, 3 + 400)) , max_new_tokens=8).status_code == 400     # longer than the limit
    assert requests.get(server + "/health", timeout=30).status_code == 200


@pytest.mark.timeout(300)
def test_length_repair_and_stop_sequences(server):
    # prompt + max_new_tokens beyond the request limit: max_new_tokens is reduced silently, the request ends "length"
    ids = list(range(10, 110))
    r = _gen(server, ids, max_new_tokens=65535, ignore_eos=True).json()
    assert r["finish_reason"] == "length" and r["prompt_tokens"] == 100 and 100 <= r["count_output_tokens"] <= 156
    # stop sequences given as token ids end the request with "stop" and are matched inside the rank
    base = [t["id"] for t in _gen(server, ids[:30], max_new_tokens=12, ignore_eos=True,
                                  return_details=True).json()["tokens"]]
    r = _gen(server, ids[:30], max_new_tokens=12, ignore_eos=True, return_details=True,
             stop_sequences=[base[3:5]]).json()
    got = [t["id"] for t in r["tokens"]]
    assert r["finish_reason"] == "stop" and got == base[:5]
    # min_new_tokens keeps a request going past a stop token sequence that comes too early
    r = _gen(server, ids[:30], max_new_tokens=12, min_new_tokens=8, ignore_eos=True, return_details=True,
             stop_sequences=[base[3:5]]).json()
    assert r["count_output_tokens"] >= 8


@pytest.mark.timeout(600)
def test_prompt_logprobs(server):
    """`--enable_prompt_logprobs`: `prompt_logprobs` = 0 returns every prompt token's logprob and rank, k > 0 also the
    k most likely tokens per position (reference: lightllm/server/core/objs/token_metadata.py:100-157)."""
    import math

    ids = list(range(7, 37))
    body = {"inputs": ids, "parameters": {"max_new_tokens": 3, "ignore_eos": True, "prompt_logprobs": 0}}
    r0 = requests.post(server + "/generate", json=body, timeout=120).json()
    assert r0["prompt_token_ids"] == ids and len(r0["prompt_logprobs"]) == 30 and r0["prompt_logprobs"][0] is None
    own = []
    for pos in range(1, 30):
        entry = r0["prompt_logprobs"][pos]
        assert list(entry) == [str(ids[pos])]
        e = entry[str(ids[pos])]
        assert e["logprob"] < 0 and 1 <= e["rank"] <= 512
        own.append((e["logprob"], e["rank"]))
    body["parameters"]["prompt_logprobs"] = 3
    r3 = requests.post(server + "/generate", json=body, timeout=120).json()        # no prefix-cache shortcut
    for pos in range(1, 30):
        entry = r3["prompt_logprobs"][pos]
        e = entry[str(ids[pos])]
        assert abs(e["logprob"] - own[pos - 1][0]) < 1e-4 and e["rank"] == own[pos - 1][1]
        top = sorted((v for v in entry.values() if v["rank"] <= 3), key=lambda v: v["rank"])
        assert [v["rank"] for v in top][:3] == [1, 2, 3] and len(entry) in (3, 4)
        assert top[0]["logprob"] >= top[1]["logprob"] >= top[2]["logprob"] >= e["logprob"] - 1e-6 or e["rank"] <= 3
        assert math.exp(top[0]["logprob"]) <= 1.0
    plain = requests.post(server + "/generate", json={"inputs": ids, "parameters": {"max_new_tokens": 3}},
                          timeout=120).json()
    assert "prompt_logprobs" not in plain


@pytest.mark.timeout(300)
def test_completions_echo_with_logprobs_scores_the_prompt(server):
    """/v1/completions with echo + logprobs (+ max_tokens 0): the way evaluation harnesses score a continuation."""
    ids = list(range(7, 37))
    want = _gen(server, ids, max_new_tokens=1, prompt_logprobs=0).json()["prompt_logprobs"]
    body = {"model": "m", "prompt": ids, "echo": True, "logprobs": 2, "max_tokens": 0}
    c = requests.post(server + "/v1/completions", json=body, timeout=120).json()
    lp = c["choices"][0]["logprobs"]
    assert len(lp["tokens"]) == 30 and lp["token_logprobs"][0] is None and lp["top_logprobs"][0] is None
    for pos in range(1, 30):
        assert abs(lp["token_logprobs"][pos] - want[pos][str(ids[pos])]["logprob"]) < 1e-4
        assert 2 <= len(lp["top_logprobs"][pos]) <= 3
    assert lp["text_offset"] == [sum(len(t) for t in lp["tokens"][:i]) for i in range(30)]
    assert c["usage"]["completion_tokens"] == 0 and c["choices"][0]["text"] == "".join(lp["tokens"])
    # with output: the generated tokens follow the prompt's
    body.update(max_tokens=3, ignore_eos=True)
    c = requests.post(server + "/v1/completions", json=body, timeout=120).json()
    lp = c["choices"][0]["logprobs"]
    assert len(lp["tokens"]) == 33 and all(x is not None for x in lp["token_logprobs"][1:])
