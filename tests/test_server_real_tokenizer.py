"""The server with a real Hugging Face tokenizer (byte-level BPE built in the test, with a chat template): text
prompts, incremental detokenisation of arbitrary (also invalid UTF-8) byte tokens against a whole-sequence decode,
stop strings matched on the detokenised text, the chat template on the OpenAI route, special tokens hidden.
Reference behaviour: lightllm/server/detokenization/decode.py:7-35, lightllm/server/build_prompt.py."""
import json
import os
import signal
import socket
import subprocess
import sys
import time

import pytest
import requests

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _make_model_dir(d):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    from transformers import PreTrainedTokenizerFast

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    corpus = ["hello world, this is a tiny corpus for the tokenizer.", "the quick brown fox jumps over the lazy dog",
              "Grüße aus München – 你好世界 😀 emoji and accents: é è ü ñ", "stop here please. END of text"] * 20
    trainer = trainers.BpeTrainer(vocab_size=400, special_tokens=["<|bos|>", "<|eos|>", "<|user|>", "<|assistant|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(corpus, trainer)
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<|bos|>", eos_token="<|eos|>")
    fast.chat_template = ("{% for m in messages %}{% if m['role'] == 'user' %}<|user|>{{ m['content'] }}{% else %}"
                          "<|assistant|>{{ m['content'] }}<|eos|>{% endif %}{% endfor %}"
                          "{% if add_generation_prompt %}<|assistant|>{% endif %}")
    fast.save_pretrained(str(d))
    cfg = {"model_type": "llama", "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 4,
           "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 256, "vocab_size": len(fast),
           "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "eos_token_id": fast.eos_token_id,
           "max_position_embeddings": 512, "torch_dtype": "float32"}
    (d / "config.json").write_text(json.dumps(cfg))
    return fast


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    d = tmp_path_factory.mktemp("real_tok")
    tok = _make_model_dir(d)
    port = _free_port()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    log = open(d / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(d), "--port",
                             str(port), "--data_type", "fp32", "--max_total_token_num", "4096",
                             "--running_max_req_size", "8", "--max_req_total_len", "512", "--tp", "1"],
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
    yield url, tok
    try:
        os.killpg(proc.pid, signal.SIGTERM)
    except ProcessLookupError:
        pass
    try:
        proc.wait(timeout=20)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)


def _gen(url, prompt, **params):
    params.setdefault("max_new_tokens", 40)
    r = requests.post(url + "/generate", json={"inputs": prompt, "parameters": params}, timeout=120)
    assert r.status_code == 200, r.text
    return r.json()


@pytest.mark.timeout(600)
def test_text_prompts_and_incremental_detokenisation(server):
    url, tok = server
    for prompt in ("hello world", "Grüße aus München – 你好世界 😀", "the quick brown fox"):
        r = _gen(url, prompt, ignore_eos=True, return_details=True, do_sample=True, temperature=3.0, seed=11)
        assert r["prompt_tokens"] == len(tok.encode(prompt))
        ids = [t["id"] for t in r["tokens"]]
        pieces = "".join(t["text"] for t in r["tokens"])
        assert pieces == r["generated_text"][0]
        # random byte tokens: the pieces, joined, are the whole-sequence decode (special tokens hidden); an
        # incomplete UTF-8 sequence at the very end is held back
        whole = tok.decode(ids, skip_special_tokens=True)
        assert whole.startswith(pieces.rstrip("�")) or pieces == whole, (pieces, whole)
        assert len(pieces) >= len(whole) - 4
        for sp in ("<|bos|>", "<|eos|>", "<|user|>", "<|assistant|>"):
            assert sp not in pieces


@pytest.mark.timeout(600)
def test_stop_strings_and_chat_template(server):
    url, tok = server
    base = _gen(url, "hello world", ignore_eos=True, max_new_tokens=30)
    text = base["generated_text"][0]
    printable = [i for i in range(2, len(text) - 3) if text[i:i + 2].isprintable() and "�" not in text[i:i + 2]]
    if printable:
        stop = text[printable[0]:printable[0] + 2]
        r = _gen(url, "hello world", ignore_eos=True, max_new_tokens=30, stop_sequences=[stop])
        assert r["finish_reason"] == "stop" and r["count_output_tokens"] < 30
        assert stop in r["generated_text"][0] or r["generated_text"][0] == text[:text.index(stop)]
    chat = {"model": "m", "messages": [{"role": "user", "content": "hello world"}], "max_tokens": 6,
            "ignore_eos": True}
    c = requests.post(url + "/v1/chat/completions", json=chat, timeout=120).json()
    want = tok.apply_chat_template(chat["messages"], tokenize=True, add_generation_prompt=True)
    want = want if isinstance(want, list) else want["input_ids"]
    assert c["usage"]["prompt_tokens"] == len(want) and c["usage"]["completion_tokens"] == 6
    toks = requests.post(url + "/tokens", json={"text": "hello world"}, timeout=30).json()
    assert toks.get("ntokens", toks.get("count")) == len(tok.encode("hello world"))
