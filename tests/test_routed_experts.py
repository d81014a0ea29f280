"""`--enable_return_routed_experts`: the routed expert ids of every token (all MoE layers) come back with the result.
Offline: the captured ids equal the router's choice recomputed from a hooked run, and tokens served from the prefix
cache bring their routing with them.  Server: `/generate` returns {"shape", "dtype", "data"}.
Reference: lightllm/common/basemodel/moe_route_info_manager.py:1-263."""
import json
import os
import signal
import socket
import subprocess
import sys
import time

import numpy as np
import pytest
import requests
import torch

from lightllm_b200.common import route_capture as rc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MOE = dict(model_type="qwen3_moe", hidden_size=128, intermediate_size=256, moe_intermediate_size=64,
           num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_experts=8,
           num_experts_per_tok=2, norm_topk_prob=True, vocab_size=512, rms_norm_eps=1e-6, eos_token_id=2,
           decoder_sparse_step=1, mlp_only_layers=[1], torch_dtype="float32", max_position_embeddings=512)


def test_layer_maps():
    assert rc.moe_layer_map(MOE) == {0: 0, 2: 1}
    ds = dict(num_hidden_layers=6, n_routed_experts=300, first_k_dense_replace=2, moe_layer_freq=2, num_experts_per_tok=8)
    assert rc.moe_layer_map(ds) == {2: 0, 4: 1} and rc.np_dtype_of(ds) == np.int16 and rc.top_k_of(ds) == 8
    assert rc.moe_layer_map(dict(num_hidden_layers=4, hidden_size=8)) == {}
    a = np.arange(24, dtype=np.uint8).reshape(3, 4, 2)
    assert np.array_equal(rc.decode(rc.encode(a)), a)


def test_offline_capture_matches_the_router_and_survives_prefix_reuse():
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.models import moe as moe_mod
    from lightllm_b200.parallel import dist as pdist

    pdist.init_distributed(1, 0, device=torch.device("cpu"))
    llm = LLM(config=MOE, data_type="float32", max_total_token_num=2048, running_max_req_size=4, max_req_total_len=128,
              batch_max_tokens=64, random_seed=0, enable_return_routed_experts=True)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(3, 512, (40,), generator=g).tolist()
    # record what the router chose, in call order, through the capture hook itself
    seen = []
    real = llm.model.route_capture.capture

    def spy(layer, ids, mem_index):
        seen.append((layer, ids.clone(), mem_index.clone()))
        return real(layer, ids, mem_index)

    llm.model.route_capture.capture = spy
    out = llm.generate([prompt], {"max_new_tokens": 6, "ignore_eos": True})[0]
    r = out["routed_experts"]
    assert r.shape == (40 + 6 - 1, 2, 2) and r.dtype == np.uint8      # the last produced token never ran
    # rebuild per-position routing from the hooked calls (prefill chunks of 64 tokens, then one token per step)
    want = {0: [], 2: []}
    for layer, ids, _ in seen:
        want[layer].append(ids)
    for layer, j in ((0, 0), (2, 1)):
        w = torch.cat(want[layer])[:45].numpy()
        assert np.array_equal(np.sort(r[:, j], -1), np.sort(w, -1)), layer
    assert len({int(x) for x in r.reshape(-1)}) > 2                    # not a constant
    # the same prompt again: its first 32+ tokens come out of the prefix cache and are not recomputed,
    # yet their routing is returned (the buffer is indexed by KV slot)
    seen.clear()
    out2 = llm.generate([prompt], {"max_new_tokens": 6, "ignore_eos": True})[0]
    assert out2["prompt_cache_len"] >= 32 and out2["token_ids"] == out["token_ids"]
    assert sum(ids.shape[0] for layer, ids, _ in seen if layer == 0) < 45
    assert np.array_equal(out2["routed_experts"], r)
    pdist.destroy()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.timeout(600)
def test_server_returns_routed_experts(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(MOE))
    port = _free_port()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    log = open(tmp_path / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(tmp_path),
                             "--port", str(port), "--data_type", "fp32", "--max_total_token_num", "2048",
                             "--running_max_req_size", "4", "--max_req_total_len", "128", "--tp", "1",
                             "--enable_return_routed_experts"],
                            env=env, stdout=log, stderr=subprocess.STDOUT, cwd=ROOT, start_new_session=True)
    url = f"http://127.0.0.1:{port}"
    try:
        t0, up = time.time(), False
        while time.time() - t0 < 240 and proc.poll() is None:
            try:
                if requests.get(url + "/liveness", timeout=2).status_code == 200:
                    up = True
                    break
            except Exception:
                time.sleep(1)
        assert up, open(tmp_path / "server.log").read()[-3000:]
        body = {"inputs": list(range(5, 35)), "parameters": {"max_new_tokens": 5, "ignore_eos": True}}
        r1 = requests.post(url + "/generate", json=body, timeout=120).json()
        a = rc.decode(r1["routed_experts"])
        assert a.shape == (30 + 5 - 1, 2, 2) and a.dtype == np.uint8 and int(a.max()) < 8
        r2 = requests.post(url + "/generate", json=body, timeout=120).json()       # prefix cache hit
        assert np.array_equal(rc.decode(r2["routed_experts"]), a)
        body["parameters"]["return_routed_experts"] = False
        assert "routed_experts" not in requests.post(url + "/generate", json=body, timeout=120).json()
    finally:
        try:
            os.killpg(proc.pid, signal.SIGTERM)
        except ProcessLookupError:
            pass
        try:
            proc.wait(timeout=20)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
