"""Vision-language serving end to end on CPU: HTTP worker (image preload, embed-cache records, placeholder
expansion) -> embed cache service + shared arena -> visual server (vision tower) -> router -> model rank (embedding
merge + M-RoPE).  A tiny random-weight Qwen2-VL; the first tokens equal an offline run with the same image."""
import base64
import json
import os
import signal
import socket
import subprocess
import sys
import time
from io import BytesIO

import numpy as np
import pytest
import requests
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = {"model_type": "qwen2_vl", "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
       "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 300, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
       "rope_scaling": {"type": "mrope", "mrope_section": [2, 3, 3]}, "eos_token_id": 2, "max_position_embeddings": 512,
       "torch_dtype": "float32", "image_token_id": 290, "tie_word_embeddings": False,
       "vision_config": {"depth": 2, "embed_dim": 32, "hidden_size": 64, "num_heads": 4, "mlp_ratio": 2, "patch_size": 14,
                         "spatial_merge_size": 2, "temporal_patch_size": 2}}


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _png(w, h):
    from PIL import Image

    rng = np.random.default_rng(5)
    buf = BytesIO()
    Image.fromarray(rng.integers(0, 255, (h, w, 3), dtype=np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    d = tmp_path_factory.mktemp("vl")
    (d / "config.json").write_text(json.dumps(CFG))
    port = _free_port()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    log = open(d / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(d), "--port",
                             str(port), "--data_type", "fp32", "--max_total_token_num", "4096", "--running_max_req_size",
                             "8", "--max_req_total_len", "256", "--tp", "1", "--embed_cache_storage_size", "0.01"],
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
    yield url, d
    try:
        os.killpg(proc.pid, signal.SIGTERM)
    except ProcessLookupError:
        pass
    try:
        proc.wait(timeout=20)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)


def offline_tokens(raw, pre, post, n_new=5):
    """The first `n_new` greedy tokens of prompt `pre + picture + post` computed in this process: the same tower
    and language model as the servers of these tests (random weights are a function of the tensor names)."""
    from lightllm_b200.common.infer_state import ModelInput
    from lightllm_b200.models.registry import get_model
    from lightllm_b200.models.vit.qwen2_vl_visual import Qwen2VLVisionTower, preprocess_image
    from lightllm_b200.models.weights import RandomSource
    from lightllm_b200.parallel import dist as pdist

    vcfg = dict(CFG["vision_config"])
    tower = Qwen2VLVisionTower(vcfg, RandomSource(Qwen2VLVisionTower.weight_shapes(vcfg), dtype=torch.float32),
                               torch.device("cpu"), torch.float32)
    patches, grid = preprocess_image(raw)
    t, gh, gw = grid
    emb = tower.forward(patches, [grid]).bfloat16().float()      # the arena stores bf16
    n_img = emb.shape[0]

    class Arena:
        def read_rows(self, rows):
            return emb[rows]

    ps = pdist.ParallelState(device=torch.device("cpu"))
    m = get_model(CFG, pstate=ps, data_type="float32", max_total_token_num=512, max_req_num=2, max_seq_length=256,
                  disable_cudagraph=True)
    m.embed_arena = Arena()
    tok0 = 100_000_000
    ids = pre + list(range(tok0, tok0 + n_img)) + post
    item = {"token_id": tok0, "token_num": n_img, "start_index_in_embed_cache": 0, "grid_thwd": (t, gh, gw, 2)}
    req = m.req_manager.alloc()
    n = len(ids)
    mi = ModelInput(batch_size=1, total_token_num=n, max_kv_len=n, is_prefill=True,
                    b_req_idx=torch.tensor([req], dtype=torch.int32), b_seq_len=torch.tensor([n], dtype=torch.int32),
                    mem_indexes=m.mem_manager.alloc(n).clone(), input_ids=torch.tensor(ids),
                    b_ready_cache_len=torch.zeros(1, dtype=torch.int32), max_q_len=n,
                    multimodal_params=[{"images": [item], "audios": []}])
    want = [int(m.forward(mi).logits[0].argmax())]
    for k in range(n_new - 1):
        m.req_manager.req_to_next_token_ids[req] = want[-1]
        mi = ModelInput(batch_size=1, total_token_num=n + k + 1, max_kv_len=n + k + 1, is_prefill=False,
                        b_req_idx=torch.tensor([req], dtype=torch.int32),
                        b_seq_len=torch.tensor([n + k + 1], dtype=torch.int32), mem_indexes=m.mem_manager.alloc(1).clone())
        want.append(int(m.forward(mi).logits[0].argmax()))
    return want


@pytest.mark.timeout(900)
def test_image_request_matches_offline(server):
    from lightllm_b200.models.vit.qwen2_vl_visual import image_token_num

    url, d = server
    raw = _png(84, 56)
    n_img, (t, gh, gw) = image_token_num(84, 56)
    pre, post = [5, 17, 33], [9, 44, 120, 7]
    body = {"inputs": pre + [290] + post,
            "parameters": {"max_new_tokens": 5, "ignore_eos": True, "return_details": True},
            "multimodal_params": {"images": [{"type": "base64", "data": base64.b64encode(raw).decode()}]}}
    r = requests.post(url + "/generate", json=body, timeout=180)
    log = open(d / "server.log").read()[-3000:]
    assert r.status_code == 200, r.text + log
    out = r.json()
    assert out["prompt_tokens"] == len(pre) + n_img + len(post), str(out) + log
    got = [tk["id"] for tk in out["tokens"]]
    want = offline_tokens(raw, pre, post)
    assert got == want, log
    # the same image again: served from the embed cache (same virtual ids -> prefix cache hit on the prompt)
    r2 = requests.post(url + "/generate", json=body, timeout=180).json()
    assert [tk["id"] for tk in r2["tokens"]] == want and r2["tokens"][0]["prompt_cache_len"] >= len(pre) + n_img
