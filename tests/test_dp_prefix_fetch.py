"""Cross-replica prefix fetch (`--enable_dp_prompt_cache_fetch`): the plan on hand-made cases, and two replicas on
CPU / gloo where the second one copies a cached prompt prefix from the first instead of recomputing it.
Reference: lightllm/server/router/model_infer/mode_backend/dp_backend/dp_shared_kv_trans.py:1-139."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from lightllm_b200.engine.dp_prefix_fetch import plan_fetches

CFG = dict(model_type="llama", hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
           head_dim=32, intermediate_size=256, vocab_size=512, rms_norm_eps=1e-6, rope_theta=10000.0, eos_token_id=2)


def test_plan():
    # 3 replicas, 4 requests.  match[replica, request]
    match = np.array([[100, 0, 40, 10],
                      [0, 64, 40, 30],
                      [100, 200, 0, 0]])
    owners, lens = [1, 0, 2, 0], [150, 150, 41, 100]
    free = np.array([1000, 90, 1000])
    plan = plan_fetches(match, owners, lens, free, min_gain=32)
    # req 0: owner 1 has nothing, replicas 0 and 2 have 100 -> from 0 (lowest), but owner 1 has only 90 free: skipped
    # req 1: owner 0 has 0, replica 2 has 200 -> capped at prompt_len - 1 = 149
    # req 2: owner 2, replica 0 has 40 = prompt_len - 1 -> 40 tokens from 0
    # req 3: owner 0 has 10, replica 1 has 30: gain 20 < 32 -> skipped
    assert plan == [(1, 2, 0, 0, 149), (2, 0, 2, 0, 40)]
    free[1] = 101
    assert plan_fetches(match, owners, lens, free, 32)[0] == (0, 0, 1, 0, 100)
    # an owner that already has the longest match never fetches
    assert plan_fetches(np.array([[50], [50]]), [1], [80], np.array([500, 500]), 1) == []


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.parallel import dist as pdist

    torch.set_num_threads(2)
    pdist.init_distributed(world, rank, dp=world, host="127.0.0.1", port=port, backend="gloo", device=torch.device("cpu"))
    llm = LLM(config=CFG, data_type="float32", max_total_token_num=2048, running_max_req_size=4, max_req_total_len=256,
              batch_max_tokens=128, random_seed=0)
    g = torch.Generator().manual_seed(5)
    shared = torch.randint(3, 512, (96,), generator=g).tolist()
    tail = torch.randint(3, 512, (20,), generator=g).tolist()
    other = torch.randint(3, 512, (30,), generator=g).tolist()
    par = {"max_new_tokens": 6, "ignore_eos": True}
    # scheduling pass 1: replica 0 serves the shared prompt, replica 1 something else
    first = llm.generate([shared] if rank == 0 or world == 1 else [other], par)
    # scheduling pass 2: the router gives shared + tail to replica 1 (replica 0 gets an unrelated prompt); every rank sees the
    # same list of new requests
    new = [(world - 1, np.array(shared + tail)), (0, np.array(other + tail))]
    got = llm.backend.fetch_prefixes(new) if world > 1 else 0
    mine = [shared + tail] if rank == world - 1 else [other + tail]
    second = llm.generate(mine, par)
    torch.save({"first": first[0]["token_ids"], "second": second[0]["token_ids"], "got": got,
                "cache_len": second[0]["prompt_cache_len"],
                "served": llm.backend._prefix_fetch.stats["served_tokens"] if world > 1 else 0},
               os.path.join(out_dir, f"w{world}_r{rank}.pt"))
    pdist.destroy()


@pytest.mark.timeout(600)
def test_second_replica_copies_the_prefix(tmp_path):
    mp.spawn(_worker, args=(1, _free_port(), str(tmp_path)), nprocs=1, join=True)
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    one = torch.load(tmp_path / "w1_r0.pt")
    r0, r1 = torch.load(tmp_path / "w2_r0.pt"), torch.load(tmp_path / "w2_r1.pt")
    # replica 0 cached the 96 prompt tokens + 5 produced ones; shared + tail shares the first 96 with that path
    assert r1["got"] == 96 and r0["served"] == 96 and r0["got"] == 0
    assert r1["cache_len"] == 96                         # admission found the copied rows in replica 1's own tree
    assert r1["second"] == one["second"]                 # and they hold the right KV: same tokens as a single process
    assert r0["first"] == one["first"]


@pytest.mark.timeout(900)
def test_server_dp2_fetches_across_replicas(tmp_path):
    """The whole process tree with `--tp 2 --dp 2 --enable_dp_prompt_cache_fetch` on CPU / gloo: a prompt served by
    replica 0 is a cache hit for a longer prompt sent to replica 1."""
    import json
    import signal
    import subprocess
    import sys
    import time

    import requests

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = dict(CFG, max_position_embeddings=512, torch_dtype="float32")
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    port = _free_port()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=root)
    log = open(tmp_path / "server.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(tmp_path),
                             "--port", str(port), "--data_type", "fp32", "--max_total_token_num", "2048",
                             "--running_max_req_size", "4", "--max_req_total_len", "256", "--tp", "2", "--dp", "2",
                             "--enable_dp_prompt_cache_fetch"],
                            env=env, stdout=log, stderr=subprocess.STDOUT, cwd=root, start_new_session=True)
    url = f"http://127.0.0.1:{port}"
    try:
        t0, up = time.time(), False
        while time.time() - t0 < 300 and proc.poll() is None:
            try:
                if requests.get(url + "/liveness", timeout=2).status_code == 200:
                    up = True
                    break
            except Exception:
                time.sleep(1)
        assert up, open(tmp_path / "server.log").read()[-3000:]
        base = list(range(5, 101))

        def ask(ids, dp):
            body = {"inputs": ids, "parameters": {"max_new_tokens": 4, "ignore_eos": True, "return_details": True,
                                                  "suggested_dp_index": dp}}
            return requests.post(url + "/generate", json=body, timeout=120).json()

        a = ask(base, 0)
        assert a["tokens"][0]["prompt_cache_len"] == 0
        b = ask(base + [7, 8, 9, 10, 11, 12], 1)          # another replica, whose own tree is empty
        assert b["tokens"][0]["prompt_cache_len"] >= 90, b["tokens"][0]
        c = ask(base + [7, 8, 9, 10, 11, 12], 0)          # same question to the replica that computed it all itself
        assert [t["id"] for t in c["tokens"]] == [t["id"] for t in b["tokens"]]
    finally:
        try:
            os.killpg(proc.pid, signal.SIGTERM)
        except ProcessLookupError:
            pass
        try:
            proc.wait(timeout=20)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
