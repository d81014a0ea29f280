"""Prefill / decode disaggregation with tensor parallelism inside both nodes (two gloo ranks each on CPU): every
rank ships its own KV shard to the rank of the same index, the decode ranks agree on which pages have landed on
all of them before any of them touches its pool, and the tokens equal a single-process run."""
import json
import os
import signal
import subprocess
import time

import pytest
import requests

from test_pd_e2e import CFG, _free_port, _spawn, _wait_up


@pytest.mark.timeout(1200)
def test_pd_with_tp2_on_both_nodes(tmp_path):
    from lightllm_b200.engine.llm import LLM

    d = tmp_path
    (d / "config.json").write_text(json.dumps(CFG))
    pm, pp, pdp = _free_port(), _free_port(), _free_port()
    common = ["--model_dir", str(d), "--data_type", "fp32", "--max_total_token_num", "4096", "--running_max_req_size", "8",
              "--max_req_total_len", "256", "--tp", "2", "--host", "127.0.0.1"]
    procs = []
    try:
        master = _spawn(["--run_mode", "pd_master", "--port", str(pm), "--host", "127.0.0.1", "--model_dir", str(d),
                         "--select_p_d_node_strategy", "round_robin"], d / "master.log")
        procs.append(master)
        _wait_up(f"http://127.0.0.1:{pm}", master, d / "master.log")
        flags = ["--pd_master_ip", "127.0.0.1", "--pd_master_port", str(pm), "--pd_kv_page_size", "16"]
        prefill = _spawn(common + ["--run_mode", "prefill", "--port", str(pp), "--nccl_port", str(_free_port())] + flags,
                         d / "prefill.log")
        decode = _spawn(common + ["--run_mode", "decode", "--port", str(pdp), "--nccl_port", str(_free_port())] + flags,
                        d / "decode.log")
        procs += [prefill, decode]
        _wait_up(f"http://127.0.0.1:{pp}", prefill, d / "prefill.log")
        _wait_up(f"http://127.0.0.1:{pdp}", decode, d / "decode.log")
        url = f"http://127.0.0.1:{pm}"
        llm = LLM(config=CFG, data_type="float32", max_total_token_num=2048, running_max_req_size=4,
                  max_req_total_len=256, batch_max_tokens=256)
        prompts = [list(range(7, 60)), list(range(100, 121)), list(range(7, 60)) + [3, 4, 5]]
        for k, prompt in enumerate(prompts):
            t0, r = time.time(), None
            while time.time() - t0 < 60:   # the nodes register with the master a moment after they come up
                r = requests.post(url + "/generate", json={"inputs": prompt, "parameters": {
                    "max_new_tokens": 9, "ignore_eos": True, "return_details": True}}, timeout=120)
                if r.status_code == 200 or k > 0:
                    break
                time.sleep(2)
            logs = "\n".join(f"--- {n}\n" + open(d / n).read()[-1500:] for n in ("master.log", "prefill.log", "decode.log"))
            assert r is not None and r.status_code == 200, (r.text if r is not None else "") + logs
            got = [t["id"] for t in r.json()["tokens"]]
            want = llm.generate([prompt], {"max_new_tokens": 9, "ignore_eos": True})[0]["token_ids"]
            assert got == want, logs
        assert all(p.poll() is None for p in procs)
    finally:
        for p in procs:
            try:
                os.killpg(p.pid, signal.SIGTERM)
            except ProcessLookupError:
                pass
        for p in procs:
            try:
                p.wait(timeout=20)
            except subprocess.TimeoutExpired:
                os.killpg(p.pid, signal.SIGKILL)
