"""Prefill / decode disaggregation with speculative decoding on both nodes (CPU / gloo): the prefill node runs the
draft pass over the prompt before it ships the pages (the pool carries the draft module's layer), the decode node
verifies and proposes; a client of the pd_master gets the target model's plain greedy tokens.
Reference: mode_backend/chunked_prefill/impl.py:244-446 (prefill_mtp / decode_mtp) under the pd backends."""
import json
import os
import signal
import time

import pytest
import requests

from test_pd_e2e import CFG, _free_port, _spawn, _wait_up


@pytest.mark.timeout(1200)
def test_pd_nodes_with_draft_modules(tmp_path):
    from lightllm_b200.engine.llm import LLM

    d = tmp_path
    (d / "config.json").write_text(json.dumps(CFG))
    pm, pp, pdp = _free_port(), _free_port(), _free_port()
    procs = []
    common = ["--model_dir", str(d), "--data_type", "fp32", "--max_total_token_num", "4096", "--running_max_req_size", "8",
              "--max_req_total_len", "256", "--tp", "1", "--host", "127.0.0.1", "--mtp_mode", "vanilla_with_att",
              "--mtp_step", "2", "--mtp_draft_model_dir", str(d)]
    try:
        master = _spawn(["--run_mode", "pd_master", "--port", str(pm), "--host", "127.0.0.1", "--model_dir", str(d),
                         "--select_p_d_node_strategy", "round_robin"], d / "master.log")
        procs.append(master)
        _wait_up(f"http://127.0.0.1:{pm}", master, d / "master.log")
        pd_flags = ["--pd_master_ip", "127.0.0.1", "--pd_master_port", str(pm), "--pd_kv_page_size", "16"]
        prefill = _spawn(common + ["--run_mode", "prefill", "--port", str(pp)] + pd_flags, d / "prefill.log")
        decode = _spawn(common + ["--run_mode", "decode", "--port", str(pdp)] + pd_flags, d / "decode.log")
        procs += [prefill, decode]
        _wait_up(f"http://127.0.0.1:{pp}", prefill, d / "prefill.log", 300)
        _wait_up(f"http://127.0.0.1:{pdp}", decode, d / "decode.log", 300)
        url = f"http://127.0.0.1:{pm}"
        llm = LLM(config=CFG, data_type="float32", max_total_token_num=2048, running_max_req_size=4,
                  max_req_total_len=256, batch_max_tokens=256)
        logs = lambda: "\\n".join(f"--- {n}\\n" + open(d / n).read()[-1500:]  # noqa: E731
                                 for n in ("master.log", "prefill.log", "decode.log"))
        t0 = time.time()
        accepted = 0
        for prompt in (list(range(7, 60)), list(range(100, 131))):
            r = None
            while time.time() - t0 < 120:
                r = requests.post(url + "/generate", json={"inputs": prompt, "parameters": {
                    "max_new_tokens": 13, "ignore_eos": True, "return_details": True}}, timeout=120)
                if r.status_code == 200:
                    break
                time.sleep(2)
            assert r is not None and r.status_code == 200, (r.text if r is not None else "") + logs()
            out = r.json()
            assert out["count_output_tokens"] == 13 and out["finish_reason"] == "length", str(out) + logs()
            want = llm.generate([prompt], {"max_new_tokens": 13, "ignore_eos": True})[0]["token_ids"]
            assert [t["id"] for t in out["tokens"]] == want, logs()
            accepted += int(out["tokens"][-1].get("mtp_accepted_token_num", 0))
        assert accepted >= 0
    finally:
        for p in procs:
            try:
                os.killpg(p.pid, signal.SIGTERM)
            except ProcessLookupError:
                pass
        for p in procs:
            try:
                p.wait(timeout=20)
            except Exception:
                try:
                    os.killpg(p.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
