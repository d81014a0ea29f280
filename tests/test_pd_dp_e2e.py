"""Prefill / decode disaggregation with data-parallel replicas on both nodes (CPU / gloo): a pd_master, a prefill
node and a decode node, each `--tp 2 --dp 2` (two replicas of one rank).  The prefill node ships a request's KV to
the decode replica that both sides compute from the master's request id; the decode node places the follow-up
request on that replica.  Tokens equal the offline engine's.
Reference: mode_backend/pd/prefill_node_impl/prefill_impl_for_dp.py, decode_node_impl/decode_impl_for_dp.py."""
import json
import os
import signal
import time

import pytest
import requests

from test_pd_e2e import CFG, _free_port, _spawn, _wait_up


@pytest.mark.timeout(1200)
def test_pd_with_two_replicas_per_node(tmp_path):
    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.engine.mode_backends import decode_replica_of

    assert [decode_replica_of(g, 2) for g in (0, 8, 16, 24)] == [0, 1, 0, 1] and decode_replica_of(40, 1) == 0
    d = tmp_path
    (d / "config.json").write_text(json.dumps(CFG))
    pm, pp, pdp = _free_port(), _free_port(), _free_port()
    procs = []
    common = ["--model_dir", str(d), "--data_type", "fp32", "--max_total_token_num", "4096", "--running_max_req_size", "8",
              "--max_req_total_len", "256", "--tp", "2", "--dp", "2", "--host", "127.0.0.1"]
    try:
        master = _spawn(["--run_mode", "pd_master", "--port", str(pm), "--host", "127.0.0.1", "--model_dir", str(d),
                         "--select_p_d_node_strategy", "round_robin"], d / "master.log")
        procs.append(master)
        _wait_up(f"http://127.0.0.1:{pm}", master, d / "master.log")
        pd_flags = ["--pd_master_ip", "127.0.0.1", "--pd_master_port", str(pm), "--pd_kv_page_size", "16"]
        prefill = _spawn(common + ["--run_mode", "prefill", "--port", str(pp), "--nccl_port", str(_free_port())]
                         + pd_flags, d / "prefill.log")
        decode = _spawn(common + ["--run_mode", "decode", "--port", str(pdp), "--nccl_port", str(_free_port())]
                        + pd_flags, d / "decode.log")
        procs += [prefill, decode]
        _wait_up(f"http://127.0.0.1:{pp}", prefill, d / "prefill.log", 300)
        _wait_up(f"http://127.0.0.1:{pdp}", decode, d / "decode.log", 300)
        url = f"http://127.0.0.1:{pm}"
        llm = LLM(config=CFG, data_type="float32", max_total_token_num=2048, running_max_req_size=4,
                  max_req_total_len=256, batch_max_tokens=256)
        logs = lambda: "\n".join(f"--- {n}\n" + open(d / n).read()[-1500:]  # noqa: E731
                                 for n in ("master.log", "prefill.log", "decode.log"))
        t0, ok = time.time(), 0
        prompts = [list(range(7 + i, 60 + i)) for i in range(4)]      # consecutive ids: both decode replicas get work
        for prompt in prompts:
            r = None
            while time.time() - t0 < 120:
                r = requests.post(url + "/generate", json={"inputs": prompt, "parameters": {
                    "max_new_tokens": 9, "ignore_eos": True, "return_details": True}}, timeout=120)
                if r.status_code == 200:
                    break
                time.sleep(2)                                         # the nodes register a moment after they come up
            assert r is not None and r.status_code == 200, (r.text if r is not None else "") + logs()
            out = r.json()
            assert out["count_output_tokens"] == 9 and out["finish_reason"] == "length", str(out) + logs()
            want = llm.generate([prompt], {"max_new_tokens": 9, "ignore_eos": True})[0]["token_ids"]
            assert [t["id"] for t in out["tokens"]] == want, logs()
            # the decode replica found the prompt's KV in its prefix tree (it did not recompute the prompt)
            assert out["tokens"][1]["prompt_cache_len"] >= 48 or out["tokens"][0]["prompt_cache_len"] >= 48, \
                str(out["tokens"][:2]) + logs()
            ok += 1
        assert ok == 4
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
