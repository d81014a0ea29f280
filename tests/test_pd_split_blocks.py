"""pd_master serves a long `max_new_tokens` in blocks: each block is a request of its own on the same pair of nodes
with the prompt grown by what was generated so far; the client sees one stream with whole-request counters."""
import asyncio
import json
import os
import pickle
import signal
import subprocess
import time
from types import SimpleNamespace

import pytest
import requests

from lightllm_b200.server.core.objs.req import FinishStatus
from lightllm_b200.server.core.objs.sampling_params import SamplingParams
from lightllm_b200.server.httpserver_for_pd_master import manager as pdm
from lightllm_b200.server.pd_io_struct import PDPromptIds, PDRegister, PDRequest, PDToken, UpKVStatus


class Node:
    """A prefill or decode node whose "model" continues any prompt with last id + 1 and stops at id 50."""

    def __init__(self, mgr, role):
        self.mgr, self.role, self.got = mgr, role, []

    async def send_bytes(self, b):
        obj = pickle.loads(b)
        self.got.append(obj)
        if not isinstance(obj, PDRequest):
            return
        gid = obj.group_req_id
        if self.role == "prefill":
            ids = [ord(c) % 40 for c in obj.prompt] if isinstance(obj.prompt, str) else list(obj.prompt)
            await self.mgr.on_node_message(PDPromptIds(gid, ids))
            nxt = ids[-1] + 1
            fin = FinishStatus.FINISHED_STOP if nxt == 50 else (
                FinishStatus.FINISHED_LENGTH if obj.sampling_params["max_new_tokens"] == 1 else 0)
            await self.mgr.on_node_message(PDToken(gid, gid, f"<{nxt}>", {
                "id": nxt, "logprob": -0.1, "prompt_tokens": len(ids), "prompt_cache_len": max(0, len(ids) - 3),
                "count_output_tokens": 1}, fin))
            await self.mgr.on_node_message(UpKVStatus(gid, ok=True))
        else:
            cur = obj.prompt[-1]
            n = obj.sampling_params["max_new_tokens"]
            for i in range(n):
                cur += 1
                fin = FinishStatus.FINISHED_STOP if cur == 50 else (FinishStatus.FINISHED_LENGTH if i == n - 1 else 0)
                await self.mgr.on_node_message(PDToken(gid, gid, f"<{cur}>", {"id": cur, "count_output_tokens": i + 1}, fin))
                if fin:
                    break


def test_split_budgets(monkeypatch):
    monkeypatch.setenv("LIGHTLLM_PD_SPLIT_MAX_NEW_TOKENS", "4")
    assert [pdm.split_max_new_tokens(n) for n in (1, 4, 5, 8, 11)] == [[1], [4], [4, 1], [4, 4], [4, 4, 3]]
    monkeypatch.delenv("LIGHTLLM_PD_SPLIT_MAX_NEW_TOKENS")
    assert pdm.split_block_tokens() == 2048 and pdm.split_max_new_tokens(5000) == [2048, 2048, 904]


def test_one_stream_over_several_blocks(monkeypatch):
    monkeypatch.setenv("LLB_PD_SPLIT_MAX_NEW_TOKENS", "4")

    async def go():
        m = pdm.HttpServerManagerForPDMaster(SimpleNamespace(select_p_d_node_strategy="round_robin", pd_master_mode="elastic"))
        wp, wd = Node(m, "prefill"), Node(m, "decode")
        await m.register_pd(PDRegister(1, "10.0.0.1:8001", "prefill", {"tp": 1, "pd_kv_port": 9001}), wp)
        await m.register_pd(PDRegister(2, "10.0.0.2:8002", "decode", {"tp": 1, "pd_kv_port": 9002}), wd)
        out = [(sid, t, md, fs) async for sid, t, md, fs in m.generate([7, 8, 9], SamplingParams().init(max_new_tokens=10))]
        assert [o[1] for o in out] == [f"<{i}>" for i in range(10, 20)]
        assert len({o[0] for o in out}) == 1                               # one id towards the client
        assert [o[3].is_finished() for o in out] == [False] * 9 + [True] and out[-1][3].get_finish_reason() == "length"
        assert [o[2]["count_output_tokens"] for o in out] == list(range(1, 11))
        assert all(o[2]["prompt_tokens"] == 3 and o[2].get("prompt_cache_len", 0) == 0 for o in out)
        # three blocks: 4 + 4 + 2 tokens; later blocks carry the grown prompt as token ids, on the same nodes
        reqs_p = [g for g in wp.got if isinstance(g, PDRequest)]
        assert [r.sampling_params["max_new_tokens"] for r in reqs_p] == [4, 4, 2]
        assert reqs_p[1].prompt == [7, 8, 9, 10, 11, 12, 13] and reqs_p[2].prompt == list(range(7, 18))
        assert len({r.group_req_id for r in reqs_p}) == 3 and not m.reqs and not m.alias and not m.block_prompt_ids
        assert m.nodes[1].dispatched_req_num == 0 and m.nodes[2].dispatched_req_num == 0
        # a stop inside the second block ends the request there
        out = [(t, fs) async for _, t, md, fs in m.generate([44], SamplingParams().init(max_new_tokens=30))]
        assert [o[0] for o in out] == ["<45>", "<46>", "<47>", "<48>", "<49>", "<50>"] and out[-1][1].get_finish_reason() == "stop"
        # an abort by the client's id reaches the block that is running
        sent = []

        async def fake_send(node, obj):
            sent.append(obj)

        m.alias[1000], m.reqs[1016] = 1016, SimpleNamespace(p=wp, d=wd)
        monkeypatch.setattr(m, "_send", fake_send)
        assert await m.abort(1000) and sent == [("ABORT", 1016), ("ABORT", 1016)]

    asyncio.run(go())


@pytest.mark.timeout(1200)
def test_cluster_with_small_blocks_matches_offline(tmp_path, monkeypatch):
    from test_pd_e2e import CFG, _free_port, _spawn, _wait_up

    from lightllm_b200.engine.llm import LLM

    monkeypatch.setenv("LLB_PD_SPLIT_MAX_NEW_TOKENS", "4")
    d = tmp_path
    (d / "config.json").write_text(json.dumps(CFG))
    pm, pp, pdp = _free_port(), _free_port(), _free_port()
    common = ["--model_dir", str(d), "--data_type", "fp32", "--max_total_token_num", "4096", "--running_max_req_size", "8",
              "--max_req_total_len", "256", "--tp", "1", "--host", "127.0.0.1"]
    procs = []
    try:
        master = _spawn(["--run_mode", "pd_master", "--port", str(pm), "--host", "127.0.0.1", "--model_dir", str(d),
                         "--select_p_d_node_strategy", "round_robin"], d / "master.log")
        procs.append(master)
        _wait_up(f"http://127.0.0.1:{pm}", master, d / "master.log")
        flags = ["--pd_master_ip", "127.0.0.1", "--pd_master_port", str(pm), "--pd_kv_page_size", "16"]
        procs.append(_spawn(common + ["--run_mode", "prefill", "--port", str(pp)] + flags, d / "prefill.log"))
        procs.append(_spawn(common + ["--run_mode", "decode", "--port", str(pdp)] + flags, d / "decode.log"))
        _wait_up(f"http://127.0.0.1:{pp}", procs[1], d / "prefill.log")
        _wait_up(f"http://127.0.0.1:{pdp}", procs[2], d / "decode.log")
        url = f"http://127.0.0.1:{pm}"
        prompt = list(range(7, 60))
        t0, r = time.time(), None
        while time.time() - t0 < 60:
            r = requests.post(url + "/generate", json={"inputs": prompt, "parameters": {
                "max_new_tokens": 11, "ignore_eos": True, "return_details": True}}, timeout=120)
            if r.status_code == 200:
                break
            time.sleep(2)
        logs = "\n".join(f"--- {n}\n" + open(d / n).read()[-1500:] for n in ("master.log", "prefill.log", "decode.log"))
        assert r is not None and r.status_code == 200, (r.text if r is not None else "") + logs
        out = r.json()
        llm = LLM(config=CFG, data_type="float32", max_total_token_num=2048, running_max_req_size=4,
                  max_req_total_len=256, batch_max_tokens=256)
        want = llm.generate([prompt], {"max_new_tokens": 11, "ignore_eos": True})[0]["token_ids"]
        assert [t["id"] for t in out["tokens"]] == want, logs
        assert out["count_output_tokens"] == 11 and out["finish_reason"] == "length" and out["prompt_tokens"] == len(prompt)
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
