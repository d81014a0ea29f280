"""Failure detection without touching a GPU: the health monitor's kill decision, a rank that leaves between steps
(the survivor's next host collective ends with an error instead of hanging), a prefill/decode node that drops
out of the pd_master's registry, and the status-word checks of the fused kernels' host wrappers."""
import asyncio
import datetime
import os
import socket
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_health_monitor_kills_after_consecutive_failures():
    from lightllm_b200.server.health_monitor import manager as hm

    calls, killed = {"n": 0}, []

    def get(url, timeout):
        calls["n"] += 1
        ok = calls["n"] in (1, 3)   # ok, fail, ok, fail, fail, fail -> kill on the 6th probe
        if not ok:
            raise ConnectionError("down")
        return SimpleNamespace(status_code=200)

    mon = hm.HealthMonitor(SimpleNamespace(port=1234), get=get, kill=killed.append, sleep=lambda s: None)
    assert mon.run(max_iters=10) == "killed"
    assert calls["n"] == 6 and killed == [mon.parent]
    ok_mon = hm.HealthMonitor(SimpleNamespace(port=1), get=lambda u, timeout: SimpleNamespace(status_code=200),
                              kill=killed.append, sleep=lambda s: None)
    assert ok_mon.run(max_iters=5) == "stopped" and len(killed) == 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, out_dir):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", world_size=world, rank=rank,
                            timeout=datetime.timedelta(seconds=5))
    t = torch.ones(1)
    dist.all_reduce(t)                       # step 1: everybody is there
    if rank == 1:
        os._exit(0)                          # leaves between steps, nothing in flight
    try:
        dist.all_reduce(t)                   # step 2: the peer is gone
        result = "no error"
    except Exception as e:                   # connection closed by peer / timeout
        result = type(e).__name__
    with open(os.path.join(out_dir, "r0.txt"), "w") as f:
        f.write(result)
    os._exit(0)


@pytest.mark.timeout(120)
def test_survivor_gets_an_error_when_a_rank_leaves(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    ps = [ctx.Process(target=_rank, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in ps:
        p.start()
    for p in ps:
        p.join(timeout=60)
        assert not p.is_alive(), "a rank hung instead of failing"
    assert open(tmp_path / "r0.txt").read() != "no error"


def test_pd_master_fails_requests_of_a_lost_node():
    from lightllm_b200.server.core.objs.sampling_params import SamplingParams
    from lightllm_b200.server.httpserver_for_pd_master.manager import HttpServerManagerForPDMaster
    from lightllm_b200.server.pd_io_struct import PDRegister

    async def go():
        m = HttpServerManagerForPDMaster(SimpleNamespace(select_p_d_node_strategy="round_robin", pd_master_mode="elastic"))

        class Silent:   # a prefill node that accepts the request and then disappears
            async def send_bytes(self, b):
                asyncio.get_running_loop().call_later(0.05, lambda: asyncio.ensure_future(m.remove_pd(1)))

        await m.register_pd(PDRegister(1, "a:1", "prefill", {}), Silent())
        await m.register_pd(PDRegister(2, "b:2", "decode", {}), Silent())
        out = [(t, fs.get_finish_reason()) async for _, t, md, fs in m.generate("x", SamplingParams().init(max_new_tokens=4))]
        assert out[-1][1] == "error" and 1 not in m.nodes

    asyncio.run(go())


def test_fused_wrappers_raise_on_status():
    from lightllm_b200.parallel.ep import EPGroup
    from lightllm_b200.parallel.fused import FusedTP

    f = FusedTP.__new__(FusedTP)
    f.local = torch.tensor([0, 0, 101, 0], dtype=torch.int32)   # status word: wait for rank 1 ran out
    with pytest.raises(RuntimeError, match="timed out"):
        f.check()
    f.local[2] = 0
    f.check()
    e = EPGroup.__new__(EPGroup)
    e.cuda, e.local = True, torch.tensor([0, 0, 390, 0], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="exchange failed"):
        e.check()
