"""PD disaggregation on CPU: selector policies and the master's request flow with in-memory fake nodes,
and the KV page transport between two processes over gloo."""
import asyncio
import multiprocessing as mp
import pickle
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from lightllm_b200.server.core.objs.req import FinishStatus
from lightllm_b200.server.core.objs.sampling_params import SamplingParams
from lightllm_b200.server.httpserver_for_pd_master.manager import HttpServerManagerForPDMaster
from lightllm_b200.server.httpserver_for_pd_master.selector import (CacheAwareSelector, RoundRobinSelector,
                                                                     SampledPrefixIndex, create_selector)
from lightllm_b200.server.pd_io_struct import (NodeRunStatus, PDClient, PDHeartbeat, PDPromptIds, PDRegister,
                                                PDRequest, PDToken, UpKVStatus)


def _node(i, mode, usage=0.0):
    n = PDClient(i, f"10.0.0.{i}:80{i:02d}", mode, {"tp": 1, "pd_kv_port": 9000 + i})
    n.run_status = NodeRunStatus(total_token_usage_rate=usage)
    return n


def test_round_robin_and_adaptive():
    ps, ds = [_node(1, "prefill"), _node(2, "prefill")], [_node(3, "decode"), _node(4, "decode", usage=1.0)]
    rr = RoundRobinSelector()
    rr.update_nodes(ps, ds)
    picks = [rr.select_p_d_node("x") for _ in range(4)]
    assert [p.node_id for p, _ in picks] == [1, 2, 1, 2] and [d.node_id for _, d in picks] == [3, 4, 3, 4]
    ad = create_selector("adaptive_load")
    ad.update_nodes(ps, ds)
    c = sum(ad.select_p_d_node("x")[1].node_id == 3 for _ in range(300))
    assert c > 250  # the full decode node is picked with weight 0.02
    with pytest.raises(ValueError):
        create_selector("nope")


def test_prefix_index():
    idx = SampledPrefixIndex(stride=4, max_nodes=8, evict_batch=4)
    idx.insert("abcdefghijklmnop", "A")
    idx.insert("abcdefghXXXXXXXX", "B")
    m = idx.match("abcdefghijklZZZZ")
    assert m["A"] == 12 and m["B"] == 8
    for i in range(10):
        idx.insert(f"{i:04d}" * 3, "C")
    assert idx.size <= 8 + 3


def test_cache_aware_affinity_and_balance():
    sel = CacheAwareSelector(stride=4)
    ps, ds = [_node(1, "prefill"), _node(2, "prefill")], [_node(3, "decode")]
    sel.update_nodes(ps, ds)
    prompt = "system prompt " * 20
    p0, _ = sel.select_p_d_node(prompt + "q1")
    for n in ps:  # nobody idle any more
        n.dispatched_req_num, n.dispatched_prompt_chars = 1, 100
    p1, _ = sel.select_p_d_node(prompt + "q2")
    assert p1 is p0  # prefix affinity
    p0.dispatched_prompt_chars = 10_000  # far above 1.5x the other node
    p2, _ = sel.select_p_d_node(prompt + "q3")
    assert p2 is not p0
    before = sel.balance_rel_threshold
    sel.window = 2
    for r in (0.9, 0.9, 0.1, 0.1):
        sel.record_prompt_cache_hit_rate(r)
    assert sel.balance_rel_threshold > before


class FakeWS:
    """Plays a P or D node: answers a PDRequest the way httpserver/pd_loop.py would."""

    def __init__(self, mgr, role, n_tokens=3):
        self.mgr, self.role, self.n_tokens, self.got = mgr, role, n_tokens, []

    async def send_bytes(self, b):
        obj = pickle.loads(b)
        self.got.append(obj)
        if not isinstance(obj, PDRequest):
            return
        gid = obj.group_req_id
        if self.role == "prefill":
            await self.mgr.on_node_message(PDPromptIds(gid, [5, 6, 7]))
            await self.mgr.on_node_message(PDToken(gid, gid, "A", {"id": 11, "logprob": -0.1, "prompt_tokens": 3,
                                                                   "prompt_cache_len": 0, "count_output_tokens": 1}, 0))
            await self.mgr.on_node_message(UpKVStatus(gid, ok=True))
        else:
            assert obj.prompt == [5, 6, 7, 11] and obj.first_token[0] == 11
            for i in range(self.n_tokens):
                fin = FinishStatus.FINISHED_LENGTH if i == self.n_tokens - 1 else 0
                await self.mgr.on_node_message(PDToken(gid, gid, "BCD"[i], {"id": 20 + i, "count_output_tokens": i + 1}, fin))


def _master(mode="elastic"):
    args = SimpleNamespace(select_p_d_node_strategy="round_robin", pd_master_mode=mode)
    return HttpServerManagerForPDMaster(args)


def test_master_flow():
    async def go():
        m = _master()
        sp = SamplingParams().init(max_new_tokens=4)
        with pytest.raises(Exception):
            async for _ in m.generate("hi", sp):
                pass
        wp, wd = FakeWS(m, "prefill"), FakeWS(m, "decode")
        await m.register_pd(PDRegister(1, "10.0.0.1:8001", "prefill", {"tp": 1, "pd_kv_port": 9001}), wp)
        await m.register_pd(PDRegister(2, "10.0.0.2:8002", "decode", {"tp": 1, "pd_kv_port": 9002}), wd)
        m.update_node_status(PDHeartbeat(2, NodeRunStatus(0.5)))
        assert m.nodes[2].run_status.total_token_usage_rate == 0.5
        out = [(t, fs.is_finished(), md.get("count_output_tokens")) async for _, t, md, fs in m.generate("hi", sp)]
        assert [o[0] for o in out] == ["A", "B", "C", "D"] and [o[1] for o in out] == [False, False, False, True]
        assert [o[2] for o in out] == [1, 2, 3, 4]
        assert wp.got[0].peer["node_id"] == 2 and wp.got[0].peer["kv_endpoint"] == ("10.0.0.2", 9002)
        assert wd.got[0].sampling_params["max_new_tokens"] == 3
        assert m.nodes[1].dispatched_req_num == 0 and not m.reqs
        await m.remove_pd(2)
        assert not m.topology_ready()

    asyncio.run(go())


def test_master_fixed_topology_and_kv_failure():
    async def go():
        m = _master("1p2d")
        wp, wd = FakeWS(m, "prefill"), FakeWS(m, "decode")
        await m.register_pd(PDRegister(1, "a:1", "prefill", {}), wp)
        await m.register_pd(PDRegister(2, "b:2", "decode", {}), wd)
        assert not m.topology_ready()
        await m.register_pd(PDRegister(3, "c:3", "decode", {}), wd)
        assert m.topology_ready()

        class BadP(FakeWS):
            async def send_bytes(self, b):
                obj = pickle.loads(b)
                gid = obj.group_req_id
                await self.mgr.on_node_message(PDPromptIds(gid, [1]))
                await self.mgr.on_node_message(PDToken(gid, gid, "A", {"id": 2}, 0))
                await self.mgr.on_node_message(UpKVStatus(gid, ok=False))

        m.nodes[1].websocket = BadP(m, "prefill")
        out = [(t, fs.get_finish_reason()) async for _, t, md, fs in m.generate("x", SamplingParams().init(max_new_tokens=4))]
        assert out[-1][1] == "error"

    asyncio.run(go())


# ------------------------------------------------------------------ KV transport, 2 processes over gloo
def _pool(seed):
    from lightllm_b200.common.mem_manager import MemoryManager

    mm = MemoryManager(256, torch.float32, 2, 8, 3, torch.device("cpu"))
    g = torch.Generator().manual_seed(seed)
    mm.kv_buffer.copy_(torch.randn(mm.kv_buffer.shape, generator=g))
    return mm


NTOK = 100   # 7 pages of 16 tokens: more pages than the slot allocator's ring of host buffers is deep


def _recv_proc(q_port, q_out):
    from lightllm_b200.engine.pd import KVReceiver
    from lightllm_b200.engine.radix_cache import RadixCache

    mm = _pool(1)
    cache = RadixCache("pdtest", 256, 0, mem_manager=mm)
    rx = KVReceiver(mm, "127.0.0.1", 0, page_tokens=16, page_num=2)
    q_port.put(rx.port)
    import time

    # a stranger without the deployment's key is turned away and the listener keeps serving
    import os
    from multiprocessing.connection import Client

    try:
        Client(("127.0.0.1", rx.port), authkey=b"not the key")
        raise SystemExit("a wrong key was accepted")
    except Exception as e:
        assert "AuthenticationError" in type(e).__name__ or isinstance(e, (EOFError, OSError)), e

    done, t0 = [], time.time()
    scratch = []
    while len(done) < 2 and time.time() - t0 < 60:
        done += rx.drain(cache)
        # what a busy decode node does between two drains: a few decode-step allocations (they rotate the
        # allocator's small ring of host buffers, which an uncopied slot list of an earlier page would alias)
        for _ in range(5):
            scratch.append(mm.alloc(1).clone())
        if len(scratch) > 20:
            for sl in scratch:
                mm.free(sl)
            scratch = []
        time.sleep(0.01)
    for sl in scratch:
        mm.free(sl)
    res = {}
    for gid, ok, first in done:
        ids = np.arange(100 * gid, 100 * gid + NTOK, dtype=np.int64)
        node, n, slots = cache.match_prefix(ids, update_refs=False)
        res[gid] = (ok, first, n, mm.gather_pages(torch.from_numpy(np.asarray(slots))).numpy().copy())
    q_out.put(res)
    rx.close()


def test_kv_transport_gloo():
    ctx = mp.get_context("spawn")
    q_port, q_out = ctx.Queue(), ctx.Queue()
    p = ctx.Process(target=_recv_proc, args=(q_port, q_out))
    p.start()
    try:
        port = q_port.get(timeout=60)
        from lightllm_b200.engine.pd import KVSender

        mm = _pool(2)
        tx = KVSender(mm, page_tokens=16)
        sent = {}
        for gid in (1, 2):
            slots = mm.alloc(NTOK).clone()
            ids = list(range(100 * gid, 100 * gid + NTOK))
            if gid == 1:
                assert tx.send_request(("127.0.0.1", port), gid, ids, slots, first_token=(7, -0.5)) == 7
            else:   # the worker-thread path the prefill backend uses
                tx.submit(("127.0.0.1", port), gid, ids, slots, first_token=(7, -0.5), tag="second")
                import time

                t0, got = time.time(), []
                while not got and time.time() - t0 < 60:
                    got = tx.poll_done()
                    time.sleep(0.01)
                assert got == [("second", True, None)]
            sent[gid] = mm.gather_pages(slots).clone()
        res = q_out.get(timeout=60)
        tx.close()
        for gid in (1, 2):
            ok, first, n, kv = res[gid]
            assert ok and first == (7, -0.5) and n == NTOK
            assert np.array_equal(kv, sent[gid].numpy())
    finally:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()


def test_kv_sender_peer_that_never_accepts():
    """A decode node that is gone (a port nobody serves) or hangs (a socket that never answers the challenge) costs
    the worker thread a bounded wait and ends the request with an error; the caller is never blocked."""
    import socket
    import time

    from lightllm_b200.engine.pd import KVSender

    mm = _pool(3)
    tx = KVSender(mm, page_tokens=16, connect_timeout_s=1.0)
    silent = socket.socket()
    silent.bind(("127.0.0.1", 0))
    silent.listen(1)           # accepts at the TCP level, never speaks
    dead = socket.socket()
    dead.bind(("127.0.0.1", 0))
    dead_port = dead.getsockname()[1]
    dead.close()               # nobody listens here any more
    slots = mm.alloc(20).clone()
    t0 = time.time()
    tx.submit(("127.0.0.1", silent.getsockname()[1]), 1, list(range(20)), slots, tag="silent")
    tx.submit(("127.0.0.1", dead_port), 2, list(range(20)), slots, tag="dead")
    tx.submit(("127.0.0.1", dead_port), 3, list(range(20)), slots, tag="dead-again")
    assert time.time() - t0 < 0.5      # submit never waits
    got = []
    while len(got) < 3 and time.time() - t0 < 30:
        got += tx.poll_done()
        time.sleep(0.02)
    assert [g[0] for g in got] == ["silent", "dead", "dead-again"] and not any(g[1] for g in got)
    assert "failed" in got[2][2] and time.time() - t0 < 10   # the second try on a broken peer fails at once
    tx.close()
    silent.close()


def test_nodes_follow_the_config_servers_list_of_masters(monkeypatch):
    """One link per listed pd_master; a master that leaves the list is let go, a decode node gets one status queue
    per master and a transfer note goes to all of them."""
    from lightllm_b200.server.httpserver import pd_loop
    from lightllm_b200.server.pd_io_struct import PDMasterInfo

    started, cancelled = [], []

    async def fake_link(g, url, *a, **kw):
        started.append(("link", url))
        try:
            await asyncio.sleep(3600)
        except asyncio.CancelledError:
            cancelled.append(("link", url))
            raise

    async def fake_status(g, url, queue, *a, **kw):
        started.append(("status", url))
        try:
            await asyncio.sleep(3600)
        except asyncio.CancelledError:
            cancelled.append(("status", url))
            raise

    monkeypatch.setattr(pd_loop, "pd_master_link", fake_link)
    monkeypatch.setattr(pd_loop, "kv_status_link", fake_status)
    listed = [PDMasterInfo(1, "10.0.0.1:9000")]

    async def go():
        g = SimpleNamespace(args=SimpleNamespace(run_mode="decode", config_server_host="h", config_server_port=1))
        queues, links = {}, {}
        task = asyncio.create_task(pd_loop.follow_config_server(g, queues, links, fetch=lambda: list(listed), every_s=0.05))
        await asyncio.sleep(0.2)
        assert set(links) == {"ws://10.0.0.1:9000"} and set(queues) == set(links)
        listed.append(PDMasterInfo(2, "10.0.0.2:9000"))
        await asyncio.sleep(0.2)
        assert set(links) == {"ws://10.0.0.1:9000", "ws://10.0.0.2:9000"}
        for q in queues.values():               # what kv_status_pump does with one note
            await q.put(UpKVStatus(8, ok=True))
        assert all(q.qsize() == 1 for q in queues.values())
        del listed[0]
        await asyncio.sleep(0.2)
        assert set(links) == {"ws://10.0.0.2:9000"} and set(queues) == set(links)
        assert sorted(cancelled) == [("link", "ws://10.0.0.1:9000"), ("status", "ws://10.0.0.1:9000")]
        listed.clear()
        listed.append(None)                     # a broken answer: the links stay as they are
        await asyncio.sleep(0.2)
        assert set(links) == {"ws://10.0.0.2:9000"}
        task.cancel()

    asyncio.run(go())
    assert sorted(started) == [("link", "ws://10.0.0.1:9000"), ("link", "ws://10.0.0.2:9000"),
                               ("status", "ws://10.0.0.1:9000"), ("status", "ws://10.0.0.2:9000")]
