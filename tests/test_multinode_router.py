"""Multi-node tensor parallelism, host side: the routers of two nodes (two processes, gloo) must write the same
message sequence to their ranks although requests reach them at different times and only node 0 learns of aborts,
and node 0's HTTP server relays requests to the other node.
Reference behaviour: lightllm/server/router/multinode_tp_helper.py:1-219, lightllm/server/httpserver/manager.py:201-260."""
import asyncio
import socket

import torch.distributed as dist
import torch.multiprocessing as mp

from lightllm_b200.server.core.objs.req import Req


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class _Mailbox:
    def __init__(self):
        self.msgs, self.busy = [], False

    def is_empty(self):
        return not self.busy

    def write_obj(self, cmds):
        self.msgs.append(cmds)

    def set_ready(self):
        pass


def _req(rid, n_in=100, max_new=10):
    r = Req()
    r.index_in_shm_mem = rid + 1000      # node-local in a real deployment
    r.init(rid, list(range(1, n_in + 1)), {"max_new_tokens": max_new, "ignore_eos": True}, None,
           chunked_prefill_size=4096, router_max_wait_tokens=1, max_total_len=1 << 20)
    r.group_req_id = rid
    return r


def _router(node_rank):
    from lightllm_b200.server.router.manager import RouterManager
    from lightllm_b200.server.router.multinode_sync import MultiNodeRouterSync
    from lightllm_b200.server.router.req_queue import ChunkedPrefillQueue, RouterStatics

    r = RouterManager.__new__(RouterManager)
    r.mailbox, r.pending_cmds, r.running_batch, r.batch_id = _Mailbox(), [], None, 0
    r.dp_size_in_node, r.statics, r._mn_dropped, r._exit_flushed = 1, RouterStatics(), set(), False
    r.req_queue = ChunkedPrefillQueue(max_total_tokens=128 * 2 + 1, batch_max_tokens=4096, running_max_req_size=16)
    r._usage_ratio = lambda: 0.0
    r.mn_sync = MultiNodeRouterSync(None, node_rank, 2)
    return r


def _describe(msgs):
    from lightllm_b200.server.core.objs.io_objs import NewReqsCmd

    out = []
    for cmds in msgs:
        out.append([(type(c).__name__, [x[0] for x in c.reqs] if isinstance(c, NewReqsCmd) else
                     getattr(c, "req_id", None)) for c in cmds])
    return out


def _node(rank, port, q):
    from lightllm_b200.server.core.objs.io_objs import FlushCacheCmd
    from lightllm_b200.server.router.model_rank import ExitCmd

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=2)
    r = _router(rank)
    reqs = {i: _req(8 * i) for i in range(4)}
    # scheduling pass 1: node 0 has requests 0, 1, 2; node 1 only 1 and 0 (other order, 2 not yet relayed) -> 0, 1 admitted
    r.req_queue.extend([reqs[0], reqs[1], reqs[2]] if rank == 0 else [reqs[1], reqs[0]])
    r._round_multinode()
    # scheduling pass 2: request 2 has arrived everywhere, but node 1's mailbox is still full -> nothing is written anywhere
    if rank == 1:
        r.req_queue.append(reqs[2])
        r.mailbox.busy = True
    r._round_multinode()
    r.mailbox.busy = False
    # scheduling pass 3: node 0 learns that request 0 was aborted and gets a cache flush command; the pool (2 requests' worth)
    # is full, so request 2 keeps waiting; node 1 must send the same abort + flush
    if rank == 0:
        reqs[0].is_aborted = True
        r.pending_cmds.append(FlushCacheCmd())
    r._round_multinode()
    # scheduling pass 4: both running requests have finished on node 1 already, on node 0 not yet (node-local timing);
    # request 3 arrives on node 0 only and request 2's client goes away on node 0 before admission
    if rank == 1:
        r.running_batch = None
    if rank == 0:
        r.req_queue.append(reqs[3])
        reqs[2].is_aborted = True
        r._mn_dropped.add(reqs[2].group_req_id)
        r.req_queue.pop_aborted()
    r._round_multinode()
    dropped_on_follower = rank == 1 and reqs[2].is_aborted
    if rank == 1:
        r.req_queue.pop_aborted()
        r.req_queue.append(reqs[3])
    else:
        r.running_batch = None
    # scheduling pass 5: request 3 everywhere -> admitted; exit command from node 0
    if rank == 0:
        r.pending_cmds.append(ExitCmd())
    r._round_multinode()
    # a request that never reaches node 1 (its relay failed there): node 0 gives it up after the waiting limit, the
    # requests behind it are no longer blocked
    r2 = _router(rank)
    r2.MULTINODE_WAIT_S = 0.2
    lost, behind = _req(800), _req(808)
    if rank == 0:
        r2.req_queue.extend([lost, behind])
    else:
        r2.req_queue.extend([behind])
    r2._round_multinode()
    first = _describe(r2.mailbox.msgs)
    import time as _t

    _t.sleep(0.3)
    r2._round_multinode()           # node 0 marks the lost request as aborted ...
    if rank == 0:
        r2._mn_dropped.update(x.group_req_id for x in r2.req_queue.waiting_req_list if x.is_aborted)
        r2.req_queue.pop_aborted()
    r2._round_multinode()           # ... and the one behind it is admitted everywhere
    q.put((rank, _describe(r.mailbox.msgs), r._exit_flushed, dropped_on_follower, first, _describe(r2.mailbox.msgs),
           lost.is_aborted))
    dist.barrier()
    dist.destroy_process_group()


def test_two_routers_write_identical_message_sequences():
    ctx = mp.get_context("spawn")
    q, port = ctx.Queue(), _free_port()
    ps = [ctx.Process(target=_node, args=(r, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = dict((r, rest) for r, *rest in (q.get(timeout=60) for _ in range(2)))
    for p in ps:
        p.join(timeout=30)
        assert p.exitcode == 0
    m0, m1 = got[0][0], got[1][0]
    assert m0 == m1
    assert m0 == [[("NewReqsCmd", [0, 8])],                                   # node 0's order, only common ones
                  [("FlushCacheCmd", None), ("AbortedReqCmd", 0)],
                  [("ExitCmd", None), ("NewReqsCmd", [24])]]
    assert got[0][1] and got[1][1]                                           # both loops leave after the exit
    assert got[1][2]                                                         # the follower dropped request 2 too
    assert got[0][3] == [] and got[1][3] == []                               # blocked while the lost request waits
    assert got[0][4] == got[1][4] == [[("NewReqsCmd", [808])]] and got[0][5]  # given up on node 0, the next one runs


class _FakeManager:
    def __init__(self):
        self.seen = []

    async def generate(self, prompt, sp, mm, group_req_id=None):
        self.seen.append((group_req_id, list(prompt), sp.max_new_tokens, mm))
        yield None


def test_request_relay_between_http_servers():
    from lightllm_b200.server.core.objs.sampling_params import SamplingParams
    from lightllm_b200.server.httpserver.multinode_relay import RelayFollower, RelayMaster

    async def run():
        port = _free_port()
        follower = RelayFollower("127.0.0.1", port, 1)      # comes up first, keeps saying hello
        hello = asyncio.create_task(follower.hello(timeout_s=20))
        await asyncio.sleep(0.2)
        master = RelayMaster(port, 1, host="127.0.0.1")
        await master.wait_peers(timeout_s=20)
        await hello
        fm = _FakeManager()
        task = asyncio.create_task(follower.follow(fm))
        sp = SamplingParams()
        sp.init(None, max_new_tokens=17)
        await master.relay(4242, [5, 6, 7], sp, {"images": []})
        await master.relay(4250, [9], sp, None)
        for _ in range(200):
            if len(fm.seen) == 2:
                break
            await asyncio.sleep(0.01)
        task.cancel()
        master.close()
        follower.close()
        return fm.seen

    seen = asyncio.run(run())
    assert seen == [(4242, [5, 6, 7], 17, {"images": []}), (4250, [9], 17, None)]
