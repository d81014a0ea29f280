"""Shared-memory request objects: slot manager, cross-process locks, the out-token ring and the router -> rank
mailbox, each exercised from two processes.  Invariants follow the reference's unit tests
(unit_tests/server/core/objs/test_shm_req_manager.py, test_atomic_lock.py, test_atomic_array_lock.py,
test_out_token_circlequeue.py)."""
import multiprocessing as mp
import os
import time
import uuid

import pytest

from lightllm_b200.server.core.objs.atomic_lock import (AtomicShmArrayLock, AtomicShmLock, LockTimeout, SharedArray,
                                                        SharedInt)
from lightllm_b200.server.core.objs.req import LIGHTLLM_OUT_TOKEN_QUEUE_SIZE, OutTokenRing, Req
from lightllm_b200.server.core.objs.shm_objs_io_buffer import ShmObjsIOBuffer
from lightllm_b200.server.core.objs.shm_req_manager import ShmReqManager


def _name():
    return f"llbt{os.getpid()}x{uuid.uuid4().hex[:6]}"


# ---------------------------------------------------------------- out-token ring
def test_ring_order_capacity_and_wrap():
    q = OutTokenRing()
    q.reset()
    assert q.is_empty() and len(q) == 0
    with pytest.raises(BufferError):
        q.peek()
    with pytest.raises(BufferError):
        q.pop_no_ret()
    n = LIGHTLLM_OUT_TOKEN_QUEUE_SIZE
    for i in range(n):                       # every slot is usable
        q.push(f"tok{i}", 100 + i, i % 2 == 0, i + 1)
    assert q.is_full() and len(q) == n
    with pytest.raises(BufferError):
        q.push("x", 0, False, 0)
    assert q.peek() == ("tok0", 100, True, 1) and len(q) == n       # peek does not consume
    for i in range(n):
        assert q.pop() == (f"tok{i}", 100 + i, i % 2 == 0, i + 1)
    assert q.is_empty()
    q.consumed = q.produced = q.WRAP - 3     # counters about to wrap
    for r in range(3 * n):
        q.push(f"w{r}", r, False, r)
        q.push(f"v{r}", r, True, r)
        assert q.pop()[0] == f"w{r}" and q.pop()[0] == f"v{r}"
    assert q.is_empty() and q.produced < 3 * n * 2


def test_ring_text_is_utf8_and_truncated():
    from lightllm_b200.server.core.objs.req import LIGHTLLM_TOKEN_MAX_BYTES

    q = OutTokenRing()
    q.reset()
    q.push("héllo 世界", 1, False, 1)
    assert q.pop()[0] == "héllo 世界"
    q.push("a" * (LIGHTLLM_TOKEN_MAX_BYTES + 50), 2, False, 2)
    assert len(q.pop()[0]) == LIGHTLLM_TOKEN_MAX_BYTES


def _ring_consumer(server, idx, n, out):
    mgr = ShmReqManager(server, max_req_num=4, req_class=Req)
    r = mgr.get_req_obj_by_index(idx)
    got, t0 = [], time.time()
    while len(got) < n and time.time() - t0 < 60:
        if not r.out_tokens_queue.is_empty():
            got.append(r.out_tokens_queue.pop())
    mgr.put_back_req_obj(r)
    out.put(got)


def test_ring_between_two_processes_through_the_shared_request():
    server = _name()
    mgr = ShmReqManager(server, max_req_num=4, req_class=Req)
    try:
        idx = mgr.alloc_req_index()
        r = mgr.get_req_obj_by_index(idx)
        r.out_tokens_queue.reset()
        ctx = mp.get_context("spawn")
        out = ctx.Queue()
        n = 200
        p = ctx.Process(target=_ring_consumer, args=(server, idx, n, out))
        p.start()
        sent = 0
        t0 = time.time()
        while sent < n and time.time() - t0 < 60:
            if not r.out_tokens_queue.is_full():
                r.out_tokens_queue.push(f"t{sent}", sent, False, sent + 1)
                sent += 1
        got = out.get(timeout=60)
        p.join(30)
        assert got == [(f"t{i}", i, False, i + 1) for i in range(n)]     # nothing lost, duplicated or reordered
        assert mgr.put_back_req_obj(r) == 0
    finally:
        mgr.close(unlink=True)


# ---------------------------------------------------------------- locks and counters
def _adder(lock_name, counter_name, n, use_lock):
    lock = AtomicShmLock(lock_name)
    arr = SharedArray(counter_name, (1,), "int64")
    for _ in range(n):
        if use_lock:
            with lock:
                arr.arr[0] = arr.arr[0] + 1
        else:
            arr.arr[0] = arr.arr[0] + 1


def test_lock_makes_read_modify_write_safe_across_processes():
    ln, cn = _name() + "_l", _name() + "_c"
    lock = AtomicShmLock(ln)
    arr = SharedArray(cn, (1,), "int64")
    ctx = mp.get_context("spawn")
    n = 3000
    ps = [ctx.Process(target=_adder, args=(ln, cn, n, True)) for _ in range(3)]
    [p.start() for p in ps]
    [p.join(120) for p in ps]
    assert int(arr.arr[0]) == 3 * n
    for s in (lock.shm, arr.shm):
        s.close()
        s.unlink()


def test_lock_timeout_and_forced_release():
    lock = AtomicShmLock(_name() + "_t", timeout_s=0.2)
    other = AtomicShmLock(lock.lock_name, timeout_s=0.2)    # a second view of the same word
    lock.acquire()
    t0 = time.time()
    with pytest.raises(LockTimeout):
        other.acquire()                                      # bounded wait, not a hang
    assert 0.15 < time.time() - t0 < 5
    other.force_release()                                    # supervisor knows the holder died
    with other:
        pass
    lock.shm.close()
    other.shm.close()
    other.shm.unlink()


def test_array_lock_slots_are_independent():
    locks = AtomicShmArrayLock(_name() + "_a", 4, timeout_s=0.2)
    with locks.get_lock_context(1):
        with locks.get_lock_context(2):                      # another slot: no contention
            pass
        with pytest.raises(LockTimeout):
            with locks.get_lock_context(1):                  # same slot: held
                pass
    with locks.get_lock_context(1):
        pass
    with pytest.raises(AssertionError):
        locks.get_lock_context(4)
    locks.shm.close()
    locks.shm.unlink()


def _shared_int_adder(name, n):
    v = SharedInt(name)
    for _ in range(n):
        v.add(1)


def test_shared_int_atomic_add_across_processes():
    name = _name() + "_i"
    v = SharedInt(name, init=5)
    ctx = mp.get_context("spawn")
    ps = [ctx.Process(target=_shared_int_adder, args=(name, 5000)) for _ in range(3)]
    [p.start() for p in ps]
    [p.join(120) for p in ps]
    assert v.get_value() == 5 + 15000
    v.shm.close()
    v.shm.unlink()


# ---------------------------------------------------------------- request slots
def _slot_worker(server, q_in, q_out):
    mgr = ShmReqManager(server, max_req_num=4, req_class=Req)
    idx = q_in.get(timeout=60)
    r = mgr.get_req_obj_by_index(idx)
    q_out.put((r.request_id, r.ref_count, r.index_in_shm_mem))
    q_in.get(timeout=60)                 # wait until told to let go
    q_out.put(mgr.put_back_req_obj(r))
    mgr.close()


def test_req_manager_slots_refcounts_and_visibility():
    server = _name()
    mgr = ShmReqManager(server, max_req_num=4, req_class=Req)
    try:
        assert mgr.free_count() == 4
        idxs = [mgr.alloc_req_index() for _ in range(4)]
        assert sorted(idxs) == [0, 1, 2, 3] and mgr.alloc_req_index() is None     # exhausted -> None, no raise
        r = mgr.get_req_obj_by_index(idxs[0])
        assert r.ref_count == 1 and r.index_in_shm_mem == idxs[0]
        r.request_id = 4242
        ctx = mp.get_context("spawn")
        q_in, q_out = ctx.Queue(), ctx.Queue()
        p = ctx.Process(target=_slot_worker, args=(server, q_in, q_out))
        p.start()
        q_in.put(idxs[0])
        assert q_out.get(timeout=60) == (4242, 2, idxs[0])      # the other process sees the write and the count
        with pytest.raises(AssertionError):
            mgr.release_req_index(idxs[0])                       # still referenced
        q_in.put("go")
        assert q_out.get(timeout=60) == 1
        p.join(30)
        assert mgr.put_back_req_obj(r) == 0
        mgr.release_req_index(idxs[0])
        assert mgr.free_count() == 1 and mgr.alloc_req_index() == idxs[0]
        second = ShmReqManager(server, max_req_num=4, req_class=Req)   # linking must not re-initialise the free list
        assert second.free_count() == 0
        second.close()
    finally:
        mgr.close(unlink=True)


# ---------------------------------------------------------------- router -> rank mailbox
def _mailbox_reader(name, n_msgs, out, world):
    box = ShmObjsIOBuffer(name, world, size=1 << 20)
    seen, gen, t0 = [], 0, time.time()
    while len(seen) < n_msgs and time.time() - t0 < 60:
        g = box.generation()
        if g != gen and box.is_ready():
            seen.append(box.read_obj())
            gen = g
            box.sub_state()
    out.put(seen)


def test_mailbox_every_reader_sees_every_message_once():
    name = _name() + "_mb"
    world = 2
    box = ShmObjsIOBuffer(name, world, size=1 << 20)
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    msgs = [{"seq": i, "payload": list(range(i))} for i in range(25)]
    ps = [ctx.Process(target=_mailbox_reader, args=(name, len(msgs), out, world)) for _ in range(world)]
    [p.start() for p in ps]
    t0 = time.time()
    for m in msgs:
        while not box.is_empty():             # the writer only overwrites a fully consumed message
            assert time.time() - t0 < 60
        box.write_obj(m)
        box.set_ready()
    got = [out.get(timeout=60) for _ in range(world)]
    [p.join(30) for p in ps]
    assert got[0] == msgs and got[1] == msgs
    assert box.is_empty() and box.generation() == len(msgs)
    with pytest.raises(ValueError):
        box.write_obj(b"x" * (2 << 20))       # larger than the buffer: refused, not truncated
    box.shm.close()
    box.shm.unlink()


def _racer(i, name, n_rounds, barrier, out):
    from lightllm_b200.server.core.objs.shm_array import create_or_link_shm

    bad = 0
    for r in range(n_rounds):
        barrier.wait()
        shm, created = create_or_link_shm(f"{name}_{r}", 4096)
        shm.buf[i] = i + 1
        barrier.wait()
        if bytes(shm.buf[:4]) != bytes([1, 2, 3, 4]):      # everybody landed in the same segment
            bad += 1
        barrier.wait()
        shm.close()
        if created:
            try:
                shm.unlink()
            except FileNotFoundError:
                pass
    out.put((i, bad))


def test_processes_that_start_together_share_one_segment():
    """Processes of a server start side by side: whoever loses the creation race must wait for the winner to size
    the segment, not replace it (a freshly created POSIX segment is empty for an instant)."""
    import multiprocessing as mp
    import os

    ctx = mp.get_context("spawn")
    barrier, out = ctx.Barrier(4), ctx.Queue()
    name = f"llb_race_{os.getpid()}"
    ps = [ctx.Process(target=_racer, args=(i, name, 40, barrier, out)) for i in range(4)]
    for p in ps:
        p.start()
    res = sorted(out.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(timeout=30)
    assert res == [(0, 0), (1, 0), (2, 0), (3, 0)]
