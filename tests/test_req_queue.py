"""Past-Future admission arithmetic on hand-computed cases (reference:
lightllm/server/router/req_queue/chunked_prefill/impl.py:12-93)."""
from lightllm_b200.server.core.objs.req import ADDED_OUTPUT_LEN, Req
from lightllm_b200.server.router.req_queue import (Batch, ChunkedBeamContinuesBatchQueue, ChunkedPrefillQueue, PDQueue,
                                                   PeakEstimate, RouterStatics)


def _req(rid, n_in, max_new, chunk=4096, group=None, ignore_eos=True):
    r = Req()
    r.index_in_shm_mem = -1
    r.init(rid, list(range(1, n_in + 1)), {"max_new_tokens": max_new, "ignore_eos": ignore_eos}, None,
           chunked_prefill_size=chunk, router_max_wait_tokens=1, max_total_len=1 << 20)
    if group is not None:
        r.group_req_id = group
    return r


def test_peak_estimate_by_hand():
    # (held, growth): sorted by growth desc -> (10, 50), (30, 20), (5, 5)
    # i=1: 1*50 + 10 = 60; i=2: 2*20 + 40 = 80; i=3: 3*5 + 45 = 60  -> peak 80
    e = PeakEstimate([(30, 20), (10, 50), (5, 5)])
    assert e.peak() == 80 and e.held() == 45 and len(e) == 3
    assert PeakEstimate().peak() == 0
    # one long request dominates: 1*1000 + 1 = 1001 against 2*10 + 101 = 121
    assert PeakEstimate([(1, 1000), (100, 10)]).peak() == 1001


def test_tuple_of_a_fresh_request():
    r = _req(8, 100, 50, chunk=64)
    held, growth = r.get_tuple_tokens(False, 2048)
    # prompt + first token; two prefill chunks of 64 -> 2 * (router_max_wait_tokens + 1) extra steps, + 50 - 0 - 1
    assert held == 101 and growth == 2 * 2 + 49 + ADDED_OUTPUT_LEN
    assert r.get_first_router_need_tokens() == 64 and r.get_decode_need_tokens() == 64


def test_fcfs_admission_stops_at_the_first_misfit():
    # each request: held 101, growth 1*2 + 9 + 16 = 27 (one chunk).  k requests: peak = 27k + 101k = 128k
    q = ChunkedPrefillQueue(max_total_tokens=128 * 3 + 1, batch_max_tokens=4096, running_max_req_size=16)
    reqs = [_req(8 * i, 100, 10) for i in range(5)]
    q.extend(reqs)
    b = q.generate_new_batch(None)
    assert [r.request_id for r in b.reqs] == [0, 8, 16]            # the fourth would need 512 >= 385
    assert q.get_wait_req_num() == 2
    # with the three running nothing more fits; after they finish the rest is admitted
    assert q.generate_new_batch(b) is None
    assert [r.request_id for r in q.generate_new_batch(Batch(1, [])).reqs] == [24, 32]


def test_peak_must_stay_strictly_below_the_pool():
    q = ChunkedPrefillQueue(max_total_tokens=128, batch_max_tokens=4096, running_max_req_size=16)
    q.append(_req(0, 100, 10))
    assert q.generate_new_batch(None) is None                       # peak 128 is not < 128
    q.max_total_tokens = 129
    assert q.generate_new_batch(None) is not None


def test_request_count_limit():
    q = ChunkedPrefillQueue(max_total_tokens=1 << 20, batch_max_tokens=4096, running_max_req_size=3)
    q.extend([_req(8 * i, 10, 4) for i in range(5)])
    running = Batch(0, [_req(800, 10, 4)])
    assert len(q.generate_new_batch(running).reqs) == 2              # 1 running + 2 new = 3
    full = Batch(0, [_req(900 + 8 * i, 10, 4) for i in range(3)])
    assert q.generate_new_batch(full) is None


def test_prompt_budget_starts_from_the_running_batch():
    """New prompts may add up to two forward passes of tokens ON TOP of what the running requests already need in
    the next pass (one token per decoding request, the next chunk of a prompt still in prefill)."""
    q = ChunkedPrefillQueue(max_total_tokens=1 << 24, batch_max_tokens=100, running_max_req_size=1000)
    new = [_req(8 * i, 60, 4, chunk=4096) for i in range(5)]          # 60 prompt tokens each
    q.extend(new)
    assert len(q.generate_new_batch(None).reqs) == 3                 # 180 <= 200 < 240
    # 30 running requests in decode: 30 tokens already owed -> 30 + 120 <= 200 < 30 + 180
    running = []
    for i in range(30):
        r = _req(1000 + 8 * i, 20, 40)
        r.shm_cur_kv_len, r.shm_cur_output_len = 20, 1
        assert r.get_decode_need_tokens() == 1
        running.append(r)
    q2 = ChunkedPrefillQueue(max_total_tokens=1 << 24, batch_max_tokens=100, running_max_req_size=1000)
    q2.extend([_req(8 * i, 60, 4) for i in range(5)])
    assert len(q2.generate_new_batch(Batch(0, running)).reqs) == 2
    # a running request still in chunked prefill owes its next chunk
    big = _req(5000, 500, 4, chunk=150)
    big.shm_cur_kv_len = 150
    assert big.get_decode_need_tokens() == 150
    q3 = ChunkedPrefillQueue(max_total_tokens=1 << 24, batch_max_tokens=100, running_max_req_size=1000)
    q3.extend([_req(8 * i, 60, 4) for i in range(5)])
    assert q3.generate_new_batch(Batch(0, [big])) is None            # 150 + 60 > 200


def test_busy_router_counts_every_request_to_its_limit():
    st = RouterStatics(init_len=64)
    q = ChunkedPrefillQueue(max_total_tokens=1 << 20, batch_max_tokens=4096, running_max_req_size=16,
                            router_token_ratio=0.5, statics=st)
    r = _req(0, 100, 1000, ignore_eos=False)
    q.cur_token_usage_ratio = 0.1
    assert q._tuple_of(r, q.is_busy())[1] == 2 + 63 + ADDED_OUTPUT_LEN     # expects the moving average (64)
    q.cur_token_usage_ratio = 0.9
    assert q.is_busy() and q._tuple_of(r, True)[1] == 2 + 999 + ADDED_OUTPUT_LEN
    for n in (10, 10, 10, 10):
        st.update(n)
    assert st.ema_req_out_len == st.floor == 64                              # never below the floor


def test_aborted_waiting_requests_are_skipped_and_returned():
    q = ChunkedPrefillQueue(max_total_tokens=1 << 20, batch_max_tokens=4096, running_max_req_size=16)
    reqs = [_req(8 * i, 10, 4) for i in range(3)]
    reqs[1].is_aborted = True
    q.extend(reqs)
    assert [r.request_id for r in q.pop_aborted()] == [8]
    assert [r.request_id for r in q.generate_new_batch(None).reqs] == [0, 16]


def test_pd_queue_counts_a_new_request_at_full_length():
    q = PDQueue(max_total_tokens=1 << 20, batch_max_tokens=4096, running_max_req_size=16)
    assert q._tuple_of(_req(0, 100, 50, ignore_eos=False), False) == (101, 66)


def test_group_queue_admits_whole_groups_and_counts_the_prompt_once():
    q = ChunkedBeamContinuesBatchQueue(max_total_tokens=1 << 20, batch_max_tokens=100, running_max_req_size=5)
    g1 = [_req(0 + i, 120, 4, group=0) for i in range(3)]            # one prompt of 120 tokens, 3 samples
    g2 = [_req(8 + i, 70, 4, group=8) for i in range(3)]
    q.extend(g1 + g2)
    b = q.generate_new_batch(None)
    # group 1 fits (120 prompt tokens counted once, not 360); group 2 would exceed 5 requests -> rejected as a whole
    assert [r.request_id for r in b.reqs] == [0, 1, 2] and q.get_wait_req_num() == 3
