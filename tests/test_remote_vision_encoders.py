"""Vision encoders as their own service (`--run_mode visual_only`) and servers that use them
(`--visual_use_proxy_mode`): the shared embedding directory, the request protocol with a stand-in tower, fail-over
and failure handling, and the three kinds of processes together on CPU."""
import base64
import json
import os
import signal
import subprocess
import sys
import threading
import time
from types import SimpleNamespace

import pytest
import requests
import torch
import zmq

from lightllm_b200.server.core.objs.io_objs import GroupReqIndexes
from lightllm_b200.server.visualserver import remote

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shared_embed_dir(tmp_path):
    d = remote.SharedEmbedDir(str(tmp_path / "emb"), capacity=3)
    assert d.load("aa11") is None and not d.has("aa11")
    for i, k in enumerate(["aa11", "ab22", "cc33"]):
        d.store(k, torch.full((2, 4), float(i), dtype=torch.bfloat16))
        os.utime(d._path(k), (1000 + i, 1000 + i))
    got = d.load("aa11")                       # a read makes it the most recent one
    assert got.dtype == torch.bfloat16 and torch.equal(got, torch.zeros(2, 4, dtype=torch.bfloat16))
    d.store("dd44", torch.ones(1, 4))          # over capacity: the least recently used file goes
    assert d.has("aa11") and not d.has("ab22") and d.has("cc33") and d.has("dd44")
    assert not [f for sub in os.listdir(d.root) for f in os.listdir(os.path.join(d.root, sub)) if f.endswith(".part")]
    open(d._path("cc33"), "wb").write(b"torn")  # an unreadable file is a miss, not an error
    assert d.load("cc33") is None
    d.store("", torch.ones(1))                  # items without a content hash are not kept
    assert remote.shared_dir_of(SimpleNamespace(afs_image_embed_dir=None)) is None


class _Tower:
    """Embedding = the payload's bytes repeated over `token_num` rows."""

    out_hidden = 4

    def __init__(self):
        self.calls = []

    def encode_images(self, payloads, items=None):
        self.calls.append(len(payloads))
        return [torch.tensor(list(p[:4]), dtype=torch.float32).repeat(it["token_num"], 1) for p, it in zip(payloads, items)]


class _Cache:
    def __init__(self, payloads):
        self.payloads, self.ready, self.rows = payloads, set(), {}
        self.arena = SimpleNamespace(write=lambda start, e: self.rows.__setitem__(start, e.clone()))

    def get_items_embed(self, ids):
        return [i in self.ready for i in ids]

    def set_items_embed(self, ids):
        self.ready.update(ids)

    def get_payload(self, uid):
        return self.payloads[uid]


def _encoder(tower, shared=None):
    sock = zmq.Context.instance().socket(zmq.ROUTER)
    port = sock.bind_to_random_port("tcp://127.0.0.1")
    srv = remote.VisualOnlyServer(tower, sock, shared, infer_batch_size=2)
    stop = threading.Event()
    th = threading.Thread(target=srv.loop, args=(stop,), daemon=True)
    th.start()
    return srv, port, stop, th


def _item(uid, md5, n, start):
    return {"uuid": uid, "md5": md5, "token_num": n, "start_index_in_embed_cache": start, "token_id": 10 ** 8 + start}


def test_proxy_asks_encoders_and_reuses_the_shared_directory(tmp_path):
    shared = remote.SharedEmbedDir(str(tmp_path / "emb"))
    tower = _Tower()
    srv, port, stop, th = _encoder(tower, shared)
    dead = zmq.Context.instance().socket(zmq.ROUTER)       # registered, never answers
    dead_port = dead.bind_to_random_port("tcp://127.0.0.1")
    listed = [remote.VitNode(1, "127.0.0.1", port)]
    enc = remote.RemoteEncoders(None, None, fetch=lambda: list(listed))
    cache = _Cache({1: b"abcdX", 2: b"efghY", 3: b"ijklZ"})
    sent = []
    args = SimpleNamespace(afs_image_embed_dir=None)
    vm = remote.ProxyVisualManager(args, cache, sent.append, None, infer_batch_size=2, encoders=enc, shared=shared,
                                   timeout_s=1.0)
    try:
        g1 = GroupReqIndexes(8, {"images": [_item(1, "m1", 3, 0), _item(2, "m2", 2, 3)], "audios": []}, [0], 0.0)
        g2 = GroupReqIndexes(16, {"images": [_item(3, "m3", 1, 5), _item(1, "m1", 3, 0)], "audios": []}, [1], 0.0)
        vm.handle_many([g1, "control", g2])
        assert sent == [g1, "control", g2] and cache.ready == {1, 2, 3}
        assert torch.equal(cache.rows[0], torch.tensor([97., 98., 99., 100.]).repeat(3, 1))
        assert torch.equal(cache.rows[5], torch.tensor([105., 106., 107., 108.]).repeat(1, 1))
        assert tower.calls == [2, 1] and srv.served == 3      # three pictures, batches of two
        assert shared.has("m1") and shared.has("m2") and shared.has("m3")
        # another server (fresh cache records) meets the same pictures: no encoder is asked
        cache2 = _Cache({7: b"abcdX"})
        vm2 = remote.ProxyVisualManager(args, cache2, sent.append, None, encoders=remote.RemoteEncoders(
            None, None, fetch=lambda: []), shared=shared, timeout_s=1.0)
        vm2.handle_many([GroupReqIndexes(24, {"images": [_item(7, "m1", 3, 9)], "audios": []}, [2], 0.0)])
        assert cache2.ready == {7} and torch.equal(cache2.rows[9], cache.rows[0]) and srv.served == 3
        # fail-over: a registered encoder that never answers is given up after the limit and the other one is asked
        listed.insert(0, remote.VitNode(2, "127.0.0.1", dead_port))
        enc.refresh(force=True)
        assert set(enc.nodes) == {1, 2}
        cache.payloads[4] = b"mnopW"
        for _ in range(3):     # whichever is picked first, the request ends on the live one
            cache.ready.discard(4)
            os.path.exists(shared._path("m4")) and os.unlink(shared._path("m4"))
            vm.handle_many([GroupReqIndexes(32, {"images": [_item(4, "m4", 2, 20)], "audios": []}, [3], 0.0)])
            assert 4 in cache.ready
            enc.refresh(force=True)
        # a sender with another key gets no answer and the tower is not run for it
        before = len(tower.calls)
        stranger = remote.ProxyVisualManager(args, _Cache({8: b"uvwxU"}), sent.append, None, encoders=enc, shared=None,
                                             timeout_s=0.5, key=b"k" * 32)
        try:
            stranger._ask(1, [(_item(8, "m8", 1, 40), b"uvwxU")])
            raise AssertionError("a request signed with another key was answered")
        except TimeoutError:
            pass
        assert len(tower.calls) == before
        # an encoder that dies while a request waits for it: it leaves the list, the wait ends long before the limit
        listed.insert(0, remote.VitNode(2, "127.0.0.1", dead_port))
        enc.refresh(force=True)
        slow = remote.ProxyVisualManager(args, cache, sent.append, None, encoders=enc, shared=None, timeout_s=30.0)
        slow.LOOK_EVERY_S = 0.2
        listed[:] = [remote.VitNode(1, "127.0.0.1", port)]          # what the config server says from now on
        t0 = time.time()
        try:
            slow._ask(2, [(_item(9, "m9", 1, 50), b"zzzzZ")])
            raise AssertionError("a dead encoder answered")
        except ConnectionError as e:
            assert "no longer registered" in str(e) and time.time() - t0 < 5
        # an encoder that leaves the list is dropped
        listed[:] = [remote.VitNode(1, "127.0.0.1", port)]
        enc.refresh(force=True)
        assert set(enc.nodes) == {1}
        # the tower's answer does not fit the reserved rows: an error reply, the request is marked aborted
        aborted = []
        vm.shm_req_manager = SimpleNamespace(get_req_obj_by_index=lambda i: SimpleNamespace(index=i, is_aborted=False),
                                             put_back_req_obj=lambda r: aborted.append((r.index, r.is_aborted)))
        cache.payloads[5] = b"qrstV"
        tower.encode_images = lambda payloads, items=None: [torch.zeros(it["token_num"] + 1, 4) for it in items]
        g5 = GroupReqIndexes(40, {"images": [_item(5, "m5", 2, 30)], "audios": []}, [4, 5], 0.0)
        vm.handle_many([g5])
        assert sent[-1] is g5 and aborted == [(4, True), (5, True)] and 5 not in cache.ready
        # no encoder at all: the same ending
        enc2 = remote.RemoteEncoders(None, None, fetch=lambda: [])
        vm.encoders, aborted[:] = enc2, []
        vm.handle_many([g5])
        assert aborted == [(4, True), (5, True)]
    finally:
        stop.set()
        th.join(timeout=5)
        enc.close()
        srv.sock.close(0)
        dead.close(0)


def _free_port():
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _wait_http(url, proc, log_path, limit=240):
    t0 = time.time()
    while time.time() - t0 < limit and proc.poll() is None:
        try:
            if requests.get(url, timeout=2).status_code == 200:
                return
        except Exception:
            time.sleep(1)
    pytest.fail(f"{url} did not come up:\n" + open(log_path).read()[-3000:])


@pytest.mark.timeout(1200)
def test_config_server_encoder_and_proxy_server_together(tmp_path):
    from test_multimodal_e2e import CFG, _png, offline_tokens

    d = tmp_path / "vl"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(CFG))
    shared = tmp_path / "shared_embeds"
    cport, vport, port = _free_port(), _free_port(), _free_port()
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT, LLB_REMOTE_VIT_TIMEOUT_S="60")
    procs = []

    def spawn(name, argv):
        log = open(tmp_path / f"{name}.log", "w")
        p = subprocess.Popen([sys.executable, "-m", "lightllm_b200.server.api_server"] + argv, env=env, stdout=log,
                             stderr=subprocess.STDOUT, cwd=ROOT, start_new_session=True)
        procs.append(p)
        return p

    try:
        cs = spawn("config", ["--run_mode", "config_server", "--config_server_host", "127.0.0.1",
                              "--config_server_port", str(cport)])
        _wait_http(f"http://127.0.0.1:{cport}/liveness", cs, tmp_path / "config.log")
        where = ["--config_server_host", "127.0.0.1", "--config_server_port", str(cport)]
        spawn("encoder", ["--run_mode", "visual_only", "--model_dir", str(d), "--host", "127.0.0.1", "--visual_rpyc_port",
                          str(vport), "--afs_image_embed_dir", str(shared), "--data_type", "fp32"] + where)
        srv = spawn("server", ["--model_dir", str(d), "--host", "127.0.0.1", "--port", str(port), "--data_type", "fp32",
                               "--max_total_token_num", "4096", "--running_max_req_size", "8", "--max_req_total_len",
                               "256", "--tp", "1", "--embed_cache_storage_size", "0.01", "--visual_use_proxy_mode",
                               "--afs_image_embed_dir", str(shared)] + where)
        url = f"http://127.0.0.1:{port}"
        _wait_http(url + "/liveness", srv, tmp_path / "server.log")
        t0 = time.time()          # the encoder registers on its own schedule
        while time.time() - t0 < 240:
            import pickle

            listed = pickle.loads(base64.b64decode(
                requests.get(f"http://127.0.0.1:{cport}/registered_visual_objects", timeout=5).json()["data"]))
            if listed:
                break
            time.sleep(1)
        assert listed and listed[0].port == vport, open(tmp_path / "encoder.log").read()[-3000:]

        raw = _png(84, 56)
        pre, post = [5, 17, 33], [9, 44, 120, 7]
        body = {"inputs": pre + [290] + post,
                "parameters": {"max_new_tokens": 5, "ignore_eos": True, "return_details": True},
                "multimodal_params": {"images": [{"type": "base64", "data": base64.b64encode(raw).decode()}]}}
        r = requests.post(url + "/generate", json=body, timeout=300)
        logs = "".join(open(tmp_path / f"{n}.log").read()[-2000:] for n in ("server", "encoder"))
        assert r.status_code == 200, r.text + logs
        assert [tk["id"] for tk in r.json()["tokens"]] == offline_tokens(raw, pre, post), logs
        files = [f for sub in os.listdir(shared) for f in os.listdir(shared / sub)]
        assert len(files) == 1 and files[0].endswith(".pt")
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
