"""Watchdog / retry / moving average, shared-memory cleanup, the workspace sub-allocator and the token-capacity
estimate."""
import json
import os
import subprocess
import sys
import time

import pytest
import torch

from lightllm_b200.utils.tensor_buffer import TensorBufferManager
from lightllm_b200.utils.watchdog import MovingAverage, TimeChecker, Watchdog, retry


def test_watchdog_fires_only_without_heartbeat():
    hits = []
    w = Watchdog(1.0, on_timeout=lambda: hits.append(time.monotonic()), poll=0.05).start()
    for _ in range(8):
        time.sleep(0.05)
        w.heartbeat()
    assert not hits
    time.sleep(1.6)
    w.stop()
    assert 1 <= len(hits) <= 2


def test_retry_and_moving_average():
    calls = []

    @retry(max_attempts=3, wait_time=0.0)
    def flaky():
        calls.append(1)
        if len(calls) < 3:
            raise ValueError("not yet")
        return "ok"

    assert flaky() == "ok" and len(calls) == 3

    @retry(max_attempts=2, wait_time=0.0)
    def broken():
        raise KeyError("x")

    with pytest.raises(RuntimeError) as e:
        broken()
    assert isinstance(e.value.__cause__, KeyError)
    m = MovingAverage()
    for v in (1, 2, 3, 6):
        m.add(v)
    assert m.average() == 3.0
    t = TimeChecker(0.05)
    assert not t.has_exceeded()
    time.sleep(0.07)
    assert t.has_exceeded() and not t.has_exceeded()


def test_tensor_buffer_alignment_reuse_and_merging():
    ws = torch.empty(64 * 1024 + 100, dtype=torch.uint8)
    m = TensorBufferManager(ws, alignment_bytes=256)
    a = m.alloc((10, 7), torch.float32)
    b = m.alloc(1000, torch.bfloat16)
    c = m.alloc((3, 5, 2), torch.int64)
    for t in (a, b, c):
        assert t.data_ptr() % 256 == 0 and t.is_contiguous()
    a.fill_(1.0), b.fill_(2.0), c.fill_(3)
    assert float(a.sum()) == 70 and float(b.float().sum()) == 2000 and int(c.sum()) == 90   # no overlap
    used = m.capacity - m.free_bytes
    assert used == 512 + 2048 + 256
    m.free(b)
    assert m.alloc(900, torch.bfloat16).data_ptr() == b.data_ptr()       # best fit: the hole it left
    m.free(a)
    with pytest.raises(ValueError):
        m.free(a)
    m.reset()
    big = m.alloc(m.capacity, torch.uint8)
    with pytest.raises(MemoryError):
        m.alloc(1, torch.uint8)
    m.free(big)
    x, y, z = (m.alloc(256, torch.uint8) for _ in range(3))
    m.free(x), m.free(z), m.free(y)                                       # out of order: ranges merge back
    assert m.largest_free_block == m.capacity
    assert m.alloc((0, 4), torch.float32).numel() == 0


def test_shm_segments_are_removed_when_the_creator_is_terminated(tmp_path):
    name = f"llb_cleanup_test_{os.getpid()}"
    code = f"""
import os, signal, sys, time
from multiprocessing import shared_memory, resource_tracker
from lightllm_b200.utils.shm_cleanup import get_cleanup, register_posix_shm_for_cleanup
get_cleanup(signals=True)
s = shared_memory.SharedMemory(name={name!r}, create=True, size=4096)
resource_tracker.unregister(s._name, "shared_memory")     # only our own registry may remove it
register_posix_shm_for_cleanup({name!r})
print("ready", flush=True)
time.sleep(30)
"""
    p = subprocess.Popen([sys.executable, "-c", code], stdout=subprocess.PIPE, cwd=os.getcwd())
    assert p.stdout.readline().strip() == b"ready"
    assert os.path.exists("/dev/shm/" + name)
    p.terminate()
    p.wait(timeout=10)
    assert not os.path.exists("/dev/shm/" + name)


def test_shm_size_recommendation():
    from types import SimpleNamespace

    from lightllm_b200.utils.shm_cleanup import check_shm_size, recommended_shm_gib

    small = SimpleNamespace(running_max_req_size=100, max_req_total_len=4096)
    big = SimpleNamespace(running_max_req_size=100, max_req_total_len=4096, enable_multimodal=True, cache_capacity=10,
                          embed_cache_storage_size=4, enable_cpu_cache=True, cpu_cache_storage_size=8)
    assert recommended_shm_gib(small) < 0.01
    assert 12 < recommended_shm_gib(big) < 13
    have, want, ok = check_shm_size(small)
    assert ok == (have >= want)


def test_token_capacity_estimate(tmp_path):
    from safetensors.torch import save_file

    from lightllm_b200.utils.profile_max_tokens import kv_bytes_per_token, max_total_tokens, safetensors_bytes

    cfg = dict(model_type="llama", hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
               num_key_value_heads=8, vocab_size=128256)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({"a": torch.zeros(1024, 1024, dtype=torch.bfloat16), "b": torch.zeros(512, dtype=torch.float32)},
              str(tmp_path / "model.safetensors"))
    total, by = safetensors_bytes(str(tmp_path))
    assert total == 2 * 1024 * 1024 + 2048 and by == {"BF16": 2 * 1024 * 1024, "F32": 2048}
    assert kv_bytes_per_token(cfg, 1) == 32 * 2 * 8 * 128 * 2          # 128 KiB per token for Llama-3-8B
    assert kv_bytes_per_token(cfg, 8) == 32 * 2 * 1 * 128 * 2
    assert kv_bytes_per_token(cfg, 16) == kv_bytes_per_token(cfg, 8)     # heads replicated beyond 8 ranks
    mla = dict(num_hidden_layers=61, num_attention_heads=128, kv_lora_rank=512, qk_rope_head_dim=64, hidden_size=7168)
    assert kv_bytes_per_token(mla, 8) == 61 * 576 * 2
    hybrid = dict(num_hidden_layers=48, num_attention_heads=16, num_key_value_heads=2, head_dim=256, hidden_size=2048,
                  full_attention_interval=4, linear_num_key_heads=16)
    assert kv_bytes_per_token(hybrid, 1) == 12 * 2 * 2 * 256 * 2
    r = max_total_tokens(str(tmp_path), tp=1, mem_fraction=0.5, gpu_gib=1.0)
    assert r["max_total_token_num"] == int((0.5 * 2 ** 30 - total) // (128 * 1024))


def test_compatibility_only_flags_are_reported():
    from lightllm_b200.server.api_cli import COMPAT_ONLY_FLAGS, FLAGS, compat_only_flags_in_use, make_argument_parser

    known = {f[0].lstrip("-") for f in FLAGS}
    assert set(COMPAT_ONLY_FLAGS) <= known
    p = make_argument_parser()
    assert compat_only_flags_in_use(p.parse_args(["--model_dir", "/x"])) == []
    used = compat_only_flags_in_use(p.parse_args(["--model_dir", "/x", "--enable_mps", "--pd_trans_mode", "nixl"]))
    assert sorted(used) == ["enable_mps", "pd_trans_mode"]


def test_env_knobs_of_the_reference(monkeypatch):
    """NTK alpha raises the rotary base; the websocket size limit and the TGI list wrapper follow their variables."""
    import importlib

    import torch

    from lightllm_b200.engine.llm import LLM
    from lightllm_b200.ops import reference as ref
    from lightllm_b200.server.httpserver import pd_loop

    cfg = dict(model_type="llama", hidden_size=64, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2,
               head_dim=32, intermediate_size=128, vocab_size=128, rms_norm_eps=1e-6, rope_theta=1e4, eos_token_id=2)
    kw = dict(data_type="float32", max_total_token_num=256, running_max_req_size=2, max_req_total_len=64, batch_max_tokens=64)
    plain = LLM(config=cfg, **kw).model
    monkeypatch.setenv("LIGHTLLM_NTK_ALPHA", "4")
    ntk = LLM(config=cfg, **kw).model
    want_cos, _ = ref.build_rope_cache(plain.cos.shape[0], 32, 1e4 * 4 ** (32 / 30), None, device=torch.device("cpu"))
    assert torch.allclose(ntk.cos, want_cos) and not torch.allclose(ntk.cos, plain.cos)
    monkeypatch.delenv("LIGHTLLM_WEBSOCKET_MAX_SIZE", raising=False)
    assert pd_loop.ws_max_size() is None
    monkeypatch.setenv("LIGHTLLM_WEBSOCKET_MAX_SIZE", "1048576")
    assert pd_loop.ws_max_size() == 1 << 20
    from lightllm_b200.server import api_tgi

    monkeypatch.setenv("RETURN_LIST", "1")
    assert importlib.reload(api_tgi).RETURN_LIST is True
    monkeypatch.delenv("RETURN_LIST")
    assert importlib.reload(api_tgi).RETURN_LIST is False


def test_loggers_follow_the_environment(monkeypatch, tmp_path, capsys):
    import logging

    from lightllm_b200.utils import log_utils

    log_utils.reset_for_tests()
    monkeypatch.setenv("LIGHTLLM_LOG_LEVEL", "warning")
    monkeypatch.setenv("LIGHTLLM_LOG_DIR", str(tmp_path / "logs"))
    lg = log_utils.init_logger("lightllm_b200.server.somewhere")
    assert lg is log_utils.init_logger("lightllm_b200.server.somewhere") and lg.name == "lightllm_b200.server.somewhere"
    lg.info("quiet")
    lg.warning("loud %d", 7)
    out = capsys.readouterr().out
    assert "loud 7" in out and "quiet" not in out and "WARNING" in out and "server.somewhere" in out
    files = list((tmp_path / "logs").iterdir())
    assert len(files) == 1 and "loud 7" in files[0].read_text()
    log_utils.reset_for_tests()
    monkeypatch.setenv("LLB_LOG_LEVEL", "10")
    monkeypatch.delenv("LIGHTLLM_LOG_DIR")
    assert log_utils.log_level() == logging.DEBUG
    monkeypatch.setenv("LLB_LOG_LEVEL", "nonsense")
    assert log_utils.log_level() == logging.INFO
    log_utils.reset_for_tests()


def test_orphan_shared_memory_segments(tmp_path, monkeypatch):
    from lightllm_b200.utils import shm_cleanup as sc

    names = ["llb111xabcdef_req_shm_total", "llb111xabcdef_token_load", "llb222x012345_req_shm_total",
             "llb333xdeadbe_shm_prompts_0", "psm_1234", "llbXYZ_notours", "llb111xabcdef"]
    for n in names:
        (tmp_path / n).write_bytes(b"x")
    alive = lambda pid: pid == 222  # noqa: E731
    found = sc.orphan_segments(str(tmp_path), alive)
    assert {k: sorted(v) for k, v in found.items()} == {
        "llb111xabcdef": ["llb111xabcdef_req_shm_total", "llb111xabcdef_token_load"],
        "llb333xdeadbe": ["llb333xdeadbe_shm_prompts_0"]}
    assert sc.sweep_orphans(str(tmp_path), alive) == 3
    assert sorted(p.name for p in tmp_path.iterdir()) == sorted(["llb222x012345_req_shm_total", "psm_1234",
                                                                 "llbXYZ_notours", "llb111xabcdef"])
    # this process is alive: its own segments are never listed
    (tmp_path / f"llb{os.getpid()}xabc123_x").write_bytes(b"x")
    assert f"llb{os.getpid()}xabc123" not in sc.orphan_segments(str(tmp_path))
    monkeypatch.delenv("LLB_SWEEP_ORPHAN_SHM", raising=False)
    assert sc.note_or_sweep_orphans(str(tmp_path)) == 0


def test_a_busy_http_port_stops_the_launcher_before_anything_starts(tmp_path):
    import socket
    import subprocess

    from lightllm_b200.utils.net_utils import port_is_free, require_free_ports

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    s.listen(1)
    port = s.getsockname()[1]
    try:
        assert not port_is_free("127.0.0.1", port)
        with pytest.raises(SystemExit) as e:
            require_free_ports("127.0.0.1", [port, None], "HTTP server")
        assert str(port) in str(e.value)
        (tmp_path / "config.json").write_text("{}")
        t0 = time.time()
        r = subprocess.run([sys.executable, "-m", "lightllm_b200.server.api_server", "--model_dir", str(tmp_path),
                            "--host", "127.0.0.1", "--port", str(port)], capture_output=True, text=True, timeout=120,
                           env=dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=os.path.dirname(os.path.dirname(__file__))))
        assert r.returncode != 0 and "in use" in (r.stderr + r.stdout) and time.time() - t0 < 60
    finally:
        s.close()
    assert port_is_free("127.0.0.1", port)
    require_free_ports("127.0.0.1", [port])
