"""Tuned-config store (nearest run key, user file shadows the shipped one) and the candidate benchmark split over
the ranks of a gloo group."""
import json
import os
import socket

import torch
import torch.multiprocessing as mp

from lightllm_b200.utils import autotuner as at


def test_store_lookup_and_shadowing(tmp_path, monkeypatch):
    shipped = tmp_path / "pkg"
    monkeypatch.setattr(at, "PKG_DIR", shipped)
    (shipped / "devX").mkdir(parents=True)
    (shipped / "devX" / "gemm_bf16.json").write_text(json.dumps(
        {"N=4096,K=4096,epi=store": {"16": {"bn": 64}, "256": {"bn": 1012}}}))
    st = at.KernelConfigStore(device="devX", user_dir=str(tmp_path / "user"))
    key = at.gemm_static_key(4096, 4096, "store")
    assert st.lookup("gemm_bf16", key, 1)["bn"] == 64 and st.lookup("gemm_bf16", key, 100)["bn"] == 64
    assert st.lookup("gemm_bf16", key, 136)["bn"] == 1012 and st.lookup("gemm_bf16", key, 4000)["bn"] == 1012
    assert st.lookup("gemm_bf16", "N=1,K=1,epi=store", 8) is None
    st.store("gemm_bf16", key, 16, {"bn": 128})          # the user's entry shadows the shipped one
    st.store("gemm_bf16", key, 64, {"bn": 1111})
    st2 = at.KernelConfigStore(device="devX", user_dir=str(tmp_path / "user"))
    assert st2.lookup("gemm_bf16", key, 16)["bn"] == 128 and st2.lookup("gemm_bf16", key, 70)["bn"] == 1111
    assert st2.has("gemm_bf16", key, 64) and not st2.has("gemm_bf16", key, 65)
    at.reset_store(st2)
    try:
        assert at.gemm_lookup(16, 4096, 4096, "store") == 128 and at.gemm_lookup(16, 8, 8, "store") == 0
    finally:
        at.reset_store(None)
    best, scored = at.tune([{"bn": 1}, {"bn": 2}, {"bn": 3}], lambda c: {1: 5.0, 2: 1.0, 3: 9.0}[c["bn"]])
    assert best == {"bn": 2} and [c["bn"] for _, c in scored] == [2, 1, 3]

    def failing(c):
        if c["bn"] == 2:
            raise RuntimeError("unsupported variant")
        return float(c["bn"])

    assert at.tune([{"bn": 1}, {"bn": 2}, {"bn": 3}], failing)[0] == {"bn": 1}


def _rank(rank, world, port, out):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    seen = []

    def bench(c):
        seen.append(c["bn"])
        return abs(c["bn"] - 7) + 0.5

    best, scored = at.tune([{"bn": b} for b in range(12)], bench, group=dist.group.WORLD)
    torch.save({"best": best, "seen": seen, "n": len(scored)}, os.path.join(out, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_candidates_are_split_across_ranks(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "r0.pt"), torch.load(tmp_path / "r1.pt")
    assert a["best"] == b["best"] == {"bn": 7} and a["n"] == b["n"] == 12
    assert sorted(a["seen"] + b["seen"]) == list(range(12)) and not set(a["seen"]) & set(b["seen"])
