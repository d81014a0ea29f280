"""Host memory of the CPU KV tier: huge-page request with fallback, NUMA placement helpers, pre-faulting, tensor
views; and the host cache running on such a buffer."""
import numpy as np
import torch

from lightllm_b200.utils import host_memory as hm


def test_parsers(tmp_path):
    assert hm.parse_node_list("0-1,4\n") == [0, 1, 4] and hm.parse_node_list("") == [] and hm.parse_node_list("3") == [3]
    (tmp_path / "meminfo").write_text("MemTotal: 1 kB\nHugepagesize:    1048576 kB\n")
    assert hm.default_huge_page_size(str(tmp_path / "meminfo")) == 1 << 30
    assert hm.default_huge_page_size(str(tmp_path / "absent")) == 2 << 20
    node_dir = tmp_path / "node"
    node_dir.mkdir()
    (node_dir / "online").write_text("0-3\n")
    assert hm.nodes_with_memory(str(node_dir)) == [0, 1, 2, 3]
    (node_dir / "has_memory").write_text("0,2\n")
    assert hm.nodes_with_memory(str(node_dir)) == [0, 2]
    pci = tmp_path / "pci" / "0000:1b:00.0"
    pci.mkdir(parents=True)
    (pci / "numa_node").write_text("1\n")
    assert hm.numa_node_of_pci("0000:1B:00.0", str(tmp_path / "pci")) == 1
    assert hm.numa_node_of_pci("00000000:1B:00.0", str(tmp_path / "pci")) == 1     # the 8-digit domain spelling
    (pci / "numa_node").write_text("-1\n")
    assert hm.numa_node_of_pci("0000:1b:00.0", str(tmp_path / "pci")) is None
    assert hm.numa_node_of_pci("0000:ff:00.0", str(tmp_path / "pci")) is None


def test_env_switches(monkeypatch):
    for k in ("LLB_HUGE_PAGE_ENABLE", "LIGHTLLM_HUGE_PAGE_ENABLE", "LLB_ENABLE_NUMA_INTERLEAVE",
              "LIGHTLLM_ENABLE_NUMA_INTERLEAVE", "LLB_CPU_CACHE_NUMA"):
        monkeypatch.delenv(k, raising=False)
    assert not hm.huge_pages_wanted() and hm.numa_policy_wanted() is None
    monkeypatch.setenv("LIGHTLLM_HUGE_PAGE_ENABLE", "1")
    monkeypatch.setenv("LIGHTLLM_ENABLE_NUMA_INTERLEAVE", "true")
    assert hm.huge_pages_wanted() and hm.numa_policy_wanted() == "interleave"
    monkeypatch.setenv("LLB_CPU_CACHE_NUMA", "local")
    assert hm.numa_policy_wanted() == "local"


def test_buffer_with_every_option_is_usable_whatever_the_machine_allows():
    nbytes = 3 * (1 << 20) + 123
    buf = hm.HostBuffer.create(nbytes, huge_pages=True, numa="interleave", device_index=None, register=True,
                               prefault_threads=4)
    assert buf.mapped >= nbytes and buf.addr % 4096 == 0
    # explicit huge pages or a note that says why not; no CUDA here, so no registration either way
    assert buf.huge_pages or any("huge pages" in n for n in buf.notes)
    assert buf.registered == torch.cuda.is_available() or any("register" in n.lower() for n in buf.notes)
    assert buf.numa is not None or any("interleave" in n or "mbind" in n for n in buf.notes)
    t = buf.tensor(torch.bfloat16, (3, 512, 1024))
    assert t.shape == (3, 512, 1024) and t.data_ptr() == buf.addr and float(t.float().abs().sum()) == 0.0
    t[1, 7].fill_(2.5)
    again = buf.tensor(torch.bfloat16, (3, 512, 1024))
    assert float(again[1, 7, 5]) == 2.5 and np.frombuffer(buf.mm, dtype=np.uint8).any()
    try:
        buf.tensor(torch.float32, (1 << 20,))
        raise AssertionError("a view past the end was accepted")
    except AssertionError as e:
        assert "larger" in str(e)
    local = hm.HostBuffer.create(1 << 16, numa="local", device_index=None)
    assert local.numa is None and any("unknown" in n for n in local.notes)
    buf.close()


def test_mbind_reports_errno_instead_of_raising():
    buf = hm.HostBuffer.create(1 << 16)
    assert hm._mbind(buf.addr, buf.mapped, hm.MPOL_INTERLEAVE, []) == 38
    r = hm._mbind(buf.addr, buf.mapped, hm.MPOL_PREFERRED, [0])
    assert isinstance(r, int) and r >= 0        # 0 where the kernel allows it, an errno in a sandbox


def test_host_cache_on_an_own_mapping(monkeypatch, tmp_path):
    """The same offload / reload round trip as with torch's allocation, on a buffer made by this module."""
    from test_host_kv_cache import test_host_tier_serves_prefix_after_gpu_eviction as round_trip

    monkeypatch.setenv("LLB_HUGE_PAGE_ENABLE", "1")
    monkeypatch.setenv("LLB_CPU_CACHE_NUMA", "interleave")
    made = []
    real = hm.HostBuffer.create.__func__
    monkeypatch.setattr(hm.HostBuffer, "create", classmethod(lambda cls, *a, **kw: made.append(real(cls, *a, **kw)) or made[-1]))
    round_trip(tmp_path)
    assert made and made[0].mapped > 0
