"""Paged GQA attention kernels against the fp32 reference (gather by slot table, softmax in fp32)."""
import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _pool(dev, n_req, lens, Hkv, D, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    total = sum(lens)
    size = total + 17
    kv = (torch.randn(size + 1, 2 * Hkv, D, generator=g) * 0.5).to(dev, BF)
    perm = torch.randperm(size, generator=g)[:total].to(torch.int32)
    max_len = max(lens) + 3
    r2t = torch.zeros(n_req + 1, max_len, dtype=torch.int32)
    off = 0
    rows = torch.randperm(n_req, generator=g)[: len(lens)]
    for i, L in enumerate(lens):
        r2t[rows[i], :L] = perm[off:off + L]
        off += L
    return kv, r2t.to(dev), rows.to(torch.int32).to(dev)


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (4, 1, 128), (8, 8, 128), (16, 1, 128), (64, 2, 128), (8, 2, 64)])
@pytest.mark.parametrize("splits", [1, 3])
def test_decode(dev, Hq, Hkv, D, splits):
    lens = [1, 15, 16, 17, 130, 500, 64, 257]
    kv, r2t, rows = _pool(dev, 12, lens, Hkv, D, 0)
    B = len(lens)
    torch.manual_seed(1)
    qfull = torch.randn(B, (Hq + 2 * Hkv) * D, device=dev, dtype=BF)  # q lives inside a wider qkv row
    q = qfull[:, : Hq * D]
    b_len = torch.tensor(lens, dtype=torch.int32, device=dev)
    got = ops.gqa_decode(q, kv, r2t, rows, b_len, Hq, Hkv, D, max(lens), num_splits=splits)
    want = ref.gqa_decode(q.reshape(B, Hq, D), kv, r2t, rows, b_len, Hq, Hkv, D)
    err = (got.float() - want.float()).abs().max().item()
    assert err < 2e-2, f"max abs err {err}"


def test_decode_auto_split_long(dev):
    Hq, Hkv, D = 32, 8, 128
    lens = [5000, 33]
    kv, r2t, rows = _pool(dev, 4, lens, Hkv, D, 2)
    q = torch.randn(2, Hq * D, device=dev, dtype=BF)
    b_len = torch.tensor(lens, dtype=torch.int32, device=dev)
    assert ops.gqa_decode_num_splits(2, Hq, Hkv, 5000) > 1
    got = ops.gqa_decode(q, kv, r2t, rows, b_len, Hq, Hkv, D, 5000)
    want = ref.gqa_decode(q.reshape(2, Hq, D), kv, r2t, rows, b_len, Hq, Hkv, D)
    assert (got.float() - want.float()).abs().max().item() < 2e-2


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (4, 4, 128), (8, 2, 64)])
def test_prefill(dev, Hq, Hkv, D):
    # (cached prefix, new tokens) per request: fresh prompts, chunked continuation, single-token tail
    ready = [0, 37, 128, 0, 200]
    new = [70, 64, 1, 129, 65]
    lens = [r + n for r, n in zip(ready, new)]
    kv, r2t, rows = _pool(dev, 9, lens, Hkv, D, 3)
    T = sum(new)
    torch.manual_seed(4)
    qfull = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev, dtype=BF)
    q = qfull[:, : Hq * D]
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=dev)
    rdy = torch.tensor(ready, dtype=torch.int32, device=dev)
    got = ops.gqa_prefill(q, kv, r2t, rows, cu, rdy, Hq, Hkv, D, max(new))
    want = ref.gqa_prefill(q.reshape(T, Hq, D), kv, r2t, rows, cu, rdy, Hq, Hkv, D)
    err = (got.float() - want.float()).abs().max().item()
    assert err < 2e-2, f"max abs err {err}"


@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (4, 1)])
def test_prefill_many_kv_tiles(dev, Hq, Hkv):
    """Head size 128 on the tcgen05 kernel: several 128-key tiles per query tile (both K/V stages and both score
    buffers wrap around), a long cached prefix, tile-unaligned lengths."""
    from lightllm_b200.ops._native import kernels

    D = 128
    ready = [0, 300, 1000, 5]
    new = [1024, 500, 130, 260]
    lens = [r + n for r, n in zip(ready, new)]
    kv, r2t, rows = _pool(dev, 6, lens, Hkv, D, 7)
    T = sum(new)
    torch.manual_seed(8)
    q = torch.randn(T, Hq * D, device=dev, dtype=BF)
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device=dev)
    rdy = torch.tensor(ready, dtype=torch.int32, device=dev)
    got = ops.gqa_prefill(q, kv, r2t, rows, cu, rdy, Hq, Hkv, D, max(new))
    want = ref.gqa_prefill(q.reshape(T, Hq, D), kv, r2t, rows, cu, rdy, Hq, Hkv, D)
    torch.cuda.synchronize()
    assert int(kernels().llb_attn_tc_status()) == 0, "a bounded wait inside the attention kernel ran out"
    err = (got.float() - want.float()).abs().max().item()
    assert err < 2e-2, f"max abs err {err}"
