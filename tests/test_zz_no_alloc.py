"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some hosts of these kernels may not call cudaMalloc (they run inside someone else's memory budget
or inside a loop that must stay off the allocator).  For them the library exports
`llb_gqa_decode_no_alloc`, whose split-KV scratch is a fixed array inside the library.  This test
checks it against the regular entry point (scratch supplied by the caller) on two calls in a row
that leave different contents in the shared scratch, and checks that an oversized request is
refused.  The file sorts last so that a `-x` run has executed every other test before it.
"""
import ctypes
import math

import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.ops._native import kernels

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _case(dev, lens, Hq, Hkv, D, seed):
    g = torch.Generator().manual_seed(seed)
    total = sum(lens)
    kv = (torch.randn(total + 9, 2 * Hkv, D, generator=g) * 0.5).to(dev, BF)
    perm = torch.randperm(total + 8, generator=g)[:total].to(torch.int32)
    r2t = torch.zeros(len(lens) + 1, max(lens) + 2, dtype=torch.int32)
    off = 0
    for i, L in enumerate(lens):
        r2t[i, :L] = perm[off:off + L]
        off += L
    q = (torch.randn(len(lens), Hq * D, generator=g)).to(dev, BF)
    return q, kv, r2t.to(dev), torch.arange(len(lens), dtype=torch.int32, device=dev), \
        torch.tensor(lens, dtype=torch.int32, device=dev)


def _call_no_alloc(q, kv, r2t, b_req, b_len, Hq, Hkv, D, splits):
    lib = kernels()
    fn = lib.llb_gqa_decode_no_alloc
    fn.restype = ctypes.c_int
    B = q.shape[0]
    out = torch.empty(B, Hq, D, dtype=q.dtype, device=q.device)
    vp = ctypes.c_void_p
    rc = fn(vp(q.data_ptr()), ctypes.c_int64(q.stride(0)), vp(kv.data_ptr()), vp(r2t.data_ptr()),
            ctypes.c_int64(r2t.stride(0)), vp(b_req.data_ptr()), vp(b_len.data_ptr()), vp(out.data_ptr()),
            ctypes.c_int64(out.stride(0)), ctypes.c_int(B), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_int(D),
            ctypes.c_int(splits), ctypes.c_float(1.0 / math.sqrt(D)), vp(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_no_alloc_matches_regular_entry_point_twice(dev):
    Hq, Hkv, D = 32, 8, 128
    # first call: long sequences, 6 splits; second call: different lengths and 3 splits, so stale
    # partials of the first call sit in the part of the scratch the second call does not rewrite
    for lens, splits, seed in (([700, 33, 1500, 257], 6, 0), ([90, 410, 17], 3, 1)):
        q, kv, r2t, b_req, b_len = _case(dev, lens, Hq, Hkv, D, seed)
        want = ops.gqa_decode(q, kv, r2t, b_req, b_len, Hq, Hkv, D, max(lens), num_splits=splits)
        rc, got = _call_no_alloc(q, kv, r2t, b_req, b_len, Hq, Hkv, D, splits)
        assert rc == 0
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        assert err < 2e-2, f"max abs err {err}"


def test_no_alloc_rejects_oversized_request(dev):
    Hq, Hkv, D = 32, 8, 128
    lens = [64] * 40  # 40 * 32 * 8 = 10240 rows > 8192
    q, kv, r2t, b_req, b_len = _case(dev, lens, Hq, Hkv, D, 2)
    rc, _ = _call_no_alloc(q, kv, r2t, b_req, b_len, Hq, Hkv, D, 8)
    assert rc == -3


def test_no_alloc_head_size_64_and_single_split(dev):
    """Head size 64 goes through the same scratch; one split needs none, so even a batch with more rows than
    the scratch holds is served."""
    Hq, Hkv, D = 16, 4, 64
    for lens, splits, seed in (([300, 41, 1200], 4, 3), ([50] * 600, 1, 4)):   # 600 * 16 = 9600 rows, one split
        q, kv, r2t, b_req, b_len = _case(dev, lens, Hq, Hkv, D, seed)
        want = ops.gqa_decode(q, kv, r2t, b_req, b_len, Hq, Hkv, D, max(lens), num_splits=splits)
        rc, got = _call_no_alloc(q, kv, r2t, b_req, b_len, Hq, Hkv, D, splits)
        assert rc == 0
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        assert err < 2e-2, f"max abs err {err}"
