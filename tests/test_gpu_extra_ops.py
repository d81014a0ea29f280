"""LayerNorm, plain activations and the generic paged attention kernel against fp32 PyTorch references."""
import math

import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("T,H", [(1, 64), (37, 2560), (300, 6144)])
@pytest.mark.parametrize("with_res,with_bias", [(False, True), (True, True), (True, False)])
def test_layernorm(T, H, with_res, with_bias):
    dev = "cuda"
    x = torch.randn(T, H, device=dev).to(BF)
    w = (torch.randn(H, device=dev) * 0.1 + 1).to(BF)
    b = (torch.randn(H, device=dev) * 0.1).to(BF) if with_bias else None
    res = torch.randn(T, H, device=dev).to(BF) if with_res else None
    res_ref = res.clone() if with_res else None
    got = ops.layernorm(x, w, b, 1e-5, residual=res)
    want = ref.layernorm(x.cpu(), w.cpu(), None if b is None else b.cpu(), 1e-5,
                         residual=None if res_ref is None else res_ref.cpu())
    assert (got.float().cpu() - want.float()).abs().max().item() < 4e-2
    if with_res:
        assert torch.equal(res.cpu(), (res_ref.float().cpu() + x.float().cpu()).to(BF))


@pytest.mark.parametrize("kind", ["silu", "gelu", "gelu_tanh", "relu", "scale"])
def test_act(kind):
    x = torch.randn(1000, 333, device="cuda").to(BF)
    want = ref.act_(x.clone().cpu(), kind, 0.37)
    got = ops.act_(x.clone(), kind, 0.37)
    assert (got.float().cpu() - want.float()).abs().max().item() < 2e-2


def _setup(B, lens, Hkv, D, dev):
    total = sum(lens)
    slots_n = total + 64
    kv = (torch.randn(slots_n, 2 * Hkv, D, device=dev) * 0.5).to(BF)
    r2t = torch.zeros(B + 2, max(lens) + 8, dtype=torch.int32, device=dev)
    perm = torch.randperm(slots_n, device=dev)[:total].to(torch.int32)
    off = 0
    for b, L in enumerate(lens):
        r2t[b + 1, :L] = perm[off:off + L]
        off += L
    b_req = torch.arange(1, B + 1, dtype=torch.int32, device=dev)
    return kv, r2t, b_req


@pytest.mark.parametrize("D,Hq,Hkv", [(256, 8, 1), (96, 12, 12), (80, 8, 8), (128, 8, 2), (64, 16, 4)])
@pytest.mark.parametrize("feature", ["plain", "window", "alibi", "softcap", "sinks"])
def test_generic_attention_decode_and_prefill(D, Hq, Hkv, feature):
    dev = "cuda"
    torch.manual_seed(D + Hq)
    lens = [5, 130, 77]
    B = len(lens)
    kv, r2t, b_req = _setup(B, lens, Hkv, D, dev)
    kw = {}
    if feature == "window":
        kw["window"] = 32
    elif feature == "alibi":
        kw["alibi"] = torch.tensor([2.0 ** (-(i + 1) * 8.0 / Hq) for i in range(Hq)], device=dev)
    elif feature == "softcap":
        kw["softcap"] = 30.0
    elif feature == "sinks":
        kw["sinks"] = torch.randn(Hq, device=dev)
    scale = 1.0 / math.sqrt(D)
    # decode: one query per request at its last position
    q = (torch.randn(B, Hq, D, device=dev)).to(BF)
    pos = torch.tensor([L - 1 for L in lens], dtype=torch.int32, device=dev)
    got = ops.attention_generic(q, kv, r2t, b_req, pos, None, Hq, Hkv, D, scale, **kw)
    cpu_kw = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in kw.items()}
    want = ref.attention_generic(q.cpu(), kv.cpu(), r2t.cpu(), b_req.cpu(), pos.cpu(), None, Hq, Hkv, D, scale, **cpu_kw)
    assert (got.float().cpu() - want.float()).abs().max().item() < 3e-2
    # prefill: the last 20 tokens of every request are new
    new = 20
    qs, ps, bs = [], [], []
    for b, L in enumerate(lens):
        n = min(new, L)
        qs.append(torch.randn(n, Hq, D, device=dev).to(BF))
        ps.append(torch.arange(L - n, L, dtype=torch.int32, device=dev))
        bs.append(torch.full((n,), b, dtype=torch.int32, device=dev))
    q, pos, batch_of = torch.cat(qs), torch.cat(ps), torch.cat(bs)
    got = ops.attention_generic(q, kv, r2t, b_req, pos, batch_of, Hq, Hkv, D, scale, **kw)
    want = ref.attention_generic(q.cpu(), kv.cpu(), r2t.cpu(), b_req.cpu(), pos.cpu(), batch_of.cpu(), Hq, Hkv, D, scale,
                                 **cpu_kw)
    assert (got.float().cpu() - want.float()).abs().max().item() < 3e-2
