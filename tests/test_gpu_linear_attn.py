"""Gated DeltaNet decode-step kernels (convolution step, recurrent state update + read-out) against the fp32 torch
restatement of the same step (`ops/linear_attn.py`: causal_conv_step, gated_delta_step)."""
import pytest
import torch

from lightllm_b200.ops import linear_attn as la

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,nk,nv,dk,dv", [(5, 2, 4, 128, 128), (33, 4, 4, 64, 64), (3, 1, 2, 32, 96),
                                           (130, 2, 8, 128, 128), (2, 2, 2, 192, 32)])
@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
def test_decode_step_matches_torch(dev, B, nk, nv, dk, dv, state_dtype):
    assert la.step_kernel_supported(dk, dv, 4)
    g_ = torch.Generator().manual_seed(B * 7 + dk)
    C, K, slots = 2 * nk * dk + nv * dv, 4, B + 9
    mixed = torch.randn(B, C, generator=g_)
    conv_state = torch.randn(slots, C, K - 1, generator=g_).to(torch.bfloat16)
    conv_w = torch.randn(C, K, generator=g_) * 0.5
    ssm = (torch.randn(slots, nv, dk, dv, generator=g_) * 0.3).to(state_dtype)
    req = torch.randperm(slots, generator=g_)[:B].to(torch.int32)
    gate = -torch.rand(B, nv, generator=g_)
    beta = torch.rand(B, nv, generator=g_)
    # torch restatement on the CPU copies
    rl = req.long()
    y, new_conv = la.causal_conv_step(mixed, conv_state[rl], conv_w)
    kd = nk * dk
    rep = nv // nk
    qq = y[:, :kd].view(B, nk, dk).repeat_interleave(rep, dim=1)
    kk = y[:, kd:2 * kd].view(B, nk, dk).repeat_interleave(rep, dim=1)
    vv = y[:, 2 * kd:].view(B, nv, dv)
    want, new_s = la.gated_delta_step(qq, kk, vv, gate, beta, ssm[rl].float())
    want_conv = conv_state.clone()
    want_conv[rl] = new_conv.to(torch.bfloat16)
    want_ssm = ssm.clone()
    want_ssm[rl] = new_s.to(state_dtype)
    # kernels
    cs, ss = conv_state.to(dev), ssm.to(dev)
    got = la.conv_and_delta_step(mixed.to(dev), cs, conv_w.to(dev), ss, req.to(dev), gate.to(dev), beta.to(dev),
                                 nk, nv, dk, dv)
    torch.cuda.synchronize()
    scale = want.abs().max().item()
    assert (got.cpu() - want).abs().max().item() < 2e-3 * scale + 1e-4
    assert torch.equal(cs.cpu(), want_conv)                       # the shifted inputs are exact copies
    tol = 1e-4 if state_dtype == torch.float32 else 2e-2
    ref_scale = want_ssm.float().abs().max().item()
    assert (ss.cpu().float() - want_ssm.float()).abs().max().item() < tol * ref_scale + 1e-5
    untouched = torch.ones(slots, dtype=torch.bool)
    untouched[rl] = False
    assert torch.equal(ss.cpu()[untouched], ssm[untouched])       # other requests' states are not written
