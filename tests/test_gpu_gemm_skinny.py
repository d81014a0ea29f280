"""Decode GEMM (M <= 256): CTA-pair tiles, K split across a cluster with a distributed-shared-memory reduction."""
import pytest
import torch

from lightllm_b200 import ops
from lightllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _check(got, want):
    err = (got.float() - want.float()).abs().max().item()
    tol = 1e-2 * want.abs().max().item() + 1e-2
    assert err < tol, f"max abs err {err} (tol {tol})"
    assert int(ops.gemm_status(got.device).item()) == 0, "a bounded wait inside the GEMM timed out"


# bn = 1000 + 10 * accumulators + splits (+ 100: half-width tiles, 128 columns per cluster)
@pytest.mark.parametrize("M", [1, 7, 100, 128, 129, 256])
@pytest.mark.parametrize("N,K", [(1024, 1024), (4096, 4096), (6144, 4096), (4096, 14336), (1032, 4160)])
@pytest.mark.parametrize("bn", [1011, 1012, 1014, 1021, 1111, 1112, 1114])
def test_skinny_store(dev, M, N, K, bn):
    torch.manual_seed(M + N)
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    _check(ops.gemm(a, w, bn=bn), a.float() @ w.float().t())


@pytest.mark.parametrize("bn", [1011, 1012, 1014, 1021, 1111, 1112, 0])
def test_skinny_epilogues(dev, bn):
    torch.manual_seed(3)
    M, N, K = 200, 2048, 2048
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    bias = torch.randn(N, device=dev).to(BF)
    res = torch.randn(M, N, device=dev).to(BF)
    acc = a.float() @ w.float().t()
    _check(ops.gemm(a, w, bias=bias, bn=bn), acc + bias.float())
    _check(ops.gemm(a, w, epi="residual", residual=res, bn=bn), acc + res.float())
    r2 = res.clone()
    ops.gemm(a, w, epi="residual", residual=r2, out=r2, bn=bn)
    _check(r2, acc + res.float())
    f = ops.gemm(a, w, epi="f32", bias=bias, bn=bn)
    assert f.dtype == torch.float32 and (f - acc - bias.float()).abs().max().item() < 2e-2
    if bn in (1011, 1021, 0):
        g = (torch.randn(N // 2, K, device=dev) * 0.1).to(BF)
        u = (torch.randn(N // 2, K, device=dev) * 0.1).to(BF)
        want = torch.nn.functional.silu(a.float() @ g.float().t()) * (a.float() @ u.float().t())
        _check(ops.gemm(a, ref.interleave_gate_up(g, u), epi="gated_silu", bn=bn), want)


def test_skinny_auto_llama_shapes(dev):
    torch.manual_seed(4)
    for M in (256, 64):
        for N, K in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)):
            a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
            w = (torch.randn(N, K, device=dev) * 0.05).to(BF)
            _check(ops.gemm(a, w), a.float() @ w.float().t())


@pytest.mark.parametrize("bn", [1011, 1012, 1014, 1021])
@pytest.mark.parametrize("M,N,K", [(256, 4096, 4096), (33, 1024, 14336), (200, 6144, 1024)])
def test_skinny_tiled_weight(dev, bn, M, N, K):
    torch.manual_seed(5)
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    tw = ops.TiledWeight(w)
    assert torch.equal(tw.dense(), w)
    _check(ops.gemm(a, tw, bn=bn), a.float() @ w.float().t())


@pytest.mark.parametrize("bn", [1011, 1021, 1012])
def test_cluster_kernel_many_m_tiles(dev, bn):
    torch.manual_seed(6)
    M, N, K = 1100, 1536, 2048
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    res = torch.randn(M, N, device=dev).to(BF)
    _check(ops.gemm(a, w, bn=bn), a.float() @ w.float().t())
    _check(ops.gemm(a, w, epi="residual", residual=res, bn=bn), a.float() @ w.float().t() + res.float())


def _table_cases():
    import json
    import os

    from lightllm_b200.utils.autotuner import PKG_DIR

    path = os.path.join(str(PKG_DIR), "NVIDIA_B200", "gemm_bf16.json")
    if not os.path.exists(path):
        return []
    table = json.load(open(path))
    cases = []
    for key, runs in sorted(table.items()):
        parts = dict(p.split("=") for p in key.split(","))
        N, K, epi = int(parts["N"]), int(parts["K"]), parts["epi"]
        for bn in sorted({int(c["bn"]) for c in runs.values()} - {0}):
            cases.append((N, K, epi, bn))
    return cases


@pytest.mark.parametrize("N,K,epi,bn", _table_cases())
def test_every_variant_of_the_shipped_table_is_numerically_right(dev, N, K, epi, bn):
    """The tuned-config table only records speed: every (shape, variant) pair it can select is checked against the
    fp32 product here, at a row count between the tuned ones as well."""
    import torch

    from lightllm_b200 import ops
    from lightllm_b200.ops import reference as ref

    if N * K > 200_000_000:          # the vocabulary projection: a slice of its columns is enough
        N = 8 * 1024 + (N % 1024)
    g = torch.Generator(device="cpu").manual_seed(N + K)
    w = (torch.randn(N, K, generator=g) * 0.05).to(dev, torch.bfloat16)
    for M in (8, 200):
        a = (torch.randn(M, K, generator=g) * 0.5).to(dev, torch.bfloat16)
        res = (torch.randn(M, N, generator=g) * 0.5).to(dev, torch.bfloat16) if epi == "residual" else None
        got = ops.gemm(a, w, epi=epi, residual=res, bn=bn).float()
        want = ref.gemm(a, w, epi, res, None).float()
        scale = max(want.abs().max().item(), 1.0)
        assert (got - want).abs().max().item() < 0.02 * scale, f"M={M} bn={bn}"


# ---- split-K kernel without clusters: bn = 2000 + splits (2000: as many splits as fit the GPU) ----
@pytest.mark.parametrize("M", [1, 100, 128, 129, 256])
@pytest.mark.parametrize("N,K", [(768, 4096), (4096, 512), (3584, 4096), (4096, 1792), (4096, 4096), (1032, 4160),
                                 (6144, 4096), (4096, 14336), (16032, 4096)])
@pytest.mark.parametrize("bn", [2000, 2001, 2002, 2004, 2008])
def test_splitk_store(dev, M, N, K, bn):
    torch.manual_seed(M + N + bn)
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    tiles, units = (N + 127) // 128, (2 if M > 128 else 1) * 4
    s = bn - 2000
    fits = s == 0 or (s <= units and tiles * s <= 148 and -(-((K + 63) // 64) // s) * (s - 1) < (K + 63) // 64)
    if not fits or tiles > 148:
        with pytest.raises(Exception):
            ops.gemm(a, w, bn=bn)
        return
    for _ in range(2):   # the second call finds the first call's values in the workspace and counters
        _check(ops.gemm(a, w, bn=bn), a.float() @ w.float().t())


@pytest.mark.parametrize("bn", [2000, 2001, 2002, 2004])
@pytest.mark.parametrize("M", [200, 64])
def test_splitk_epilogues(dev, bn, M):
    torch.manual_seed(3)
    N, K = 2048, 2048
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    bias = torch.randn(N, device=dev).to(BF)
    res = torch.randn(M, N, device=dev).to(BF)
    acc = a.float() @ w.float().t()
    _check(ops.gemm(a, w, bias=bias, bn=bn), acc + bias.float())
    _check(ops.gemm(a, w, epi="residual", residual=res, bn=bn), acc + res.float())
    r2 = res.clone()
    ops.gemm(a, w, epi="residual", residual=r2, out=r2, bn=bn)
    _check(r2, acc + res.float())
    f = ops.gemm(a, w, epi="f32", bias=bias, bn=bn)
    assert f.dtype == torch.float32 and (f - acc - bias.float()).abs().max().item() < 2e-2
    if bn != 2004 or M > 128:      # gated tiles have half as many units: 4 splits need two row blocks
        g = (torch.randn(N // 2, K, device=dev) * 0.1).to(BF)
        u = (torch.randn(N // 2, K, device=dev) * 0.1).to(BF)
        want = torch.nn.functional.silu(a.float() @ g.float().t()) * (a.float() @ u.float().t())
        _check(ops.gemm(a, ref.interleave_gate_up(g, u), epi="gated_silu", bn=bn), want)
        want = torch.nn.functional.gelu(a.float() @ g.float().t(), approximate="tanh") * (a.float() @ u.float().t())
        _check(ops.gemm(a, ref.interleave_gate_up(g, u), epi="gated_gelu", bn=bn), want)


def test_splitk_alternating_split_counts_share_the_workspace(dev):
    """Launches with different split counts follow each other on one stream (as the layers of a decode step do)."""
    torch.manual_seed(9)
    a = (torch.randn(256, 4096, device=dev) * 0.5).to(BF)
    ws = [(torch.randn(n, 4096, device=dev) * 0.1).to(BF) for n in (768, 4096, 1024)]
    want = [a.float() @ w.float().t() for w in ws]
    for _ in range(3):
        outs = [ops.gemm(a, w, bn=bn) for w, bn in zip(ws, (2008, 2004, 2002))]
        for o, t in zip(outs, want):
            _check(o, t)


# ---- the same split on CTA-pair tiles: bn = 3000 + splits (3000: as many splits as fit) ----
def _pair_fits(M, N, K, s, gated=False):
    pairs, kb = -(-M // 256) * -(-N // 256), (K + 63) // 64
    if pairs * 2 > 148:
        return False
    return s == 0 or (s <= (4 if gated else 8) and pairs * 2 * s <= 148 and -(-kb // s) * (s - 1) < kb)


@pytest.mark.parametrize("M", [1, 100, 129, 256, 300, 512])
@pytest.mark.parametrize("N,K", [(768, 4096), (4096, 512), (3584, 4096), (4096, 1792), (4096, 4096), (1032, 4160),
                                 (6144, 4096), (4096, 14336), (16032, 4096)])
@pytest.mark.parametrize("bn", [3000, 3001, 3002, 3004, 3008])
def test_pairsplit_store(dev, M, N, K, bn):
    torch.manual_seed(M + N + bn)
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    if not _pair_fits(M, N, K, bn - 3000):
        with pytest.raises(Exception):
            ops.gemm(a, w, bn=bn)
        return
    for _ in range(2):
        _check(ops.gemm(a, w, bn=bn), a.float() @ w.float().t())


@pytest.mark.parametrize("bn", [3000, 3001, 3002, 3004, 3008])
@pytest.mark.parametrize("M", [200, 64])
def test_pairsplit_epilogues(dev, bn, M):
    torch.manual_seed(3)
    N, K = 2048, 2048
    a = (torch.randn(M, K, device=dev) * 0.5).to(BF)
    w = (torch.randn(N, K, device=dev) * 0.1).to(BF)
    bias = torch.randn(N, device=dev).to(BF)
    res = torch.randn(M, N, device=dev).to(BF)
    acc = a.float() @ w.float().t()
    _check(ops.gemm(a, w, bias=bias, bn=bn), acc + bias.float())
    _check(ops.gemm(a, w, epi="residual", residual=res, bn=bn), acc + res.float())
    r2 = res.clone()
    ops.gemm(a, w, epi="residual", residual=r2, out=r2, bn=bn)
    _check(r2, acc + res.float())
    f = ops.gemm(a, w, epi="f32", bias=bias, bn=bn)
    assert f.dtype == torch.float32 and (f - acc - bias.float()).abs().max().item() < 2e-2
    if bn != 3008:
        g = (torch.randn(N // 2, K, device=dev) * 0.1).to(BF)
        u = (torch.randn(N // 2, K, device=dev) * 0.1).to(BF)
        want = torch.nn.functional.silu(a.float() @ g.float().t()) * (a.float() @ u.float().t())
        _check(ops.gemm(a, ref.interleave_gate_up(g, u), epi="gated_silu", bn=bn), want)


def test_split_kernels_alternate_on_one_stream(dev):
    torch.manual_seed(10)
    a = (torch.randn(256, 4096, device=dev) * 0.5).to(BF)
    ws = [(torch.randn(n, 4096, device=dev) * 0.1).to(BF) for n in (768, 4096, 1024, 6144)]
    want = [a.float() @ w.float().t() for w in ws]
    for _ in range(3):
        outs = [ops.gemm(a, w, bn=bn) for w, bn in zip(ws, (3008, 2004, 3004, 3002))]
        for o, t in zip(outs, want):
            _check(o, t)
