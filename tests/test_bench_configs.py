"""bench.py dry runs on CPU: every configuration's harness with toy shapes (the driver's contract: one JSON line
with the named keys; arrivals, data-parallel + expert-parallel waves and the fp8 model go through the public API)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra, nproc=1, port=29571):
    env = dict(os.environ, LLB_FORCE_CPU="1", PYTHONPATH=ROOT)
    cmd = [sys.executable]
    if nproc > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
                "--master-port", str(port)]
    cmd += ["bench.py", "--gpus", str(nproc), "--steps", "1", "--warmup", "1"] + extra
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, r.stdout[-1000:]
    return json.loads(lines[0])


def _check_contract(d, n_gpus):
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches"):
        assert k in d, k
    assert d["n_gpus"] == n_gpus and d["value"] > 0 and d["higher_is_better"] is True
    assert {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"} <= set(d["e2e"])
    assert d["e2e"]["h2d_bytes_per_step"] > 0 and d["e2e"]["d2h_bytes_per_step"] > 0


@pytest.mark.timeout(900)
def test_default_configuration_line():
    d = _run(["--model", "tiny", "--conc", "4", "--in-len", "16", "--out-len", "4", "--batch-max-tokens", "64"])
    _check_contract(d, 1)
    assert d["config"]["parallelism"] == "tp1" and d["config"]["global_batch"] == 4


@pytest.mark.timeout(900)
def test_poisson_arrivals_configuration():
    d = _run(["--config", "3", "--model", "tiny", "--requests", "10", "--rate", "50", "--in-range", "8,40",
              "--out-range", "4,10", "--conc", "8", "--batch-max-tokens", "128"])
    _check_contract(d, 1)
    assert d["config"]["requests"] == 10 and "Poisson" in d["config"]["arrivals"]
    assert d["e2e"]["p50_ttft_ms"] > 0


@pytest.mark.timeout(900)
@pytest.mark.parametrize("config,model", [(4, "tiny-moe"), (5, "tiny-ds")])
def test_expert_parallel_configurations_two_ranks(config, model):
    d = _run(["--config", str(config), "--model", model, "--conc", "8", "--in-len", "24", "--out-len", "6",
              "--batch-max-tokens", "128"], nproc=2, port=29573 + config)
    _check_contract(d, 2)
    assert d["config"]["parallelism"] == "dp2+ep2"
    # 8 requests (4 per replica) x 6 tokens in one timed wave
    assert abs(d["value"] * d["ms_per_step"] / 1e3 - 48) < 1
