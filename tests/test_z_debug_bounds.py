"""The checked kernel build (`LLB_DEBUG_BOUNDS=1`): an index beyond a table's DECLARED size is reported through the
status word and the access is redirected to entry 0.  Every case keeps the bad index inside the real allocation
(the tables are allocated larger than the size handed to the kernels), so that even a missing check could not
touch memory the test does not own.  The checked library is loaded in a child process (the parent has the regular
one).  compute-sanitizer's place in the reference's test strategy is taken by this build."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import math, torch
from lightllm_b200 import ops
from lightllm_b200.ops import moe as moe_ops
from lightllm_b200.ops._native import set_debug_bounds, debug_bounds_enabled
assert debug_bounds_enabled()
dev = torch.device("cuda", 0)
BF = torch.bfloat16
status = torch.zeros(1, dtype=torch.int32, device=dev)
# declared: 128 pool slots, 8 request rows, 32 positions, 64 experts; allocated: 256 slots, 12 rows, 64 positions
assert set_debug_bounds(pool_slots=128, req_rows=8, r2t_cols=32, num_experts=64, status=status)
r2t = torch.zeros(12, 64, dtype=torch.int32, device=dev)
nxt = torch.arange(12, dtype=torch.int64, device=dev)

def code():
    torch.cuda.synchronize()
    c = int(status.item()); status.zero_(); return c

def prologue(req, L, slot):
    return ops.decode_prologue(r2t, nxt, torch.tensor([req], dtype=torch.int32, device=dev),
                               torch.tensor([L], dtype=torch.int32, device=dev), torch.tensor([slot], dtype=torch.int32, device=dev))

prologue(3, 5, 17); assert code() == 0 and int(r2t[3, 4]) == 17                 # in range: untouched
prologue(9, 5, 18); assert code() == 902 and int(r2t[9, 4]) == 0 and int(r2t[0, 4]) == 18   # row 9 > declared 8 -> row 0
prologue(2, 40, 19); assert code() == 903 and int(r2t[2, 39]) == 0              # position 39 > declared 32 -> column 0
prologue(2, 6, 200); assert code() == 901 and int(r2t[2, 5]) == 0               # slot 200 > declared 128 -> slot 0

# decode attention over a request whose table holds a slot beyond the declared pool (still inside the real pool)
Hq, Hkv, D, L = 8, 2, 128, 20
kv = (torch.randn(256, 2 * Hkv, D, device=dev) * 0.5).to(BF)
r2t.zero_(); r2t[1, :L] = torch.arange(10, 10 + L, dtype=torch.int32, device=dev)
q = torch.randn(1, Hq * D, device=dev).to(BF)
b_req = torch.tensor([1], dtype=torch.int32, device=dev); b_len = torch.tensor([L], dtype=torch.int32, device=dev)
good = ops.gqa_decode(q, kv, r2t, b_req, b_len, Hq, Hkv, D, L, num_splits=1)
assert code() == 0
r2t[1, 7] = 200
bad = ops.gqa_decode(q, kv, r2t, b_req, b_len, Hq, Hkv, D, L, num_splits=1)
assert code() == 901
r2t[1, 7] = 0                                                                       # what the checked kernel read instead
same = ops.gqa_decode(q, kv, r2t, b_req, b_len, Hq, Hkv, D, L, num_splits=1)
assert code() == 0 and torch.equal(bad, same) and not torch.equal(bad, good)

# expert ids: 70 is beyond the declared 64 experts (negative ids mean "no expert" and pass)
ids = torch.tensor([[1, 5], [70, 2], [-1, 3]], dtype=torch.int32, device=dev)
moe_ops.moe_align(ids, 64, 0); assert code() == 904
moe_ops.moe_align(torch.tensor([[1, 5], [63, -1]], dtype=torch.int32, device=dev), 64, 0); assert code() == 0
print("CHECKED-BUILD-OK")
'''


@pytest.mark.gpu
@pytest.mark.timeout(900)
def test_checked_build_reports_indices_beyond_the_declared_sizes():
    env = dict(os.environ, LLB_DEBUG_BOUNDS="1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", CHILD], cwd=ROOT, env=env, capture_output=True, text=True, timeout=800)
    assert r.returncode == 0 and "CHECKED-BUILD-OK" in r.stdout, (r.stdout[-1500:], r.stderr[-3000:])


def test_checked_build_compiles_and_exports_its_setters():
    """No GPU needed: the -DLLB_DEBUG_BOUNDS variant cross-compiles and exports one setter per translation unit."""
    import ctypes

    from lightllm_b200 import build
    from lightllm_b200.ops._native import _DEBUG_UNITS

    lib = ctypes.CDLL(str(build.build_kernels(verbose=False, debug_bounds=True)))
    for unit in _DEBUG_UNITS:
        assert hasattr(lib, f"llb_debug_set_bounds_{unit}")
    regular = ctypes.CDLL(str(build.build_kernels(verbose=False)))
    assert not hasattr(regular, "llb_debug_set_bounds_moe")     # the regular build carries no checks
