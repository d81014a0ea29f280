"""Kernel variant autotuner and tuned-config store.

A kernel family (today: the bf16 GEMM and its tile / split variants) registers its candidates; the store keeps, per
device name and static key (e.g. N, K, epilogue), the best candidate for every tuned run key (M) in a JSON file and
answers look-ups with the nearest tuned run key.  Files shipped with the package live in
`lightllm_b200/kernel_configs/<device>/<kernel>.json`; newly tuned entries go to `$LLB_KERNEL_CONFIG_DIR` (default
`~/.cache/lightllm_b200/kernel_configs`) and shadow the shipped ones.

`LLB_AUTOTUNE_LEVEL`: 0 (default) use stored entries only; 1 tune the keys that are missing when a model warms up;
2 re-tune every key at warm-up.  With several ranks the candidates are split across the ranks of a host (gloo) group
and the timings are all-gathered, so every rank stores the same winner.

    python -m lightllm_b200.utils.autotuner --model llama3-8b --tp 1        # tune a model's GEMM shapes, print the table

Reference: lightllm/common/triton_utils/autotuner.py (`@autotune`, static / run keys, nearest-neighbour look-up,
distributed benchmarking, LIGHTLLM_TRITON_AUTOTUNE_LEVEL) and lightllm/common/kernel_config.py.
"""
from __future__ import annotations

import bisect
import json
import os
import threading
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

PKG_DIR = Path(__file__).resolve().parent.parent / "kernel_configs"


def autotune_level() -> int:
    try:
        return int(os.environ.get("LLB_AUTOTUNE_LEVEL", os.environ.get("LIGHTLLM_TRITON_AUTOTUNE_LEVEL", "0")))
    except ValueError:
        return 0


def device_key(name: Optional[str] = None) -> str:
    if name is None:
        try:
            import torch

            name = torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"
        except Exception:
            name = "cpu"
    return name.replace(" ", "_").replace("/", "_")


class KernelConfigStore:
    """kernel -> static key -> sorted [(run key, config)]."""

    def __init__(self, device: Optional[str] = None, user_dir: Optional[str] = None):
        self.device = device_key(device)
        self.user_dir = Path(user_dir or os.environ.get("LLB_KERNEL_CONFIG_DIR") or
                             Path.home() / ".cache" / "lightllm_b200" / "kernel_configs")
        self._tables: Dict[str, Dict[str, List[Tuple[int, dict]]]] = {}
        self._lock = threading.Lock()

    def _paths(self, kernel: str):
        return [PKG_DIR / self.device / f"{kernel}.json", self.user_dir / self.device / f"{kernel}.json"]

    def _load(self, kernel: str):
        t = self._tables.get(kernel)
        if t is not None:
            return t
        merged: Dict[str, Dict[int, dict]] = {}
        for p in self._paths(kernel):  # the user's file shadows the shipped one
            if p.exists():
                try:
                    data = json.loads(p.read_text())
                except (OSError, ValueError):
                    continue
                for skey, runs in data.items():
                    merged.setdefault(skey, {}).update({int(k): v for k, v in runs.items()})
        t = {skey: sorted(runs.items()) for skey, runs in merged.items()}
        self._tables[kernel] = t
        return t

    def lookup(self, kernel: str, static_key: str, run_key: int) -> Optional[dict]:
        """Config tuned for the run key nearest to `run_key` (ties go to the larger one); None if nothing is stored."""
        runs = self._load(kernel).get(static_key)
        if not runs:
            return None
        keys = [k for k, _ in runs]
        i = bisect.bisect_left(keys, run_key)
        if i == 0:
            return runs[0][1]
        if i == len(keys):
            return runs[-1][1]
        lo, hi = runs[i - 1], runs[i]
        return hi[1] if (hi[0] - run_key) <= (run_key - lo[0]) else lo[1]

    def has(self, kernel: str, static_key: str, run_key: int) -> bool:
        return any(k == run_key for k, _ in self._load(kernel).get(static_key, []))

    def store(self, kernel: str, static_key: str, run_key: int, config: dict, save: bool = True):
        with self._lock:
            t = self._load(kernel)
            runs = dict(t.get(static_key, []))
            runs[int(run_key)] = config
            t[static_key] = sorted(runs.items())
            if save:
                p = self._paths(kernel)[1]
                p.parent.mkdir(parents=True, exist_ok=True)
                existing = {}
                if p.exists():
                    try:
                        existing = json.loads(p.read_text())
                    except (OSError, ValueError):
                        existing = {}
                existing.setdefault(static_key, {})[str(int(run_key))] = config
                tmp = p.with_suffix(".tmp")
                tmp.write_text(json.dumps(existing, indent=1, sort_keys=True))
                tmp.replace(p)


_STORE: Optional[KernelConfigStore] = None


def store() -> KernelConfigStore:
    global _STORE
    if _STORE is None:
        _STORE = KernelConfigStore()
    return _STORE


def reset_store(new: Optional[KernelConfigStore] = None):
    global _STORE
    _STORE = new


def tune(candidates: Sequence[dict], bench: Callable[[dict], float], group=None) -> Tuple[dict, List[Tuple[float, dict]]]:
    """Times every candidate with `bench` (seconds or any monotone cost; exceptions count as infinity) and returns
    (best, all results).  With a process group the candidates are dealt round-robin to its ranks and the results
    all-gathered, so that all ranks agree on the winner."""
    rank, world = 0, 1
    if group is not None:
        import torch.distributed as dist

        rank, world = dist.get_rank(group), dist.get_world_size(group)
    mine = []
    for i, c in enumerate(candidates):
        if i % world != rank:
            continue
        try:
            t = float(bench(c))
        except Exception:
            t = float("inf")
        mine.append((t, i))
    results = mine
    if group is not None:
        import torch.distributed as dist

        gathered = [None] * world
        dist.all_gather_object(gathered, mine, group=group)
        results = [x for part in gathered for x in part]
    results.sort()
    scored = [(t, candidates[i]) for t, i in results]
    return scored[0][1], scored


# ------------------------------------------------------------------ bf16 GEMM
GEMM_KERNEL = "gemm_bf16"
# `bn` selectors understood by ops.gemm: 0 automatic plan, 64 / 128 / 256 one-CTA tiles, 512 CTA-pair tiles,
# 1000 + 10 * accumulators + splits cluster kernel (+ 100: 128-column tiles), 2000 + splits one-CTA tiles and
# 3000 + splits CTA-pair tiles with K split through the L2 workspace (x000: as many splits as fit)
GEMM_CANDIDATES = [{"bn": b} for b in (0, 64, 128, 256, 512, 1011, 1012, 1014, 1021, 1111, 1112,
                                       2000, 2002, 2004, 3000, 3001, 3002, 3004)]


def gemm_static_key(N: int, K: int, epi: str) -> str:
    return f"N={N},K={K},epi={epi}"


def gemm_lookup(M: int, N: int, K: int, epi: str) -> int:
    """The tuned `bn` selector for this problem, 0 (the built-in plan) when nothing is stored."""
    cfg = store().lookup(GEMM_KERNEL, gemm_static_key(N, K, epi), M)
    return int(cfg["bn"]) if cfg else 0


def tune_gemm(M: int, N: int, K: int, epi: str = "store", group=None, reps: int = 16, save: bool = True) -> dict:
    """Times the GEMM variants on random operands (CUDA-graph replays over rotating copies, L2 flushed) and stores
    the winner for (N, K, epi) at run key M."""
    import torch

    from .. import ops
    from ..ops import reference as ref
    from ..benchmark.gemm_bench import timeit_graph

    dev = torch.device("cuda")
    copies = max(1, min(reps, int((1 << 30) // max((M * K + N * K) * 2, 1))))
    xs = [(torch.randn(M, K, device=dev) * 0.5).bfloat16() for _ in range(copies)]
    ws = [(torch.randn(N, K, device=dev) * 0.05).bfloat16() for _ in range(copies)]
    res = torch.randn(M, N, device=dev).bfloat16() if epi == "residual" else None
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    del ref

    def bench(c):
        fn = lambda i: ops.gemm(xs[i % copies], ws[i % copies], epi=epi, residual=res, bn=c["bn"])  # noqa: E731
        fn(0)  # unsupported variants raise here
        torch.cuda.synchronize()
        return timeit_graph(fn, flush, n=9, reps=reps)

    best, scored = tune(GEMM_CANDIDATES, bench, group)
    t_best = scored[0][0]
    t_auto = next((t for t, c in scored if c["bn"] == 0), float("inf"))
    if t_auto <= t_best * 1.03:  # within measurement noise of the built-in plan: keep the plan
        best, t_best = {"bn": 0}, t_auto
    store().store(GEMM_KERNEL, gemm_static_key(N, K, epi), M, {"bn": best["bn"], "us": round(t_best * 1e3, 2)},
                  save=save)
    return best


def model_gemm_shapes(cfg: dict, tp: int = 1) -> List[Tuple[int, int, str]]:
    """(N, K, epilogue) of the per-rank GEMMs of a dense decoder layer and the head."""
    H = cfg["hidden_size"]
    hq, hkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    D = cfg.get("head_dim") or H // hq
    I = cfg["intermediate_size"]
    return [((hq + 2 * hkv) * D // tp, H, "store"), (H, hq * D // tp, "residual" if tp == 1 else "store"),
            (2 * I // tp, H, "gated_silu"), (H, I // tp, "residual" if tp == 1 else "store"),
            (cfg["vocab_size"] // tp, H, "f32")]


def tune_model(cfg: dict, tp: int = 1, Ms: Iterable[int] = (1, 8, 16, 32, 64, 128, 192, 256), group=None,
               force: bool = False, log=print):
    st = store()
    for N, K, epi in model_gemm_shapes(cfg, tp):
        for M in Ms:
            if not force and st.has(GEMM_KERNEL, gemm_static_key(N, K, epi), M):
                continue
            best = tune_gemm(M, N, K, epi, group)
            if log:
                log(json.dumps({"M": M, "N": N, "K": K, "epi": epi, **st.lookup(GEMM_KERNEL, gemm_static_key(N, K, epi), M)}))
            del best


def main():
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b", help="a name known to bench.py or a directory with config.json")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--ms", default="1,8,16,32,64,128,192,256", help="row counts (decode batch sizes) to tune")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--out", default=None, help="directory for the JSON table (default: the user cache)")
    a = ap.parse_args()
    if a.out:
        reset_store(KernelConfigStore(user_dir=a.out))
    if os.path.isdir(a.model):
        from ..models.base import load_config

        cfg = load_config(a.model)
    else:
        presets = {"llama3-8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                                     intermediate_size=14336, vocab_size=128256),
                   "llama3-70b": dict(hidden_size=8192, num_attention_heads=64, num_key_value_heads=8,
                                      intermediate_size=28672, vocab_size=128256)}
        cfg = presets[a.model]
    tune_model(cfg, a.tp, Ms=[int(x) for x in a.ms.split(",")], force=a.force)


if __name__ == "__main__":
    main()
