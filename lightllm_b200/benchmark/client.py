"""Load generator for a running server: fixed concurrency (closed loop) or fixed request rate (open loop),
random-token or text prompts, streaming `/generate_stream`; reports output tokens/s, request throughput and the
p50 / p90 / p99 of time-to-first-token, inter-token latency and end-to-end latency.  This is the measurement the
headline numbers of the reference are quoted with (output tok/s per box at fixed concurrency, p50 TTFT / ITL).

    python -m lightllm_b200.benchmark.client --url http://127.0.0.1:8000 --concurrency 256 --num_requests 512 \
        --input_len 1024 --output_len 256 [--qps 20] [--prefix_share 0.5] [--multiturn 3]

Reference: test/benchmark/service/{benchmark_client,benchmark_qps,benchmark_prompt_cache,benchmark_multiturn}.py.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import random
import statistics
import time
from typing import List, Optional


def percentile(xs: List[float], p: float) -> Optional[float]:
    if not xs:
        return None
    xs = sorted(xs)
    k = min(len(xs) - 1, max(0, int(round(p / 100.0 * (len(xs) - 1)))))
    return xs[k]


def make_prompts(n: int, input_len: int, vocab: int, seed: int, prefix_share: float) -> List[List[int]]:
    """Random token-id prompts; the first `prefix_share` of every prompt is common (prefix-cache workloads)."""
    rng = random.Random(seed)
    lo = min(1000, vocab // 10)              # stay clear of special ids at both ends, also for small vocabularies
    hi = max(vocab - lo, lo + 1)
    shared = [rng.randrange(lo, hi) for _ in range(int(input_len * prefix_share))]
    return [shared + [rng.randrange(lo, hi) for _ in range(input_len - len(shared))] for _ in range(n)]


async def one_request(session, url: str, prompt, output_len: int, record: dict, extra_params: dict):
    body = {"inputs": prompt, "parameters": {"max_new_tokens": output_len, "ignore_eos": True, "do_sample": False,
                                             **extra_params}}
    t0 = time.perf_counter()
    stamps, text = [], []
    try:
        async with session.post(url + "/generate_stream", json=body) as resp:
            if resp.status != 200:
                record["errors"] += 1
                return None
            async for raw in resp.content:
                line = raw.decode("utf-8", "ignore").strip()
                if not line.startswith("data:"):
                    continue
                stamps.append(time.perf_counter())
                try:
                    text.append(json.loads(line[5:])["token"]["text"])
                except Exception:
                    pass
    except Exception:
        record["errors"] += 1
        return None
    if not stamps:
        record["errors"] += 1
        return None
    record["ttft"].append(stamps[0] - t0)
    record["e2e"].append(stamps[-1] - t0)
    if len(stamps) > 1:
        record["itl"].append((stamps[-1] - stamps[0]) / (len(stamps) - 1))
    record["tokens"] += len(stamps)
    return "".join(text)


async def run(args) -> dict:
    import aiohttp

    prompts = make_prompts(args.num_requests, args.input_len, args.vocab_size, args.seed, args.prefix_share)
    record = {"ttft": [], "itl": [], "e2e": [], "tokens": 0, "errors": 0}
    extra = json.loads(args.parameters) if args.parameters else {}
    queue: asyncio.Queue = asyncio.Queue()
    for p in prompts:
        queue.put_nowait(p)
    timeout = aiohttp.ClientTimeout(total=args.timeout)
    conn = aiohttp.TCPConnector(limit=0)
    async with aiohttp.ClientSession(timeout=timeout, connector=conn) as session:
        t0 = time.perf_counter()

        async def conversation(prompt):
            # multi-turn: every turn appends the previous answer's token count of fresh random tokens
            ctx = list(prompt)
            for turn in range(max(1, args.multiturn)):
                await one_request(session, args.url, ctx, args.output_len, record, extra)
                ctx = ctx + make_prompts(1, args.output_len + 16, args.vocab_size, args.seed + turn + len(ctx), 0.0)[0]

        if args.qps > 0:  # open loop: Poisson arrivals
            tasks = []
            rng = random.Random(args.seed)
            while not queue.empty():
                tasks.append(asyncio.create_task(conversation(queue.get_nowait())))
                await asyncio.sleep(rng.expovariate(args.qps))
            await asyncio.gather(*tasks)
        else:  # closed loop: `concurrency` workers

            async def worker():
                while True:
                    try:
                        p = queue.get_nowait()
                    except asyncio.QueueEmpty:
                        return
                    await conversation(p)

            await asyncio.gather(*[worker() for _ in range(args.concurrency)])
        wall = time.perf_counter() - t0
    ms = lambda v: None if v is None else round(v * 1e3, 2)  # noqa: E731
    return {"requests": len(record["e2e"]), "errors": record["errors"], "wall_s": round(wall, 3),
            "output_tokens_per_s": round(record["tokens"] / wall, 1), "requests_per_s": round(len(record["e2e"]) / wall, 3),
            "ttft_ms": {p: ms(percentile(record["ttft"], p)) for p in (50, 90, 99)},
            "itl_ms": {p: ms(percentile(record["itl"], p)) for p in (50, 90, 99)},
            "e2e_ms": {p: ms(percentile(record["e2e"], p)) for p in (50, 90, 99)},
            "mean_itl_ms": ms(statistics.mean(record["itl"])) if record["itl"] else None,
            "config": {"concurrency": args.concurrency, "qps": args.qps, "input_len": args.input_len,
                       "output_len": args.output_len, "prefix_share": args.prefix_share, "multiturn": args.multiturn}}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--qps", type=float, default=0.0, help="> 0: open-loop Poisson arrivals instead of fixed concurrency")
    ap.add_argument("--num_requests", type=int, default=512)
    ap.add_argument("--input_len", type=int, default=1024)
    ap.add_argument("--output_len", type=int, default=256)
    ap.add_argument("--vocab_size", type=int, default=128256)
    ap.add_argument("--prefix_share", type=float, default=0.0)
    ap.add_argument("--multiturn", type=int, default=1)
    ap.add_argument("--parameters", default=None, help="JSON of extra sampling parameters")
    ap.add_argument("--timeout", type=float, default=3600)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    print(json.dumps(asyncio.run(run(args))))


if __name__ == "__main__":
    main()
