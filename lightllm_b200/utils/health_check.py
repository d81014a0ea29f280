"""/health logic: healthy if a token was produced within HEALTH_TIMEOUT seconds, or nothing is in
flight; otherwise a tiny probe request is sent through the whole pipeline.
Reference: lightllm/utils/health_check.py:14-44.
"""
from __future__ import annotations

import os
import time

HEALTH_TIMEOUT = int(os.getenv("HEALTH_TIMEOUT", 200))


async def health_check(manager, make_sampling_params) -> bool:
    if os.getenv("DEBUG_HEALTHCHECK_RETURN_FAIL") == "true":
        return False
    last = manager.latest_success_infer_time_mark.get_value()
    if time.time() - last < HEALTH_TIMEOUT and manager.run_reqs_count_mark.get_value() > 0:
        return True
    try:
        sp = make_sampling_params({"max_new_tokens": 1, "do_sample": False})
        import asyncio

        async def probe():
            async for _ in manager.generate([1, 2, 3], sp, None, None, is_health_req=True):
                pass

        await asyncio.wait_for(probe(), timeout=HEALTH_TIMEOUT)
        return True
    except Exception:
        return False
