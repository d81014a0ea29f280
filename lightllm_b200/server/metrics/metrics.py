"""Prometheus metrics of the server (names follow the reference so dashboards keep working:
lightllm/server/metrics/metrics.py:6-53).  Duration buckets are 35 steps of x1.5 from 1.5 ms."""
from __future__ import annotations

from prometheus_client import CollectorRegistry, Counter, Gauge, Histogram, generate_latest

COUNTERS = ["lightllm_request_count", "lightllm_request_success", "lightllm_request_failure",
            "lightllm_batch_inference_count", "lightllm_prompt_tokens_total", "lightllm_generation_tokens_total"]
GAUGES = ["lightllm_batch_current_size", "lightllm_batch_next_size", "lightllm_batch_pause_size", "lightllm_queue_size",
          "lightllm_num_running_reqs", "lightllm_batch_current_max_tokens", "lightllm_cache_length",
          "lightllm_cache_ratio", "lightllm_cache_hit_rate", "lightllm_mtp_avg_token_per_step",
          "lightllm_gen_throughput"]
DURATION_HISTS = ["lightllm_request_duration", "lightllm_request_validation_duration",
                  "lightllm_request_inference_duration",
                  "lightllm_request_first_token_duration", "lightllm_request_mean_time_per_token_duration",
                  "lightllm_request_queue_duration", "lightllm_batch_inference_duration_bucket"]
LENGTH_HISTS = ["lightllm_request_input_length", "lightllm_request_generated_tokens", "lightllm_request_max_new_tokens"]

_DURATION_BUCKETS = [0.0015 * (1.5 ** i) for i in range(35)]
_LENGTH_BUCKETS = [2 ** i for i in range(0, 21)]


class Monitor:
    def __init__(self, model_name: str = "default"):
        self.registry = CollectorRegistry()
        self.model_name = model_name
        self._c = {n: Counter(n, n, ["model"], registry=self.registry) for n in COUNTERS}
        self._g = {n: Gauge(n, n, ["model"], registry=self.registry) for n in GAUGES}
        self._h = {n: Histogram(n, n, ["model"], buckets=_DURATION_BUCKETS, registry=self.registry)
                   for n in DURATION_HISTS}
        self._h.update({n: Histogram(n, n, ["model"], buckets=_LENGTH_BUCKETS, registry=self.registry)
                        for n in LENGTH_HISTS})

    def counter_inc(self, name: str, v: float = 1.0):
        if name in self._c:
            self._c[name].labels(self.model_name).inc(v)

    def gauge_set(self, name: str, v: float):
        if name in self._g:
            self._g[name].labels(self.model_name).set(v)

    def histogram_observe(self, name: str, v: float):
        if name in self._h:
            self._h[name].labels(self.model_name).observe(v)

    def generate_latest(self) -> bytes:
        return generate_latest(self.registry)
