"""Engine metrics in Prometheus text exposition format.

Counters, gauges and histograms kept in plain Python (no global registry, so
several engines can live in one process); ``render()`` produces the ``/metrics``
payload.  Metric names mirror the reference's (``aphrodite:`` prefix there,
``sonar:`` here): running/waiting requests, KV-cache usage, prefix-cache hit
rate, prompt/generation token counters, TTFT / end-to-end latency / time per
output token histograms, preemptions, request outcomes.

Parity: ``aphrodite/v1/metrics/loggers.py`` and ``stats.py``.
"""
from __future__ import annotations

import bisect
import threading
import time

from sonar_b200.request import SchedulerStats

_TTFT_BUCKETS = [0.001, 0.005, 0.01, 0.02, 0.04, 0.06, 0.08, 0.1, 0.25, 0.5, 0.75, 1, 2.5, 5, 7.5, 10, 20, 40, 80]
_E2E_BUCKETS = [0.3, 0.5, 0.8, 1, 1.5, 2, 2.5, 5, 10, 15, 20, 30, 40, 50, 60, 120, 240, 480, 960]
_TPOT_BUCKETS = [0.001, 0.0025, 0.005, 0.0075, 0.01, 0.015, 0.02, 0.03, 0.04, 0.05, 0.075, 0.1, 0.15, 0.2, 0.3, 0.5, 1]


class Histogram:
    def __init__(self, buckets: list[float]) -> None:
        self.buckets = buckets
        self.counts = [0] * (len(buckets) + 1)
        self.total = 0.0
        self.n = 0

    def observe(self, v: float) -> None:
        self.counts[bisect.bisect_left(self.buckets, v)] += 1
        self.total += v
        self.n += 1

    def quantile(self, q: float) -> float:
        if not self.n:
            return 0.0
        target, cum = q * self.n, 0
        for i, c in enumerate(self.counts):
            cum += c
            if cum >= target:
                return self.buckets[i] if i < len(self.buckets) else float("inf")
        return float("inf")

    def render(self, name: str, labels: str) -> list[str]:
        out, cum = [], 0
        for b, c in zip(self.buckets, self.counts):
            cum += c
            out.append(f'{name}_bucket{{{labels},le="{b}"}} {cum}')
        out.append(f'{name}_bucket{{{labels},le="+Inf"}} {self.n}')
        out.append(f"{name}_sum{{{labels}}} {self.total}")
        out.append(f"{name}_count{{{labels}}} {self.n}")
        return out


class EngineMetrics:
    def __init__(self, model_name: str, cost=None) -> None:
        """``cost``: a ``perf_model.ModelCost`` — with it the linear-layer FLOPs of every step are accumulated
        and a model-FLOPs-utilisation gauge is kept over a sliding window."""
        self.labels = f'model_name="{model_name}"'
        self.lock = threading.Lock()
        self.cost = cost
        self._window: list[tuple[float, float]] = []          # (time, flops) of recent steps
        self.gauges = {"num_requests_running": 0.0, "num_requests_waiting": 0.0, "kv_cache_usage_perc": 0.0,
                       "model_flops_utilization": 0.0}
        self.counters = {"prompt_tokens_total": 0.0, "generation_tokens_total": 0.0, "num_preemptions_total": 0.0,
                         "prefix_cache_queries_total": 0.0, "prefix_cache_hits_total": 0.0,
                         "spec_decode_num_draft_tokens_total": 0.0, "spec_decode_num_accepted_tokens_total": 0.0,
                         "request_arrivals_total": 0.0, "model_flops_total": 0.0}
        self.finished: dict[str, int] = {}
        self.ttft = Histogram(_TTFT_BUCKETS)
        self.e2e = Histogram(_E2E_BUCKETS)
        self.tpot = Histogram(_TPOT_BUCKETS)
        self.start = time.time()

    def update_from_scheduler(self, s: SchedulerStats) -> None:
        with self.lock:
            g, c = self.gauges, self.counters
            g["num_requests_running"], g["num_requests_waiting"] = s.num_running, s.num_waiting
            g["kv_cache_usage_perc"] = s.kv_cache_usage
            c["prompt_tokens_total"] += s.step_prompt_tokens
            c["generation_tokens_total"] += s.step_generation_tokens
            c["num_preemptions_total"] = s.num_preempted
            c["prefix_cache_queries_total"] = s.prefix_cache_queries
            c["prefix_cache_hits_total"] = s.prefix_cache_hits
            c["spec_decode_num_draft_tokens_total"] = s.spec_num_drafts
            c["spec_decode_num_accepted_tokens_total"] = s.spec_num_accepted
            if self.cost is not None:
                new = s.step_prompt_tokens + s.step_generation_tokens
                if new:
                    from sonar_b200.utils.perf_model import peaks
                    flops, _ = self.cost.step(new, s.num_running or 1)
                    c["model_flops_total"] += flops
                    now = time.time()
                    self._window.append((now, flops))
                    while self._window and now - self._window[0][0] > 10.0:
                        self._window.pop(0)
                    span = max(now - self._window[0][0], 1e-3) if len(self._window) > 1 else None
                    if span:
                        g["model_flops_utilization"] = sum(f for _, f in self._window[1:]) / span / peaks()[0]

    def request_arrived(self, n_prompt: int) -> None:
        with self.lock:
            self.counters["request_arrivals_total"] += 1

    def request_finished(self, reason: str) -> None:
        with self.lock:
            self.finished[reason] = self.finished.get(reason, 0) + 1

    def observe_ttft(self, seconds: float) -> None:
        with self.lock:
            self.ttft.observe(seconds)

    def observe_e2e(self, seconds: float, n_out: int) -> None:
        with self.lock:
            self.e2e.observe(seconds)
            if n_out > 1:
                self.tpot.observe(seconds / n_out)

    def render(self) -> str:
        with self.lock:
            lines: list[str] = []
            for k, v in self.gauges.items():
                lines += [f"# TYPE sonar:{k} gauge", f"sonar:{k}{{{self.labels}}} {v}"]
            for k, v in self.counters.items():
                lines += [f"# TYPE sonar:{k} counter", f"sonar:{k}{{{self.labels}}} {v}"]
            lines.append("# TYPE sonar:request_success_total counter")
            for reason, n in sorted(self.finished.items()):
                lines.append(f'sonar:request_success_total{{{self.labels},finished_reason="{reason}"}} {n}')
            for name, h in (("time_to_first_token_seconds", self.ttft), ("e2e_request_latency_seconds", self.e2e),
                            ("time_per_output_token_seconds", self.tpot)):
                lines.append(f"# TYPE sonar:{name} histogram")
                lines += h.render(f"sonar:{name}", self.labels)
            return "\n".join(lines) + "\n"
