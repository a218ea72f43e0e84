"""Prometheus text metrics with vLLM-compatible names plus engine-specific counters, rendered by the front end from
its own request bookkeeping and the engine's `{"stats": true}` reply (reference: serve/openai_server.py:79-163)."""
from __future__ import annotations

import threading
from typing import Dict, List

_BUCKETS = {"ttft": [0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10, 30],
            "itl": [0.002, 0.005, 0.01, 0.02, 0.05, 0.1, 0.25, 0.5, 1],
            "e2e": [0.1, 0.5, 1, 2.5, 5, 10, 30, 60, 120],
            "queue": [0.001, 0.01, 0.05, 0.1, 0.5, 1, 5, 10]}


class Histogram:
    def __init__(self, buckets: List[float]):
        self.buckets, self.counts, self.sum, self.n = buckets, [0] * len(buckets), 0.0, 0

    def observe(self, v: float):
        self.sum += v
        self.n += 1
        for i, b in enumerate(self.buckets):
            if v <= b:
                self.counts[i] += 1

    def render(self, name: str, label: str) -> List[str]:
        out = [f"# TYPE {name} histogram"]
        for b, c in zip(self.buckets, self.counts):
            out.append(f'{name}_bucket{{le="{b}",{label}}} {c}')
        out += [f'{name}_bucket{{le="+Inf",{label}}} {self.n}', f"{name}_sum{{{label}}} {self.sum}", f"{name}_count{{{label}}} {self.n}"]
        return out


class Metrics:
    def __init__(self, model_name: str):
        self.label = f'model_name="{model_name}"'
        self.lock = threading.Lock()
        self.h = {k: Histogram(v) for k, v in _BUCKETS.items()}
        self.success: Dict[str, int] = {}
        self.prompt_tokens = self.generation_tokens = 0

    def finish(self, done: dict, e2e_s: float, itls: List[float]):
        with self.lock:
            self.h["ttft"].observe(done.get("ttft_ms", 0.0) / 1e3)
            self.h["queue"].observe(done.get("queue_ms", 0.0) / 1e3)
            self.h["e2e"].observe(e2e_s)
            for v in itls:
                self.h["itl"].observe(v)
            r = done.get("finish_reason", "stop")
            self.success[r] = self.success.get(r, 0) + 1
            self.generation_tokens += len(done.get("token_ids", []))

    def render(self, engine_stats: dict) -> str:
        L = self.label
        g = lambda k, d=0: engine_stats.get(k, d)
        lines = [
            "# TYPE vllm:num_requests_running gauge", f"vllm:num_requests_running{{{L}}} {g('running')}",
            "# TYPE vllm:num_requests_waiting gauge", f"vllm:num_requests_waiting{{{L}}} {g('waiting')}",
            "# TYPE vllm:kv_cache_usage_perc gauge",
            f"vllm:kv_cache_usage_perc{{{L}}} {g('kv_allocated') / max(g('kv_budget', 1), 1):.6f}",
            "# TYPE vllm:prompt_tokens_total counter", f"vllm:prompt_tokens_total{{{L}}} {g('prompt_tokens')}",
            "# TYPE vllm:generation_tokens_total counter", f"vllm:generation_tokens_total{{{L}}} {g('generation_tokens')}",
            "# TYPE spark_spec_rounds_total counter", f"spark_spec_rounds_total{{{L}}} {g('spec_rounds')}",
            "# TYPE spark_drafted_tokens_total counter", f"spark_drafted_tokens_total{{{L}}} {g('drafted_tokens')}",
            "# TYPE spark_accepted_drafts_total counter", f"spark_accepted_drafts_total{{{L}}} {g('accepted_drafts')}",
            "# TYPE spark_prefix_hit_tokens_total counter", f"spark_prefix_hit_tokens_total{{{L}}} {g('prefix_hit_tokens')}",
            "# TYPE spark_disk_restores_total counter", f"spark_disk_restores_total{{{L}}} {g('disk_restores')}",
        ]
        with self.lock:
            lines += self.h["ttft"].render("vllm:time_to_first_token_seconds", L)
            lines += self.h["itl"].render("vllm:time_per_output_token_seconds", L)
            lines += self.h["e2e"].render("vllm:e2e_request_latency_seconds", L)
            lines += self.h["queue"].render("vllm:request_queue_time_seconds", L)
            lines.append("# TYPE vllm:request_success_total counter")
            for r, c in sorted(self.success.items()):
                lines.append(f'vllm:request_success_total{{finished_reason="{r}",{L}}} {c}')
        return "\n".join(lines) + "\n"
