"""Engine observability. The reference only returns a per-step token count
(reference: src/control/core.py:127-131); this adds per-phase host time, prefix hit rate,
KV occupancy, preemptions and per-request TTFT/TPOT, and can dump JSONL or a Prometheus
text exposition.
"""

from __future__ import annotations

import json
import time
from dataclasses import dataclass, field

__all__ = ["EngineMetrics", "RequestTiming"]


@dataclass
class RequestTiming:
    seq_id: int
    prompt_tokens: int
    completion_tokens: int
    ttft_s: float
    tpot_s: float
    e2e_s: float


@dataclass
class EngineMetrics:
    steps: int = 0
    requests_added: int = 0
    requests_finished: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    sampled_tokens: int = 0
    schedule_s: float = 0.0
    execute_s: float = 0.0
    update_s: float = 0.0
    kv_usage: float = 0.0
    kv_usage_peak: float = 0.0
    preemptions: int = 0
    prefix_hit_tokens: int = 0
    prefix_query_tokens: int = 0
    max_decode_batch: int = 0
    finished: list[RequestTiming] = field(default_factory=list)
    keep_request_timings: int = 4096

    def on_step(self, sched, outputs, prefill_tokens: int, *, schedule_s: float, execute_s: float,
                update_s: float, kv_usage: float, preemptions: int, kv, now: float, sampled_total: int = 0,
                finished_lookup=None) -> None:
        self.steps += 1
        self.prefill_tokens += prefill_tokens
        self.decode_tokens += len(sched.decodes)
        self.max_decode_batch = max(self.max_decode_batch, len(sched.decodes))
        self.schedule_s += schedule_s
        self.execute_s += execute_s
        self.update_s += update_s
        self.kv_usage = kv_usage
        self.kv_usage_peak = max(self.kv_usage_peak, kv_usage)
        self.preemptions = preemptions
        self.prefix_hit_tokens = kv.num_prefix_hit_tokens
        self.prefix_query_tokens = kv.num_prefix_query_tokens
        self.sampled_tokens = sampled_total
        # decode rows that neither start nor finish a request need no per-request bookkeeping
        for seq in sched.prefills:
            if not seq.t_first_token and seq.num_known_completion_tokens > 0:
                seq.t_first_token = now
        for o in outputs:
            if not o.is_finished:
                continue
            seq = finished_lookup(o.seq_id)
            if seq is None:
                continue
            seq.t_finished = now
            self.requests_finished += 1
            if len(self.finished) < self.keep_request_timings:
                n = seq.num_known_completion_tokens
                first = seq.t_first_token or now
                self.finished.append(RequestTiming(
                    seq.seq_id, seq.num_prompt_tokens, n, first - seq.t_arrival,
                    (now - first) / max(1, n - 1), now - seq.t_arrival))

    @property
    def prefix_hit_rate(self) -> float:
        return self.prefix_hit_tokens / self.prefix_query_tokens if self.prefix_query_tokens else 0.0

    def summary(self) -> dict:
        d = {k: getattr(self, k) for k in (
            "steps", "requests_added", "requests_finished", "prefill_tokens", "decode_tokens",
            "sampled_tokens", "schedule_s", "execute_s", "update_s", "kv_usage", "kv_usage_peak",
            "preemptions", "prefix_hit_tokens", "prefix_query_tokens", "max_decode_batch")}
        d["prefix_hit_rate"] = self.prefix_hit_rate
        if self.finished:
            tt = sorted(r.ttft_s for r in self.finished)
            tp = sorted(r.tpot_s for r in self.finished)
            d["ttft_ms_p50"] = 1e3 * tt[len(tt) // 2]
            d["ttft_ms_p99"] = 1e3 * tt[min(len(tt) - 1, int(len(tt) * 0.99))]
            d["tpot_ms_p50"] = 1e3 * tp[len(tp) // 2]
            d["tpot_ms_p99"] = 1e3 * tp[min(len(tp) - 1, int(len(tp) * 0.99))]
        return d

    def to_jsonl(self, path: str, **extra) -> None:
        rec = dict(ts=time.time(), **self.summary(), **extra)
        with open(path, "a", encoding="utf-8") as f:
            f.write(json.dumps(rec) + "\n")

    def to_prometheus(self, prefix: str = "xv") -> str:
        lines = []
        for k, v in self.summary().items():
            if isinstance(v, (int, float)):
                lines.append(f"# TYPE {prefix}_{k} gauge")
                lines.append(f"{prefix}_{k} {v}")
        return "\n".join(lines) + "\n"
