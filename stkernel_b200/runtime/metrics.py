"""Prometheus-style counters with the metric names the reference's tools consume
(bench/bench-dec.py:60-119, launchers/dsv4-tp4-supervisor.sh:98-101)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List


@dataclass
class Metrics:
    requests_total: int = 0
    requests_finished: int = 0
    num_requests_running: int = 0
    num_requests_waiting: int = 0
    prompt_tokens_total: int = 0
    generation_tokens_total: int = 0
    steps_total: int = 0
    spec_num_drafts: int = 0
    spec_num_draft_tokens: int = 0
    spec_num_accepted_tokens: int = 0
    spec_accepted_per_pos: List[int] = field(default_factory=list)
    prefix_cache_resets: int = 0
    device_status_errors: int = 0
    kv_cache_usage: float = 0.0          # compressed-KV pool pages in use / pool size (the pool that grows with context)
    prefix_cache_queries: int = 0
    prefix_cache_hits: int = 0
    prefix_cache_hit_tokens: int = 0
    ttft_sum: float = 0.0                # time to first token over finished first tokens
    ttft_count: int = 0

    def record_spec(self, n_draft: int, n_accepted: int) -> None:
        """One verified draft of n_draft tokens of which the first n_accepted were accepted."""
        self.spec_num_drafts += 1
        self.spec_num_draft_tokens += n_draft
        self.spec_num_accepted_tokens += n_accepted
        while len(self.spec_accepted_per_pos) < n_draft:
            self.spec_accepted_per_pos.append(0)
        for i in range(n_accepted):
            self.spec_accepted_per_pos[i] += 1

    def render(self, model_name: str = "stk") -> str:
        lab = f'{{model_name="{model_name}"}}'
        rows = [
            ("vllm:num_requests_running", "gauge", self.num_requests_running),
            ("vllm:num_requests_waiting", "gauge", self.num_requests_waiting),
            ("vllm:prompt_tokens_total", "counter", self.prompt_tokens_total),
            ("vllm:generation_tokens_total", "counter", self.generation_tokens_total),
            ("vllm:request_success_total", "counter", self.requests_finished),
            ("vllm:spec_decode_num_drafts_total", "counter", self.spec_num_drafts),
            ("vllm:spec_decode_num_draft_tokens_total", "counter", self.spec_num_draft_tokens),
            ("vllm:spec_decode_num_accepted_tokens_total", "counter", self.spec_num_accepted_tokens),
            ("vllm:gpu_cache_usage_perc", "gauge", round(self.kv_cache_usage, 6)),
            ("vllm:prefix_cache_queries_total", "counter", self.prefix_cache_queries),
            ("vllm:prefix_cache_hits_total", "counter", self.prefix_cache_hits),
            ("stk:prefix_cache_hit_tokens_total", "counter", self.prefix_cache_hit_tokens),
            ("vllm:time_to_first_token_seconds_sum", "counter", round(self.ttft_sum, 6)),
            ("vllm:time_to_first_token_seconds_count", "counter", self.ttft_count),
            ("stk:engine_steps_total", "counter", self.steps_total),
            ("stk:prefix_cache_resets_total", "counter", self.prefix_cache_resets),
            ("stk:device_status_errors_total", "counter", self.device_status_errors),
        ]
        out = []
        for name, kind, val in rows:
            out.append(f"# TYPE {name} {kind}")
            out.append(f"{name}{lab} {val}")
        out.append("# TYPE vllm:spec_decode_num_accepted_tokens_per_pos_total counter")
        for i, v in enumerate(self.spec_accepted_per_pos):
            out.append(f'vllm:spec_decode_num_accepted_tokens_per_pos_total{{model_name="{model_name}",position="{i}"}} {v}')
        return "\n".join(out) + "\n"


def parse_prometheus(text: str) -> Dict[str, float]:
    """`name{labels}` -> value for every sample line."""
    out: Dict[str, float] = {}
    for line in text.splitlines():
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        try:
            key, val = line.rsplit(" ", 1)
            out[key] = float(val)
        except ValueError:
            continue
    return out


def acceptance_from_metrics(before: Dict[str, float], after: Dict[str, float]) -> Dict[str, float]:
    """Acceptance statistics from two metric snapshots: `raw` = accepted / drafted tokens,
    `acc` = the legacy convention (accepted + drafts) / (draft tokens + drafts) that counts the bonus
    token, mean accepted length per step, and per-position rates."""
    def delta(prefix: str) -> float:
        return sum(v - before.get(k, 0.0) for k, v in after.items() if k.startswith(prefix))

    drafts = delta("vllm:spec_decode_num_drafts_total")
    dtoks = delta("vllm:spec_decode_num_draft_tokens_total")
    acc = delta("vllm:spec_decode_num_accepted_tokens_total")
    out = {"drafts": drafts, "raw": acc / dtoks if dtoks else 0.0,
           "acc": (acc + drafts) / (dtoks + drafts) if dtoks + drafts else 0.0,
           "mean_accepted_len": acc / drafts if drafts else 0.0}
    per = {}
    for k, v in after.items():
        if k.startswith("vllm:spec_decode_num_accepted_tokens_per_pos_total"):
            pos = int(k.split('position="')[1].split('"')[0])
            per[pos] = (v - before.get(k, 0.0)) / drafts if drafts else 0.0
    out["per_position"] = [per[i] for i in sorted(per)]
    return out
