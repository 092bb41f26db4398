"""HTTP client helpers shared by the serving benchmarks (stdlib only, so they run anywhere)."""
from __future__ import annotations

import json
import time
import urllib.request
from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Tuple

from ..runtime.metrics import parse_prometheus


@dataclass
class StreamResult:
    ttft: float = 0.0                 # request sent -> first content/reasoning delta
    total: float = 0.0
    gaps: List[float] = field(default_factory=list)    # seconds between successive deltas
    text: str = ""
    completion_tokens: int = 0
    prompt_tokens: int = 0

    @property
    def decode_tok_s(self) -> float:
        span = self.total - self.ttft
        return (self.completion_tokens - 1) / span if span > 0 and self.completion_tokens > 1 else 0.0


class Client:
    def __init__(self, base: str = "http://127.0.0.1:8000", model: str = "deepseek-v4-flash", timeout: float = 1800.0):
        self.base, self.model, self.timeout = base.rstrip("/"), model, timeout

    def _req(self, path: str, body: Optional[Dict[str, Any]]):
        data = json.dumps(body).encode() if body is not None else None
        return urllib.request.Request(self.base + path, data=data, headers={"Content-Type": "application/json"},
                                      method="POST" if body is not None else "GET")

    def post(self, path: str, body: Dict[str, Any]) -> Dict[str, Any]:
        with urllib.request.urlopen(self._req(path, body), timeout=self.timeout) as r:
            return json.load(r)

    def get_text(self, path: str, timeout: float = 10.0) -> str:
        with urllib.request.urlopen(self.base + path, timeout=timeout) as r:
            return r.read().decode()

    def chat(self, content: str, max_tokens: int, temperature: float = 0.0, thinking: bool = False, **extra) -> Dict[str, Any]:
        return self.post("/v1/chat/completions", {"model": self.model, "messages": [{"role": "user", "content": content}],
                                                  "max_tokens": max_tokens, "temperature": temperature,
                                                  "chat_template_kwargs": {"thinking": thinking}, **extra})

    def chat_stream(self, content: str, max_tokens: int, temperature: float = 0.0, **extra) -> StreamResult:
        body = {"model": self.model, "messages": [{"role": "user", "content": content}], "max_tokens": max_tokens,
                "temperature": temperature, "stream": True, "stream_options": {"include_usage": True},
                "chat_template_kwargs": {"thinking": False}, **extra}
        res = StreamResult()
        t0 = time.perf_counter()
        last = None
        with urllib.request.urlopen(self._req("/v1/chat/completions", body), timeout=self.timeout) as r:
            for raw in r:
                line = raw.decode().strip()
                if not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                obj = json.loads(line[6:])
                if obj.get("usage"):
                    res.completion_tokens = obj["usage"].get("completion_tokens", 0)
                    res.prompt_tokens = obj["usage"].get("prompt_tokens", 0)
                for ch in obj.get("choices", []):
                    d = ch.get("delta", {})
                    piece = (d.get("content") or "") + (d.get("reasoning_content") or "")
                    if piece:
                        now = time.perf_counter()
                        if last is None:
                            res.ttft = now - t0
                        else:
                            res.gaps.append(now - last)
                        last = now
                        res.text += piece
        res.total = time.perf_counter() - t0
        return res

    def metrics(self) -> Dict[str, float]:
        try:
            return parse_prometheus(self.get_text("/metrics"))
        except OSError:
            return {}


def spec_counters(metrics: Dict[str, float]) -> Dict[str, float]:
    """Speculative-decoding counters with labels collapsed (per-position series summed per name)."""
    out: Dict[str, float] = {}
    for k, v in metrics.items():
        name = k.split("{")[0]
        if "spec_decode" in name:
            out[name] = out.get(name, 0.0) + v
    return out


def acceptance(before: Dict[str, float], after: Dict[str, float]) -> Dict[str, float]:
    """Acceptance over a counter delta.  `raw` = accepted / drafted tokens by exact counter name; `acc` = the
    substring-sum convention of older ledgers (accept-like over draft-like counters: it counts the
    per-position series again and the draft *count* in the denominator), kept so that old and new
    numbers can be compared on one scale (bench/bench-dec.py:90-119 in the reference)."""
    d = {k: after.get(k, 0.0) - before.get(k, 0.0) for k in after}
    acc = sum(v for k, v in d.items() if "accept" in k)
    drafts = sum(v for k, v in d.items() if "draft" in k and "accept" not in k)
    out = {"acc": acc / drafts if drafts > 0 else 0.0}
    a = sum(v for k, v in d.items() if k.endswith("num_accepted_tokens_total"))
    n = sum(v for k, v in d.items() if k.endswith("num_draft_tokens_total"))
    steps = sum(v for k, v in d.items() if k.endswith("num_drafts_total"))
    out["raw"] = a / n if n > 0 else 0.0
    out["accepted_per_step"] = a / steps if steps > 0 else 0.0
    return out


def summarize(xs: List[float]) -> Dict[str, float]:
    s = sorted(xs)
    n = len(s)
    if not n:
        return {"mean": 0.0, "median": 0.0, "min": 0.0, "max": 0.0}
    med = s[n // 2] if n % 2 else (s[n // 2 - 1] + s[n // 2]) / 2
    return {"mean": sum(s) / n, "median": med, "min": s[0], "max": s[-1]}


def unique_prompt(seed: int, n_words: int) -> str:
    """A prompt no prefix cache has seen: deterministic pseudo-words keyed by the seed."""
    import random
    rng = random.Random(seed)
    syll = ["ka", "lo", "mi", "ren", "tu", "ves", "dor", "an", "shi", "pel", "qua", "zor", "ith", "bra", "nem", "ul"]
    return " ".join("".join(rng.choice(syll) for _ in range(rng.randint(1, 3))) for _ in range(n_words))
