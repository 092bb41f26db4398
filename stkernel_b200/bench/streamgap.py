"""Co-ingest smoothness probe: stream one long decode, fire a large prefill beside it mid-generation,
and report the decode stream's chunk rate before / during / after the ingest plus the largest
inter-token gaps (bench/streamgap.py:1-85 in the reference; its ledger row reads 25.2 / 1.2 / 26.1
chunk/s, the starvation that chunked prefill with decode-first scheduling is meant to bound).

    python -m stkernel_b200.bench.streamgap [--ingest-tokens 34000] [--out-tokens 1500] [--delay 6]
"""
from __future__ import annotations

import argparse
import json
import threading
import time
import urllib.request
from typing import Dict, List, Optional, Tuple

from .http_client import Client, unique_prompt


def window_rates(stamps: List[float], t0: float, i0: Optional[float], i1: Optional[float]) -> Dict[str, float]:
    def rate(lo: float, hi: float) -> float:
        return sum(1 for t in stamps if lo <= t <= hi) / max(hi - lo, 1e-9)
    if not stamps:
        return {}
    if i0 is None or i1 is None:
        return {"all": rate(t0, stamps[-1])}
    return {"before": rate(t0, i0), "during": rate(i0, i1), "after": rate(i1, max(stamps[-1], i1 + 1e-9))}


def largest_gaps(stamps: List[float], t0: float, k: int = 8) -> List[Tuple[float, float]]:
    return sorted(((stamps[i] - stamps[i - 1], stamps[i] - t0) for i in range(1, len(stamps))), reverse=True)[:k]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="deepseek-v4-flash")
    ap.add_argument("--ingest-tokens", type=int, default=34000)
    ap.add_argument("--out-tokens", type=int, default=1500)
    ap.add_argument("--delay", type=float, default=6.0)
    a = ap.parse_args(argv)
    cl = Client(a.base, a.model, timeout=900)
    window: Dict[str, float] = {}

    def ingest() -> None:
        window["t0"] = time.time()
        cl.chat(unique_prompt(time.time_ns(), int(a.ingest_tokens * 0.55)) + " End.", 1, 0.0)
        window["t1"] = time.time()

    body = {"model": a.model, "messages": [{"role": "user", "content": "Explain geothermal power generation in great detail."}],
            "max_tokens": a.out_tokens, "temperature": 0.95, "stream": True, "ignore_eos": True,
            "chat_template_kwargs": {"thinking": False}}
    req = urllib.request.Request(a.base + "/v1/chat/completions", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    stamps: List[float] = []
    th = None
    t_start = time.time()
    with urllib.request.urlopen(req, timeout=900) as r:
        for raw in r:
            line = raw.decode().strip()
            if not line.startswith("data: ") or line[6:] == "[DONE]":
                continue
            ch = json.loads(line[6:]).get("choices") or []
            if ch and (ch[0].get("delta") or {}).get("content"):
                stamps.append(time.time())
            if th is None and stamps and time.time() - t_start > a.delay:
                th = threading.Thread(target=ingest, daemon=True)
                th.start()
    if th:
        th.join(timeout=600)
    print(f"decode chunks: {len(stamps)}, wall {(stamps[-1] - t_start) if stamps else 0:.1f}s")
    rates = window_rates(stamps, t_start, window.get("t0"), window.get("t1"))
    if "during" in rates:
        print(f"ingest window: {window['t0'] - t_start:.1f}s .. {window['t1'] - t_start:.1f}s")
    for k, v in rates.items():
        print(f"decode rate {k.upper():7s}: {v:6.1f} chunk/s")
    print("largest token gaps (s @ t):")
    for g, t in largest_gaps(stamps, t_start):
        print(f"  {g:6.2f}s @ {t:6.1f}s")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
