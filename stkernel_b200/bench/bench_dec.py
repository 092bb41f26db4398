"""Low-variance decode benchmark over HTTP: long generations at C=1/2/4 with acceptance per sample.

    python -m stkernel_b200.bench.bench_dec [--reps 6] [--out-tokens 768] [--conc 1,2,4] [--base URL]

Each sample is `conc` concurrent chat requests of `--out-tokens` tokens on unique prompts; the rate is
total completion tokens over wall time.  The `/metrics` delta around a sample gives its acceptance, the
main source of rate variance with probabilistic drafts, so an outlier can be told from a real effect
(method of bench/bench-dec.py:31-140 in the reference).
"""
from __future__ import annotations

import argparse
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Tuple

from .http_client import Client, acceptance, spec_counters, summarize, unique_prompt

TOPICS = ["the water cycle", "binary search trees", "the history of the bicycle", "how vaccines train immunity",
          "plate tectonics", "the rules of cricket", "sourdough fermentation", "orbital mechanics"]


def one(cl: Client, seed: int, out_tokens: int, temperature: float) -> int:
    topic = TOPICS[seed % len(TOPICS)]
    r = cl.chat(f"Explain {topic} in about {out_tokens} tokens, in detail. (reference {seed}: {unique_prompt(seed, 6)})",
                out_tokens, temperature, ignore_eos=True)
    return r["usage"]["completion_tokens"]


def sweep(cl: Client, conc: int, seed: int, out_tokens: int, temperature: float) -> Tuple[int, float]:
    t0 = time.time()
    with ThreadPoolExecutor(max_workers=conc) as ex:
        toks = list(ex.map(lambda s: one(cl, s, out_tokens, temperature), [seed * 131 + i for i in range(conc)]))
    return sum(toks), time.time() - t0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="deepseek-v4-flash")
    ap.add_argument("--reps", type=int, default=6)
    ap.add_argument("--out-tokens", type=int, default=768)
    ap.add_argument("--conc", default="1,2,4")
    ap.add_argument("--temperature", type=float, default=0.95)
    ap.add_argument("--tag", default="")
    a = ap.parse_args(argv)
    cl = Client(a.base, a.model)
    for c in [int(x) for x in a.conc.split(",")]:
        rates: List[float] = []
        for r in range(a.reps):
            m0 = spec_counters(cl.metrics())
            toks, dt = sweep(cl, c, r + 1 + c * 1000, a.out_tokens, a.temperature)
            acc = acceptance(m0, spec_counters(cl.metrics()))
            rates.append(toks / dt)
            suffix = f" | acc {acc['acc']:6.1%} (raw {acc['raw']:5.1%}, {acc['accepted_per_step']:.2f}/step)" if acc["raw"] else ""
            print(f"{a.tag}C={c} rep{r + 1}: {toks:>5} tok / {dt:>5.1f}s => {toks / dt:>7.1f} tok/s{suffix}", flush=True)
        s = summarize(rates)
        print(f"{a.tag}C={c} SUMMARY mean {s['mean']:.1f} | median {s['median']:.1f} | min {s['min']:.1f} | max {s['max']:.1f}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
