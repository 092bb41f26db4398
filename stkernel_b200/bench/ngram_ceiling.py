"""Offline upper bound for prompt-lookup (n-gram copy) drafting next to the parallel drafter.

    python -m stkernel_b200.bench.ngram_ceiling [--tokenizer DIR | --mode chars] FILES...

Under the seeded-Gumbel coupling the emitted token is the verifier's own sample whatever was proposed,
so the realised text IS the target sample and a deterministic copy proposal is accepted exactly where
it equals the realised continuation: acceptance of a copy drafter can be computed from transcripts
alone, before any engine work.  Three policies step through each document advancing 1 + accepted
tokens per step: the parallel drafter alone (accepted length drawn from its measured per-position
curve), a hybrid that copies when the context suffix match is at least `--threshold` tokens, and an
oracle that takes the better of the two at every step (method of bench/ngram-ceiling.py:1-40,81-196
in the reference).  Inputs: .txt (first --warmup tokens are context) or .jsonl rows with
prompt/completion or text.  `--mode chars` is a smoke test; do not quote its numbers.
"""
from __future__ import annotations

import argparse
import json
import random
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

DEFAULT_CURVE = "78.5,56.4,39.6,28.6,21.5"


def parse_curve(raw: str) -> List[float]:
    vals = [float(v) / 100.0 for v in raw.split(",") if v.strip()]
    if not vals or any(not 0.0 <= v <= 1.0 for v in vals):
        raise ValueError(f"bad per-position curve: {raw!r}")
    if any(b > a + 1e-9 for a, b in zip(vals, vals[1:])):
        raise ValueError(f"per-position curve must be non-increasing: {raw!r}")
    return vals


def accept_len_pmf(curve: Sequence[float]) -> List[float]:
    """P(accepted == m), m = 0..k, from the cumulative per-position acceptance."""
    c = [1.0, *curve, 0.0]
    return [c[m] - c[m + 1] for m in range(len(curve) + 1)]


def sample_accept_len(pmf: Sequence[float], rng: random.Random) -> int:
    x, acc = rng.random(), 0.0
    for m, p in enumerate(pmf):
        acc += p
        if x < acc:
            return m
    return len(pmf) - 1


def common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
    n = 0
    for x, y in zip(a, b):
        if x != y:
            break
        n += 1
    return n


class GramIndex:
    """Most recent end positions of every `nmin`-gram seen so far; grows with the decode position so
    that a lookup at position t can never see tokens at or after t."""

    def __init__(self, tokens: Sequence[int], nmin: int, keep: int = 64):
        self.tokens, self.nmin, self.keep = tokens, nmin, keep
        self.ends: Dict[Tuple[int, ...], List[int]] = {}
        self.upto = 0

    def reset(self) -> None:
        self.ends.clear()
        self.upto = 0

    def advance(self, t: int) -> None:
        for pos in range(max(self.upto, self.nmin), t + 1):
            bucket = self.ends.setdefault(tuple(self.tokens[pos - self.nmin:pos]), [])
            bucket.append(pos)
            if len(bucket) > self.keep:
                bucket.pop(0)
        self.upto = max(self.upto, t + 1)

    def longest(self, t: int, nmax: int) -> Tuple[int, int]:
        """(match length, position right after the earlier occurrence) for the suffix ending at t."""
        tk = self.tokens
        if t < self.nmin:
            return 0, -1
        best = (0, -1)
        for pos in reversed(self.ends.get(tuple(tk[t - self.nmin:t]), ())):
            if pos == t:
                continue
            n = self.nmin
            while n < nmax and pos - n - 1 >= 0 and tk[pos - n - 1] == tk[t - n - 1]:
                n += 1
            if (n, pos) > best:
                best = (n, pos)
        return best


def simulate(context: Sequence[int], generated: Sequence[int], pmf: Sequence[float], k: int = 5, nmin: int = 3,
             nmax: int = 16, threshold: int = 4, warmup: int = 64, keep: int = 64, seed: int = 0) -> Optional[Dict]:
    tokens = list(context) + list(generated)
    start = len(context)
    if start < nmin:
        start = max(start, min(warmup, len(tokens) - 1))
    if len(tokens) - start < 2:
        return None
    idx = GramIndex(tokens, nmin, keep)
    stats = {"gen_tokens": len(tokens) - start, "steps": {}, "copy_steps": 0, "copy_accepted": 0, "match_steps": 0}

    def copy_accept(t: int) -> Tuple[int, int]:
        idx.advance(t)
        n, pos = idx.longest(t, nmax)
        if n < threshold or pos < 0:
            return -1, n
        proposal = tokens[pos:min(pos + k, t)]             # only tokens that already exist may be copied
        if not proposal:
            return -1, n
        return common_prefix(proposal, tokens[t:t + k]), n

    for policy in ("drafter", "hybrid", "oracle"):
        rng = random.Random(seed)
        idx.reset()
        t, steps = start, 0
        while t < len(tokens):
            ds = sample_accept_len(pmf, rng)
            adv = 1 + ds
            if policy != "drafter":
                copied, n = copy_accept(t)
                if policy == "hybrid" and n >= threshold:
                    stats["match_steps"] += 1
                if copied >= 0 and policy == "oracle":
                    adv = 1 + max(copied, ds)
                elif copied >= 0:
                    adv = 1 + copied
                    stats["copy_steps"] += 1
                    stats["copy_accepted"] += copied
            steps += 1
            t += adv
        stats["steps"][policy] = steps
    return stats


def iter_docs(paths: Sequence[str]) -> Iterator[Tuple[str, str]]:
    for path in paths:
        with open(path, encoding="utf-8") as f:
            if path.endswith(".jsonl"):
                for line in f:
                    if line.strip():
                        row = json.loads(line)
                        if "completion" in row:
                            yield row.get("prompt", ""), row["completion"]
                        elif row.get("text"):
                            yield "", row["text"]
            else:
                yield "", f.read()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("files", nargs="+")
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--mode", default="tokens", choices=["tokens", "chars"])
    ap.add_argument("--curve", default=DEFAULT_CURVE)
    ap.add_argument("--k", type=int, default=5)
    ap.add_argument("--nmin", type=int, default=3)
    ap.add_argument("--nmax", type=int, default=16)
    ap.add_argument("--threshold", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=64)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    pmf = accept_len_pmf(parse_curve(a.curve))
    if a.mode == "chars" or not a.tokenizer:
        enc = lambda s: [ord(c) for c in s]
    else:
        from ..serve.tokenizer import HFTokenizer
        enc = HFTokenizer(a.tokenizer).encode
    tot = {"gen": 0, "drafter": 0, "hybrid": 0, "oracle": 0, "copy_steps": 0, "copy_acc": 0, "docs": 0}
    for prompt, completion in iter_docs(a.files):
        st = simulate(enc(prompt), enc(completion), pmf, a.k, a.nmin, a.nmax, a.threshold, a.warmup, seed=a.seed)
        if st is None:
            continue
        tot["docs"] += 1
        tot["gen"] += st["gen_tokens"]
        for p in ("drafter", "hybrid", "oracle"):
            tot[p] += st["steps"][p]
        tot["copy_steps"] += st["copy_steps"]
        tot["copy_acc"] += st["copy_accepted"]
    if not tot["docs"]:
        print("no usable documents")
        return 1
    base = tot["gen"] / tot["drafter"]
    print(f"{tot['docs']} docs, {tot['gen']} generated tokens" + ("  [chars mode: smoke test only]" if a.mode == "chars" else ""))
    for p in ("drafter", "hybrid", "oracle"):
        r = tot["gen"] / tot[p]
        print(f"  {p:8s} {r:5.2f} tok/step  ({100 * (r / base - 1):+5.1f} % vs drafter)")
    if tot["copy_steps"]:
        print(f"  copy proposals used on {tot['copy_steps']} steps, {tot['copy_acc'] / tot['copy_steps']:.2f} accepted each")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
