"""Retrieval quality gate over HTTP: planted facts at fixed depths of long filler documents.

    python -m stkernel_b200.bench.check_quality [--ctx 2000,32000,128000] [--needle 256000]

Three facts are planted at 25/50/75 % depth of a document of about N tokens and asked back one by one
at temperature 0; every accepted substring must appear in the answer.  The gate is all 9 of 9
(bench/check-quality.py:17-80 in the reference).  `--needle N` plants the same facts in one N-token
document and also asks for all of them in a single generation (bench/needle-256k.py:24-99).  With
random weights the gate fails by construction; the tool is for real checkpoints.
"""
from __future__ import annotations

import argparse
import random
from typing import List, Sequence, Tuple

from .http_client import Client

WORDS = ("river stone lantern copper meadow signal orbit timber harbor velvet cinder garnet willow quartz ember "
         "prairie falcon mosaic tundra ledger beacon saddle thistle anchor marble").split()
FACTS: Sequence[Tuple[str, str, Sequence[str]]] = (
    ("The calibration constant for the Meridian array is 8127.",
     "What is the calibration constant for the Meridian array?", ("8127",)),
    ("Dr. Halvorsen signed the tundra survey on 14 March 1997.",
     "Who signed the tundra survey, and on what date?", ("halvorsen", "14 march 1997")),
    ("The quarry's emergency shutoff is valve K-42 on the north wall.",
     "Which valve is the quarry's emergency shutoff, and where is it?", ("k-42", "north")),
)


def filler(n_tokens: float, rng: random.Random) -> str:
    return " ".join(rng.choice(WORDS) for _ in range(int(n_tokens / 1.3)))


def build_document(ctx_tokens: int, seed: int, depths: Sequence[float] = (0.25, 0.5, 0.75)) -> str:
    rng = random.Random(seed)
    chunks: List[str] = []
    prev = 0.0
    for (sentence, _, _), d in zip(FACTS, depths):
        chunks += [filler((d - prev) * ctx_tokens, rng), sentence]
        prev = d
    chunks.append(filler((1.0 - prev) * ctx_tokens, rng))
    return "\n".join(chunks)


def grade(answer: str, expect: Sequence[str]) -> bool:
    a = answer.lower()
    return all(e in a for e in expect)


def ask(cl: Client, doc: str, question: str, max_tokens: int = 120) -> str:
    r = cl.chat(f"Document:\n{doc}\n\nAnswer from the document only, in one short sentence. {question}", max_tokens, 0.0)
    return r["choices"][0]["message"].get("content") or ""


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="deepseek-v4-flash")
    ap.add_argument("--ctx", default="2000,32000,128000")
    ap.add_argument("--needle", type=int, default=0)
    ap.add_argument("--seed", type=int, default=7)
    a = ap.parse_args(argv)
    cl = Client(a.base, a.model)
    total = ok = 0
    ctxs = [a.needle] if a.needle else [int(x) for x in a.ctx.split(",")]
    for ctx in ctxs:
        doc = build_document(ctx, a.seed + ctx)
        hits = []
        for _, q, expect in FACTS:
            ans = ask(cl, doc, q)
            good = grade(ans, expect)
            hits.append("o" if good else "X")
            total += 1
            ok += good
            if not good:
                print(f"    MISS ctx~{ctx // 1000}K q={q!r} -> {ans[:110]!r}")
        print(f"ctx~{ctx // 1000:>3}K  {' '.join(hits)}", flush=True)
        if a.needle:
            ans = ask(cl, doc, "List the calibration constant, who signed the tundra survey and when, and the quarry's "
                               "emergency shutoff valve with its location.", 240)
            multi = all(grade(ans, e) for _, _, e in FACTS)
            print(f"multi-fact single generation: {'o' if multi else 'X'}")
            total += 1
            ok += multi
    print(f"=> {ok}/{total} correct")
    return 0 if ok == total else 1


if __name__ == "__main__":
    raise SystemExit(main())
