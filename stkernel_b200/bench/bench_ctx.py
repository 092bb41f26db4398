"""Time-to-first-token and decode rate at long contexts, from one streaming request per context.

    python -m stkernel_b200.bench.bench_ctx [--ctx 2000,32000,128000] [--out-tokens 128] [--conc 1,8,16,32]

`--ctx` mode: a unique prompt of about N tokens is streamed; TTFT measures prefill (prompt tokens /
TTFT = prefill tok/s), the remaining deltas measure decode (bench/bench-ctx.py:28-82 in the reference;
llama-bench style pp/tg figures of pp-ctx-benchy.py and tg-llama-benchy.py come from the same split).
`--conc` mode: a concurrency sweep of short prompts, aggregate completion tok/s (bench/bench-conc.py).
"""
from __future__ import annotations

import argparse
import time
from concurrent.futures import ThreadPoolExecutor

from .http_client import Client, summarize, unique_prompt


def run_ctx(cl: Client, ctx_tokens: int, out_tokens: int, seed: int, words_per_token: float = 0.55) -> dict:
    prompt = "Summarise the following notes.\n" + unique_prompt(seed, int(ctx_tokens * words_per_token))
    r = cl.chat_stream(prompt, out_tokens, 0.0, ignore_eos=True)
    return {"ctx": ctx_tokens, "prompt_tokens": r.prompt_tokens, "ttft_s": r.ttft,
            "prefill_tok_s": r.prompt_tokens / r.ttft if r.ttft > 0 else 0.0, "decode_tok_s": r.decode_tok_s,
            "gap_ms_p50": 1e3 * summarize(r.gaps)["median"], "gap_ms_max": 1e3 * summarize(r.gaps)["max"]}


def run_conc(cl: Client, conc: int, out_tokens: int, seed: int) -> dict:
    t0 = time.time()
    with ThreadPoolExecutor(max_workers=conc) as ex:
        toks = list(ex.map(lambda s: cl.chat(unique_prompt(s, 24), out_tokens, 0.8, ignore_eos=True)["usage"]["completion_tokens"],
                           [seed * 977 + i for i in range(conc)]))
    dt = time.time() - t0
    return {"conc": conc, "tokens": sum(toks), "seconds": dt, "tok_s": sum(toks) / dt, "per_stream_tok_s": sum(toks) / dt / conc}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="deepseek-v4-flash")
    ap.add_argument("--ctx", default="2000,32000,128000")
    ap.add_argument("--conc", default="")
    ap.add_argument("--out-tokens", type=int, default=128)
    ap.add_argument("--seed", type=int, default=1)
    a = ap.parse_args(argv)
    cl = Client(a.base, a.model)
    if a.conc:
        for c in [int(x) for x in a.conc.split(",")]:
            r = run_conc(cl, c, a.out_tokens, a.seed)
            print(f"C={r['conc']:>3}: {r['tokens']:>6} tok / {r['seconds']:6.1f}s => {r['tok_s']:8.1f} tok/s "
                  f"({r['per_stream_tok_s']:.1f}/stream)", flush=True)
        return 0
    for ctx in [int(x) for x in a.ctx.split(",")]:
        r = run_ctx(cl, ctx, a.out_tokens, a.seed + ctx)
        print(f"ctx~{ctx // 1000:>3}K ({r['prompt_tokens']} tok): TTFT {r['ttft_s']:.2f}s = pp {r['prefill_tok_s']:.0f} tok/s | "
              f"tg {r['decode_tok_s']:.1f} tok/s | gap p50 {r['gap_ms_p50']:.1f} ms max {r['gap_ms_max']:.1f} ms", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
