"""DSpark speculative decoding on the Flash-shaped model: tokens per second with and without drafts,
accepted tokens per step and per-position acceptance.

    python -m stkernel_b200.bench.spec_bench [--layers 6] [--ctx 32768] [--conc 1,16] [--steps 40]

Random-init weights: the drafter has learned nothing, so acceptance is what chance gives (about zero); the
run measures the cost side -- a verify step over 1+N rows per sequence, the context-KV insert, the 3-layer
draft block and the sequential Markov sampling over the full vocabulary -- and checks the step end to end
at the production shapes (vocabulary 129280, Markov rank 256, top-512 gather, temperature 0.6).  With a
trained drafter the tokens emitted per step are 1 + accepted-per-step at the same step cost.
"""
from __future__ import annotations

import argparse
import json
import time
from typing import Dict, List

import torch

from ..config import EngineConfig, ParallelConfig, SchedulerConfig, SpecConfig, flash_config
from ..models.dsv4 import RandomSource, build_model_weights
from ..ops import _lib
from ..runtime.engine import Engine, SamplingParams
from ..spec.dspark import build_draft_weights
from .decode_bench import add_synthetic_requests, fill_caches_synthetic


def run(layers: int, ctx: int, conc: int, steps: int, n_spec: int, temperature: float, spec: bool, shard_of: int = 1) -> Dict:
    dev = torch.device("cuda:0")
    n_mtp = 3 if spec else 0
    cfg = flash_config(layers, n_mtp_layers=n_mtp,
                       dspark_target_layer_ids=(layers // 4, layers // 2, layers - 1) if spec else ())
    sc = SchedulerConfig(max_model_len=ctx + 4096, max_num_seqs=max(conc, 2), max_num_batched_tokens=4096, graph_cap=256)
    par = ParallelConfig(tp_size=shard_of, ep_size=shard_of, fused_collectives=True) if shard_of > 1 else ParallelConfig()
    ec = EngineConfig(model=cfg, parallel=par, sched=sc, spec=SpecConfig(method="dspark" if spec else "none", num_speculative_tokens=n_spec,
                                                            markov_topk=512, temperature=temperature)).validate()
    src = RandomSource(0)
    # shard_of > 1: rank 0's shard of a tensor/expert-parallel group of that size run alone, without collectives (the
    # values mean nothing; kernels, shapes and times are those of one rank of the group)
    w = build_model_weights(cfg, src, dev, 0, shard_of, head_fp8=True)
    dw = build_draft_weights(cfg, src, w, dev, 0, shard_of) if spec else None
    eng = Engine(ec, w, dev, max_context=ctx + 4096, draft_weights=dw)
    fill_caches_synthetic(eng)
    ids = add_synthetic_requests(eng, conc, ctx, steps * (n_spec + 1) + 64, cfg.vocab_size, 7)
    for rid in ids:
        eng.requests[rid].params.temperature = temperature
    for _ in range(4):
        eng.step()
    torch.cuda.synchronize()
    _lib.check_status()
    m0 = (eng.metrics.generation_tokens_total, eng.metrics.spec_num_drafts, eng.metrics.spec_num_accepted_tokens,
          list(eng.metrics.spec_accepted_per_pos))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        eng.step()
    e1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    _lib.check_status()
    toks = eng.metrics.generation_tokens_total - m0[0]
    drafts = eng.metrics.spec_num_drafts - m0[1]
    acc = eng.metrics.spec_num_accepted_tokens - m0[2]
    per_pos = [a - (m0[3][i] if i < len(m0[3]) else 0) for i, a in enumerate(eng.metrics.spec_accepted_per_pos)]
    return {"spec": spec, "shard_of": shard_of, "conc": conc, "ctx": ctx, "layers": layers, "steps": steps, "ms_per_step_device": e0.elapsed_time(e1) / steps,
            "ms_per_step_wall": 1e3 * wall / steps, "tokens": toks, "tok_s": toks / wall,
            "accepted_per_step": acc / drafts if drafts else 0.0,
            "per_position_acceptance": [round(a / drafts, 4) for a in per_pos] if drafts else []}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--conc", default="1,16")
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--spec-tokens", type=int, default=5)
    ap.add_argument("--temperature", type=float, default=0.6)
    ap.add_argument("--out", default="")
    ap.add_argument("--shard-of", type=int, default=1, help="time rank 0's shard of a group of this size, alone")
    a = ap.parse_args()
    rows: List[Dict] = []
    for c in [int(x) for x in a.conc.split(",")]:
        for spec in (False, True):
            r = run(a.layers, a.ctx, c, a.steps, a.spec_tokens, a.temperature, spec, a.shard_of)
            rows.append(r)
            print(json.dumps(r), flush=True)
            torch.cuda.empty_cache()
    if a.out:
        with open(a.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")


if __name__ == "__main__":
    main()
