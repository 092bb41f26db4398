"""Per-kernel device time of real (not serialised) steps, from the torch profiler (CUPTI).

Prints the kernels of `--steps` steps sorted by total device time, the busy time as the union
of kernel intervals (overlapping streams are not double counted) and the idle share — the same
accounting as the reference's trace bucketing (bench/profile-step.py:166-281).

    python -m stkernel_b200.bench.kernel_table --mode decode --conc 1 --graphs 1

Under `python -m torch.distributed.run --nproc-per-node N` the model is tensor/expert parallel over the N ranks
(`--layers` is then the total layer count) and rank 0 prints its own table.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import tempfile
from typing import Dict, List, Tuple

import torch

BUCKETS = [
    ("comms", re.compile(r"nccl|allreduce|all_reduce|oneshot|twoshot|symm", re.I)),
    ("moe", re.compile(r"expert|moe_|router", re.I)),
    ("attn/indexer", re.compile(r"sparse_mla|indexer|topk|swa_indices|compress", re.I)),
    ("gemm", re.compile(r"gemm", re.I)),
    ("mhc", re.compile(r"mhc", re.I)),
    ("norm/rope/quant", re.compile(r"rmsnorm|rope|quant|swiglu|embed", re.I)),
    ("sampler", re.compile(r"gumbel|markov|accept", re.I)),
    ("memops", re.compile(r"memcpy|memset|copy|fill", re.I)),
]


def bucket_of(name: str) -> str:
    for b, rx in BUCKETS:
        if rx.search(name):
            return b
    return "other"


def interval_union(iv: List[Tuple[float, float]]) -> float:
    """Total length of the union of [start, end) intervals."""
    tot, cur_s, cur_e = 0.0, None, None
    for s, e in sorted(iv):
        if cur_e is None or s > cur_e:
            if cur_e is not None:
                tot += cur_e - cur_s
            cur_s, cur_e = s, e
        else:
            cur_e = max(cur_e, e)
    if cur_e is not None:
        tot += cur_e - cur_s
    return tot


def summarise_trace(path: str, steps: int) -> Dict:
    ev = json.load(open(path))["traceEvents"]
    ks = [e for e in ev if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset") and "dur" in e]
    per: Dict[str, List[float]] = {}
    for e in ks:
        per.setdefault(e["name"], []).append(e["dur"])
    busy = interval_union([(e["ts"], e["ts"] + e["dur"]) for e in ks])
    span = (max(e["ts"] + e["dur"] for e in ks) - min(e["ts"] for e in ks)) if ks else 0.0
    buckets: Dict[str, float] = {}
    for n, d in per.items():
        buckets[bucket_of(n)] = buckets.get(bucket_of(n), 0.0) + sum(d)
    return {"kernels": per, "busy_us": busy, "span_us": span, "buckets": buckets, "steps": steps}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="decode")
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--conc", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--chunk", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--graphs", type=int, default=1)
    ap.add_argument("--top", type=int, default=30)
    ap.add_argument("--out", default="")
    ap.add_argument("--pdl", type=int, default=0,
                    help="keep programmatic dependent launch on: a kernel's recorded time then includes its wait for "
                         "the previous kernel, so per-kernel figures overlap (off by default for the table)")
    ap.add_argument("--time-steps", type=int, default=0,
                    help="first time this many steps by CUDA events without the profiler and print us/step")
    ap.add_argument("--timeline", default="", help="also write the last step's launches in start order "
                                                   "(start offset, duration, gap to the previous end, stream, name) to this file")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="single process only: build rank 0's weight shard of a tensor/expert-parallel group of this "
                         "size and run it alone, without collectives (the sums are incomplete, so the values mean "
                         "nothing; the kernels, their shapes and their times are those of one rank of that group)")
    ap.add_argument("--index-cache", type=int, default=1, help="0: every ratio-4 layer computes its own top-k (IndexCache off)")
    ap.add_argument("--spec", type=int, default=0, help="decode mode: DSpark speculative steps with this many draft tokens "
                                                        "(3 draft layers; every step verifies conc * (spec + 1) rows)")
    a = ap.parse_args()
    from ..config import EngineConfig, ParallelConfig, SchedulerConfig, SpecConfig, flash_config
    from ..models.dsv4 import RandomSource, build_model_weights
    from ..runtime.engine import Engine, SamplingParams
    from .decode_bench import add_synthetic_requests, fill_caches_synthetic

    from ..ops import _lib
    _lib.call("stk_set_pdl", a.pdl)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(local)
    comm = None
    if world > 1:
        import torch.distributed as dist
        from ..parallel.communicator import Communicator
        dist.init_process_group("nccl", device_id=dev)
        comm = Communicator(device=dev, use_symm=True)
    spec_on = a.spec > 0 and a.mode == "decode"
    if spec_on:
        cfg = flash_config(num_layers=a.layers, n_mtp_layers=3, use_index_cache=bool(a.index_cache),
                           dspark_target_layer_ids=(a.layers // 4, a.layers // 2, a.layers - 1))
    else:
        cfg = flash_config(num_layers=a.layers, use_index_cache=bool(a.index_cache))
    shard = a.shard_of if world == 1 else 1
    group = max(world, shard)
    spec_cfg = SpecConfig(method="dspark", num_speculative_tokens=a.spec, markov_topk=512, temperature=0.6) if spec_on else SpecConfig()
    ec = EngineConfig(model=cfg, parallel=ParallelConfig(tp_size=group, ep_size=group, fused_collectives=True),
                      sched=SchedulerConfig(max_model_len=a.ctx + 8192, max_num_seqs=max(a.conc, 2),
                                            max_num_batched_tokens=a.chunk, graph_cap=256 if a.graphs else 0),
                      spec=spec_cfg).validate()
    src = RandomSource(0)
    weights = build_model_weights(cfg, src, dev, rank, group, head_fp8=True)
    draft = None
    if spec_on:
        from ..spec.dspark import build_draft_weights
        draft = build_draft_weights(cfg, src, weights, dev, rank, group)
    eng = Engine(ec, weights, dev, comm, rank, max_context=a.ctx + 8192, draft_weights=draft)
    fill_caches_synthetic(eng)
    if a.mode == "decode":
        add_synthetic_requests(eng, a.conc, a.ctx, (a.steps + 3 * a.time_steps + 8) * (a.spec + 1), cfg.vocab_size, 3,
                               0.6 if spec_on else 0.0)
    else:
        g = torch.Generator().manual_seed(0)
        eng.add_request(torch.randint(0, cfg.vocab_size, (a.chunk * (a.steps + 2),), generator=g).tolist(),
                        SamplingParams(max_tokens=1))
    for _ in range(2):
        eng.step()
    torch.cuda.synchronize()
    timed_us = None
    if a.time_steps > 0:
        # the same steps without the profiler, by CUDA events (tokens forced, so no host read-back between steps)
        g2 = torch.Generator().manual_seed(5)
        forced = [torch.randint(0, cfg.vocab_size, (max(a.conc, 1),), generator=g2).tolist() for _ in range(a.time_steps)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for rep in range(2):
            e0.record()
            for i in range(a.time_steps):
                eng.step(forced[i] if a.mode == "decode" and not spec_on else None)
            e1.record()
            torch.cuda.synchronize()
            timed_us = e0.elapsed_time(e1) * 1e3 / a.time_steps
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        for _ in range(a.steps):
            eng.step()
        torch.cuda.synchronize()
    path = os.path.join(tempfile.gettempdir(), f"stk_trace_{rank}.json")
    prof.export_chrome_trace(path)
    s = summarise_trace(path, a.steps)
    lines = [f"mode={a.mode} conc={a.conc} ctx={a.ctx} layers={a.layers} graphs={a.graphs} steps={a.steps} gpus={world}"
             + (f" shard-of={shard}" if shard > 1 else "")
             + (f"  [{timed_us:.1f} us/step by CUDA events over {a.time_steps} steps, no profiler, pdl={a.pdl}]" if timed_us else ""),
             f"busy {s['busy_us'] / a.steps:.1f} us/step, span {s['span_us'] / a.steps:.1f} us/step, "
             f"idle {100 * (1 - s['busy_us'] / max(s['span_us'], 1e-9)):.1f} %"]
    for b, v in sorted(s["buckets"].items(), key=lambda x: -x[1]):
        lines.append(f"  bucket {b:16s} {v / a.steps:9.1f} us/step  {100 * v / max(s['busy_us'], 1e-9):5.1f} %")
    rows = sorted(s["kernels"].items(), key=lambda x: -sum(x[1]))[:a.top]
    for n, d in rows:
        lines.append(f"  {sum(d) / a.steps:9.1f} us/step {len(d) // a.steps:4d}x/step avg {sum(d) / len(d):7.1f} us  {n[:70]}")
    text = "\n".join(lines)
    if a.timeline and rank == 0:
        ev = [e for e in json.load(open(path))["traceEvents"]
              if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset") and "dur" in e]
        ev.sort(key=lambda e: e["ts"])
        per_step = len(ev) // a.steps
        last = ev[len(ev) - per_step:]
        t0, prev_end, tl = last[0]["ts"], last[0]["ts"], []
        for e in last:
            tl.append(f"{e['ts'] - t0:9.1f} {e['dur']:7.1f} {e['ts'] - prev_end:7.1f}  s{e.get('args', {}).get('stream', '?')}  {e['name'][:90]}")
            prev_end = max(prev_end, e["ts"] + e["dur"])
        open(a.timeline, "w").write("# start_us dur_us gap_us stream name\n" + "\n".join(tl) + "\n")
    if rank == 0:
        print(text, flush=True)
        if a.out:
            open(a.out, "w").write(text + "\n")
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        os._exit(0)


if __name__ == "__main__":
    main()
