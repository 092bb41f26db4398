"""Run a few eager steps of the Flash-shaped model inside a cudaProfilerStart/Stop range, for
`ncu --profile-from-start off` captures (launch lists and single-kernel profiles).

    python -m stkernel_b200.bench.profile_step --mode decode --conc 1 --ctx 32768 --steps 2
    python -m stkernel_b200.bench.profile_step --mode prefill --chunk 1024 --ctx 4096
"""
from __future__ import annotations

import argparse

import torch

from ..config import EngineConfig, SchedulerConfig, flash_config
from ..models.dsv4 import RandomSource, build_model_weights
from ..ops import _lib
from ..runtime.engine import Engine, SamplingParams
from .decode_bench import add_synthetic_requests, fill_caches_synthetic


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="decode", choices=["decode", "prefill"])
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--conc", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--chunk", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    cfg = flash_config(num_layers=a.layers, n_routed_experts=a.experts)
    ec = EngineConfig(model=cfg, sched=SchedulerConfig(max_model_len=a.ctx + 4096, max_num_seqs=max(a.conc, 2),
                                                       max_num_batched_tokens=a.chunk, graph_cap=0)).validate()
    eng = Engine(ec, build_model_weights(cfg, RandomSource(0), dev, head_fp8=True), dev, max_context=a.ctx + 4096)
    fill_caches_synthetic(eng)
    if a.mode == "decode":
        add_synthetic_requests(eng, a.conc, a.ctx, a.steps + a.warmup + 2, cfg.vocab_size, 3)
        for _ in range(a.warmup):
            eng.step()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for _ in range(a.steps):
            eng.step()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    else:
        g = torch.Generator().manual_seed(0)
        n = a.chunk * (a.warmup + a.steps)
        eng.add_request(torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(), SamplingParams(max_tokens=1))
        for _ in range(a.warmup):
            eng.step()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for _ in range(a.steps):
            eng.step()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    _lib.check_status()
    print("profiled", a.mode, "launch calls", _lib.launch_count)


if __name__ == "__main__":
    main()
