"""Run under torchrun on >= 2 GPUs: the decoder as two pipeline stages on two GPUs against all layers on one GPU.

Rank 0 first decodes the prompts alone with the whole model; then both ranks run the same requests as stages (stage 0
embeds and runs the first half of the layers, stage 1 the second half, the head and the sampler; the streams, and the
IndexCache rows the second stage reuses, cross by point-to-point sends; the sampled tokens come back by broadcast).
The texts must share long prefixes (at the stage boundary the residual streams are written out between the two mixing
kernels instead of staying inside one fused launch, so a sampled token may flip).
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from stkernel_b200.ops import _lib  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    from stkernel_b200.config import EngineConfig, ParallelConfig, SchedulerConfig, flash_config
    from stkernel_b200.models.dsv4 import RandomSource, build_model_weights
    from stkernel_b200.parallel.pipeline import PipeStage, stage_starts_inside_index_group
    from stkernel_b200.runtime.engine import Engine, SamplingParams
    cfg = flash_config(num_layers=4, n_routed_experts=16, vocab_size=4096)
    gp = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gp).tolist() for n in (700, 60)]
    params = SamplingParams(temperature=1.0, seed=11, max_tokens=6)
    sched = SchedulerConfig(max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=256, graph_cap=0)
    whole = None
    if rank == 0:
        ec = EngineConfig(model=cfg, sched=sched).validate()
        eng = Engine(ec, build_model_weights(cfg, RandomSource(0), dev, head_fp8=True), dev, max_context=1024)
        whole = eng.generate(prompts, params)
        torch.cuda.synchronize()
        del eng
    dist.barrier()
    pipe = PipeStage(pp_rank=rank, pp_size=world)
    rng = pipe.layer_range(cfg.num_hidden_layers)
    ec = EngineConfig(model=cfg, parallel=ParallelConfig(pp_size=world), sched=sched).validate()
    weights = build_model_weights(cfg, RandomSource(0), dev, head_fp8=True, layer_range=rng)
    eng = Engine(ec, weights, dev, max_context=1024, pipe=pipe)
    staged = eng.generate(prompts, params)
    torch.cuda.synchronize()
    _lib.check_status()
    assert sorted(eng.kv.swa_cache.keys()) == list(range(*rng))
    mine = torch.tensor(staged, device=dev)
    ref0 = mine.clone()
    dist.broadcast(ref0, 0)
    assert torch.equal(mine, ref0), "stages disagree on the sampled tokens"
    if rank == 0:
        info = {"world": world, "layers_of_stage_0": list(rng), "whole": whole, "staged": staged,
                "next_stage_reuses_topk_rows": stage_starts_inside_index_group(cfg, *PipeStage(1, world).layer_range(cfg.num_hidden_layers))}
        print("PP_INFO " + json.dumps(info), flush=True)
        pre = []
        for a, b in zip(staged, whole):
            n = 0
            while n < len(a) and a[n] == b[n]:
                n += 1
            pre.append(n)
        info["common_prefix"] = pre
        assert min(pre) >= 2 and sum(pre) >= 8, (staged, whole)
        print("PP_OK " + json.dumps(info), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
