"""Run under torchrun on >= 2 GPUs: decode context parallelism across real ranks.

A small tensor-parallel model decodes the same prompts twice: with every rank holding all ratio-4 cache pages, and with
the pages dealt over the ranks (local indexer scoring, cross-rank candidate merge, selected rows staged on every rank).
The sampled texts (same seeds) must share long prefixes (the two runs add attention terms in different orders), every rank must hold
only its own pages, and the timings of a decode step of both runs are reported.
"""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from stkernel_b200.ops import _lib  # noqa: E402
from stkernel_b200.parallel.communicator import Communicator  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    comm = Communicator(device=dev, use_symm=True)
    from stkernel_b200.config import EngineConfig, ParallelConfig, SchedulerConfig, flash_config
    from stkernel_b200.models.dsv4 import RandomSource, build_model_weights
    from stkernel_b200.runtime.engine import Engine, SamplingParams
    cfg = flash_config(num_layers=3, n_routed_experts=16, vocab_size=4096)
    weights = build_model_weights(cfg, RandomSource(0), dev, rank, world, head_fp8=True)
    gp = torch.Generator().manual_seed(3)
    # 4 tokens per compressed row, 64 rows per page: 9000 tokens reach the 36th page and give more rows (2250) than the top-k keeps (2048) of the ratio-4 caches
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gp).tolist() for n in (9000, 300)]
    out = {"world": world}
    toks = {}
    for dcp in (1, world):
        ec = EngineConfig(model=cfg, parallel=ParallelConfig(tp_size=world, ep_size=world, dcp_size=dcp),
                          sched=SchedulerConfig(max_model_len=12288, max_num_seqs=4, max_num_batched_tokens=512,
                                                graph_cap=0)).validate()
        eng = Engine(ec, weights, dev, comm, rank, max_context=12288)
        ids = [eng.add_request(p, SamplingParams(temperature=1.0, seed=11, max_tokens=10)) for p in prompts]
        peak, step_ms = 0, []
        while eng.has_work():
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            eng.step()
            torch.cuda.synchronize()
            step_ms.append((time.perf_counter() - t0) * 1e3)
            peak = max(peak, eng.kv.c4.pages_in_use)
        _lib.check_status()
        toks[dcp] = [list(eng.requests[i].output) for i in ids]
        out[f"dcp{dcp}"] = {"c4_pages_peak": peak, "c4_pool": eng.kv.c4.num_pages,
                            "eager_decode_step_ms_median": sorted(step_ms[-8:])[4],
                            "topk_merges": eng.model.stats["dcp_topk_merges"]}
        dist.barrier()
    mine = torch.tensor(toks[world], device=dev)
    ref0 = mine.clone()
    dist.broadcast(ref0, 0)
    assert torch.equal(mine, ref0), "ranks disagree on the sampled tokens"

    def prefix(a, b):
        n = 0
        while n < len(a) and a[n] == b[n]:
            n += 1
        return n
    pre = [prefix(x, y) for x, y in zip(toks[1], toks[world])]
    out["common_prefix"] = pre
    if rank == 0:
        print("DCP_INFO " + json.dumps(out) + " " + json.dumps(toks), flush=True)
    assert min(pre) >= 2 and sum(pre) >= 10, toks
    assert out[f"dcp{world}"]["topk_merges"] > 0 and out["dcp1"]["topk_merges"] == 0
    # 9000 + 300 tokens: 36 + 2 pages when one rank holds them all
    pk = torch.tensor([out[f"dcp{world}"]["c4_pages_peak"]], device=dev)
    tot = pk.clone()
    dist.all_reduce(tot)
    assert abs(int(tot.item()) - out["dcp1"]["c4_pages_peak"]) <= 1, (int(tot.item()), out["dcp1"])
    assert int(pk.item()) < out["dcp1"]["c4_pages_peak"]
    if rank == 0:
        print("DCP_OK " + json.dumps(out), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
