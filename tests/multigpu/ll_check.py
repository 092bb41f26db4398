"""Run under torchrun on >= 2 GPUs: the all-reduce folded into producer and consumer kernels, across real ranks.

  * push + reduce on their own against the library's all-reduce (fp32 sums), repeated so that both parities and many
    epochs are used, and timed inside a captured graph against the one-shot all-reduce kernel and NCCL;
  * a row-parallel projection that pushes its partial rows, consumed by the mHC post/pre kernel;
  * the vocabulary-sharded Gumbel arg-max (each rank holds V / world logits) against the arg-max over gathered logits;
  * a small model, tensor + expert parallel over the ranks, decoded through captured graphs with every fusion on,
    against the same engine with separate launches and library collectives.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from stkernel_b200.ops import _lib  # noqa: E402
from stkernel_b200.ops import functional as Fn  # noqa: E402
from stkernel_b200.ops import sampling as S  # noqa: E402
from stkernel_b200.parallel.communicator import Communicator  # noqa: E402

BF16 = torch.bfloat16


def graph_us(fn, iters=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for _ in range(iters):
                fn()
    torch.cuda.current_stream().wait_stream(side)
    best = float("inf")
    for _ in range(5):
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / iters)
    t = torch.tensor([best], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    comm = Communicator(device=dev, use_symm=True)
    assert comm.symm is not None, comm.disabled_reason
    out = {"world": world, "push_reduce": [], "engine": {}}
    g = torch.Generator(device=dev).manual_seed(5 + rank)

    # ---- producer and consumer on their own ----
    for t, h in ((1, 4096), (2, 4096), (4, 4096), (8, 4096), (64, 4096)):
        ex = comm.symm.ll_exchange(t, h)
        assert ex is not None
        worst = 0.0
        for it in range(7):                                   # odd count: both parities, several epochs
            x = torch.randn(t, h, device=dev, generator=g).to(BF16)
            ref = x.float()
            dist.all_reduce(ref)
            y = Fn.ll_reduce(Fn.ll_push(x, ex))
            worst = max(worst, ((y.float() - ref).norm() / ref.norm()).item())
        torch.cuda.synchronize()
        _lib.check_status()
        assert worst < 1e-2, (t, h, worst)
        x = torch.randn(t, h, device=dev, generator=g).to(BF16)
        buf = x.clone()
        row = {"T": t, "H": h, "rel_err": worst,
               "folded_push_plus_reduce_us": graph_us(lambda: Fn.ll_reduce(Fn.ll_push(x, ex))),
               "oneshot_allreduce_us": graph_us(lambda: comm.all_reduce(buf)),
               "nccl_allreduce_us": graph_us(lambda: dist.all_reduce(buf))}
        out["push_reduce"].append(row)

    # ---- projection -> mHC post/pre ----
    hdim, k = 4096, 2048 // world * world
    kl = k // world
    for t in (1, 3, 6):
        gw = torch.Generator(device=dev).manual_seed(11 + rank)
        x = torch.randn(t, kl, device=dev, generator=gw).to(BF16)
        lw = Fn.LinearWeight.from_master(torch.randn(hdim, kl, device=dev, generator=gw) * 0.05, "fp8", dev)
        ex = comm.symm.ll_exchange(t, hdim)
        full = Fn.linear(x, lw).float()
        dist.all_reduce(full)
        got = Fn.ll_reduce(Fn.linear(x, lw, ll=ex))
        e = ((got.float() - full).norm() / full.norm()).item()
        assert e < 1e-2, ("projection", t, e)
        out[f"projection_T{t}_rel_err"] = e

    # ---- vocabulary-sharded arg-max ----
    v = 129280 // world // 8 * 8
    for rows in (1, 4):
        gs = torch.Generator(device=dev).manual_seed(23)           # same on every rank: the full logits
        logits_full = torch.randn(rows, v * world, device=dev, generator=gs).to(BF16)
        shard = logits_full[:, rank * v:(rank + 1) * v].contiguous()
        temp = torch.tensor([0.0, 0.8, 1.0, 0.3][:rows], device=dev)
        seed = torch.arange(rows, device=dev, dtype=torch.int64) + 9
        pos = torch.arange(rows, device=dev, dtype=torch.int64) + 100
        want, _ = S.gumbel_argmax(logits_full, temp, seed, pos)
        agreed = torch.zeros(1, dtype=torch.int32, device=dev)
        ex = comm.symm.ll_exchange(8, 64)
        for _ in range(3):
            got, _ = S.gumbel_argmax(shard, temp, seed, pos, vocab_start=rank * v, ll=ex, agreed_status=agreed)
        torch.cuda.synchronize()
        _lib.check_status()
        assert torch.equal(got.cpu(), want.cpu()), (rows, got.tolist(), want.tolist())
        assert int(agreed.item()) == 0
    out["sharded_argmax"] = "identical to the arg-max over gathered logits"

    # ---- the engine, fused against unfused ----
    from stkernel_b200.config import EngineConfig, ParallelConfig, SchedulerConfig, flash_config
    from stkernel_b200.models.dsv4 import RandomSource, build_model_weights
    from stkernel_b200.runtime.engine import Engine, SamplingParams
    cfg = flash_config(num_layers=3, n_routed_experts=16, vocab_size=4096)
    weights = build_model_weights(cfg, RandomSource(0), dev, rank, world, head_fp8=True)
    assert weights.layers[0].experts_tp is not None          # decode steps use the sliced copy of the experts ...
    os.environ["STK_MOE_DECODE_SLICED"] = "0"
    weights_ep = build_model_weights(cfg, RandomSource(0), dev, rank, world, head_fp8=True)
    del os.environ["STK_MOE_DECODE_SLICED"]
    assert weights_ep.layers[0].experts_tp is None           # ... the comparison engine whole experts per rank
    gp = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gp).tolist() for n in (300, 17)]
    toks = {}
    for mode in ("unfused", "unfused_whole_experts", "fused"):
        os.environ["STK_DECODE_FUSE"] = "1" if mode == "fused" else "0"
        c = comm if mode == "fused" else Communicator(device=dev, use_symm=False)
        ec = EngineConfig(model=cfg, parallel=ParallelConfig(tp_size=world, ep_size=world, fused_collectives=mode == "fused"),
                          sched=SchedulerConfig(max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=256,
                                                graph_cap=4)).validate()
        eng = Engine(ec, weights_ep if mode == "unfused_whole_experts" else weights, dev, c, rank, max_context=1024)
        toks[mode] = eng.generate(prompts, SamplingParams(temperature=1.0, seed=11, max_tokens=12))
        torch.cuda.synchronize()
        _lib.check_status()
        if mode == "fused":
            out["engine"]["folded_allreduce_epochs"] = int(comm.symm.ll.counters[0].item())
            assert out["engine"]["folded_allreduce_epochs"] > 0
        dist.barrier()
    # every rank must hold the same tokens (the ranks sample from the same logits)
    mine = torch.tensor(toks["fused"], device=dev)
    ref0 = mine.clone()
    dist.broadcast(ref0, 0)
    assert torch.equal(mine, ref0), "ranks disagree on the sampled tokens"
    # same weights, fused launches + own collectives against separate launches + library collectives
    def prefix(a, b):
        n = 0
        while n < len(a) and a[n] == b[n]:
            n += 1
        return n
    pre_same = [prefix(x, y) for x, y in zip(toks["fused"], toks["unfused"])]
    out["engine"]["common_prefix_with_unfused"] = pre_same
    assert min(pre_same) >= 2 and sum(pre_same) >= 10, toks
    # sliced experts against whole experts per rank: the NVFP4 scales of a slice differ from those of the whole expert,
    # so a sampled token may flip (and the text after it); the common prefixes must still be long
    pre = [prefix(x, y) for x, y in zip(toks["fused"], toks["unfused_whole_experts"])]
    out["engine"]["common_prefix_with_whole_experts"] = pre
    assert min(pre) >= 2 and sum(pre) >= 10, toks
    if rank == 0:
        print("LL_OK " + json.dumps(out), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
