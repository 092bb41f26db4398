"""Expert-parallel MoE over peer memory: numerics against an fp32 reference and device-timed comparison
with the NCCL all-to-all baseline.  Run with one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        tests/multigpu/ep_check.py [--tokens 1,16,128,1024] [--experts 256]

Prints one `EP_OK {json}` line on rank 0 (or `EP_FAIL ...`).  Every number is max over ranks of a
CUDA-event time around graph-free launches on the launching stream, after warm-up.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from stkernel_b200.ops import _lib                      # noqa: E402
from stkernel_b200.ops import moe as M                  # noqa: E402
from stkernel_b200.ops import reference as R            # noqa: E402
from stkernel_b200.parallel.communicator import Communicator   # noqa: E402
from stkernel_b200.parallel.ep_moe import EpMoE         # noqa: E402


def max_over_ranks(v: float, dev) -> float:
    t = torch.tensor([v], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def timed(fn, iters, dev) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return max_over_ranks(e0.elapsed_time(e1) / iters * 1e3, dev)


def timed_graph(fn, iters, dev) -> float:
    """The peer-memory path has no host round trip, so a whole layer call replays as one CUDA graph."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    dist.barrier()
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return max_over_ranks(e0.elapsed_time(e1) / iters * 1e3, dev)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="1,16,128,1024")
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=6)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--check-tokens", type=int, default=64)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl")
    comm = Communicator(device=dev, use_symm=False)
    E, k, H, I = a.experts, a.topk, a.hidden, a.inter
    el = E // world
    token_list = [int(x) for x in a.tokens.split(",")]
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    # local experts: NVFP4 from N(0, 0.02) masters (every rank draws its own experts from a rank-keyed seed)
    gw = torch.Generator(device=dev).manual_seed(99 + rank)
    w13 = torch.randn(el, 2 * I, H, generator=gw, device=dev) * 0.02
    w2 = torch.randn(el, H, I, generator=gw, device=dev) * 0.02
    ew = M.ExpertWeights.from_master(w13, w2, "nvfp4", dev, expert_start=rank * el)
    del w13, w2
    ep = EpMoE(comm, E, k, H, I, max(token_list + [a.check_tokens]))
    res = {"world": world, "experts": E, "rows": []}

    def make(t):
        x = torch.randn(t, H, generator=g).to(dev).to(torch.bfloat16)
        logits = torch.randn(t, E, generator=g).to(dev)
        bias = (torch.rand(E, generator=torch.Generator().manual_seed(5)) * 0.2 - 0.1).to(dev)
        ids, wts = M.router(logits, bias, k, "sigmoid", True, 1.0, None, None)
        return x, ids.contiguous(), wts.contiguous()

    # ---- numerics: gather everything, compute this rank's tokens with the dequantised weights of all ranks ----
    t = a.check_tokens
    x, ids, wts = make(t)
    shared = torch.randn(t, H, generator=g).to(dev).to(torch.bfloat16)
    out = ep.forward(x, ids, wts, ew, shared)
    torch.cuda.synchronize()
    _lib.check_status()
    out_nccl = ep.forward_nccl(x, ids, wts, ew, shared)
    if E <= 64:
        # full fp32 reference with the dequantised weights of every rank
        d13, d2 = ew.dequant()
        all13 = [torch.empty_like(d13) for _ in range(world)]
        all2 = [torch.empty_like(d2) for _ in range(world)]
        dist.all_gather(all13, d13.contiguous())
        dist.all_gather(all2, d2.contiguous())
        W13, W2 = torch.cat(all13), torch.cat(all2)
        ref = shared.float().clone()
        xf = x.to(torch.float16).float()
        for ti in range(t):
            for j in range(k):
                e = int(ids[ti, j])
                gu = W13[e] @ xf[ti]
                act = R.swiglu_clamp(gu[:I], gu[I:], 10.0).to(torch.float16).float()
                ref[ti] += float(wts[ti, j]) * (W2[e] @ act).to(torch.bfloat16).float()
        del W13, W2, all13, all2, d13, d2
        res["reference"] = "fp32 matmul over dequantised weights"
    else:
        ref = out_nccl.float()
        res["reference"] = "NCCL all-to-all path (same GEMM kernels); run with --experts 32 for the fp32 reference"
    err = ((out.float() - ref).norm() / ref.norm()).item()
    err_nccl = ((out_nccl.float() - ref).norm() / ref.norm()).item()
    res["rel_err"] = max_over_ranks(err, dev)
    res["rel_err_nccl_path"] = max_over_ranks(err_nccl, dev)
    # a second call with different routing must not see stale counters
    x2, ids2, wts2 = make(t)
    o2 = ep.forward(x2, ids2, wts2, ew, None)
    o2n = ep.forward_nccl(x2, ids2, wts2, ew, None)
    torch.cuda.synchronize()
    _lib.check_status()
    res["second_call_vs_nccl_path"] = max_over_ranks(((o2.float() - o2n.float()).norm() / o2n.float().norm()).item(), dev)

    # ---- timing ----
    for t in token_list:
        x, ids, wts = make(t)
        iters = 20 if t <= 1024 else 5
        ours = timed(lambda: ep.forward(x, ids, wts, ew, None), iters, dev)
        ours_graph = timed_graph(lambda: ep.forward(x, ids, wts, ew, None), iters, dev)
        base = timed(lambda: ep.forward_nccl(x, ids, wts, ew, None), iters, dev)
        _lib.check_status()
        flops = 2.0 * t * world * k * (2 * I * H + H * I) / world          # per rank on average
        nvl_bytes = t * k * H * (2 + 2) * (world - 1) / world               # fp16 out + bf16 back, off-rank share
        res["rows"].append({"tokens_per_gpu": t, "peer_us": ours, "peer_graph_us": ours_graph, "nccl_us": base,
                            "speedup": base / ours_graph, "gemm_tflops_per_gpu": flops / ours_graph / 1e6,
                            "nvlink_gbs_per_gpu": nvl_bytes / ours_graph / 1e3})
    ok = res["rel_err"] < 2e-2 and res["second_call_vs_nccl_path"] < 1e-2
    if rank == 0:
        print(("EP_OK " if ok else "EP_FAIL ") + json.dumps(res), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
