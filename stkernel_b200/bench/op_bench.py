"""Single-op micro-benchmarks of the decode chain (device-timed with CUDA events, weights rotated through more
than the 126 MB L2 so that every call streams its operands from HBM as it does inside a step).

    python -m stkernel_b200.bench.op_bench --op mhc_fused --T 1
    python -m stkernel_b200.bench.op_bench --op mhc --T 1 --iters 3 --sets 3      # a small case for a profiler
    python -m stkernel_b200.bench.op_bench --op indexer_tc --T 4096 --H 8192 --iters 20   # --H = compressed rows
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import functional as Fn

BF16 = torch.bfloat16


def _mhc_sets(n_sets: int, h: int, hc: int, dev):
    out = []
    for i in range(n_sets):
        g = torch.Generator(device=dev).manual_seed(i)
        fn = torch.randn(24, hc * h, device=dev, generator=g) * 0.02
        base = torch.randn(24, device=dev, generator=g) * 0.1
        scale = torch.tensor([1.0, 0.7, 1.3], device=dev)
        nw = (1 + 0.1 * torch.randn(h, device=dev, generator=g)).to(BF16)
        out.append((fn, base, scale, nw))
    return out


def run_indexer(t: int, rows: int, iters: int, tensor_core: bool) -> dict:
    """Prefill-shaped indexer scoring: t consecutive tokens of one request whose last token sees `rows` compressed rows
    (ratio 4), 64 heads x 128 dims fp8, against the paged fp8 indexer cache."""
    from ..ops import attention as A
    from ..ops import cache as C
    dev = torch.device("cuda:0")
    ih, d = 64, 128
    n_pages = (rows + 63) // 64 + 1
    cache = C.PagedCache.allocate(n_pages, d, 64, True, "indexer", dev)
    cache.buf[:, :64 * d] = torch.randint(0, 120, (n_pages, 64 * d), dtype=torch.uint8, device=dev)
    cache.buf[:, 64 * d:64 * d + 256] = torch.full((n_pages, 64), 0.01, device=dev).view(torch.uint8).view(n_pages, 256)
    bt = torch.arange(n_pages, dtype=torch.int32, device=dev)[None].contiguous()
    q = torch.randn(t, ih, d, device=dev).to(BF16)
    w = torch.rand(t, ih, device=dev)
    pos = (torch.arange(t, device=dev) + (rows * 4 - t)).clamp_(min=0)
    inv = Fn.inv_freq(64, 10000.0, dev)
    qq, wf = C.indexer_q_prep(q, w, pos, inv, 64, True)
    tok_req = torch.zeros(t, dtype=torch.int32, device=dev)
    nv = A.compressed_valid(pos, 4)
    A.USE_TENSOR_CORE_INDEXER = tensor_core
    for _ in range(3):
        A.indexer_scores(qq, wf, cache, bt, tok_req, nv, rows)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        A.indexer_scores(qq, wf, cache, bt, tok_req, nv, rows)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    pairs = float(nv.sum())
    flops = pairs * ih * d * 2
    return {"op": "indexer_tc" if tensor_core else "indexer_cuda_core", "T": t, "rows": rows, "iters": iters,
            "us_per_call": us, "token_row_pairs": pairs, "tflops": flops / us * 1e-6}


def run(op: str, t: int, h: int, iters: int, n_sets: int, graph: bool = True) -> dict:
    if op in ("indexer_tc", "indexer_cc"):
        return run_indexer(t, h, iters, op == "indexer_tc")
    dev = torch.device("cuda:0")
    hc = 4
    sets = _mhc_sets(n_sets, h, hc, dev)
    res = torch.randn(t, hc, h, device=dev).to(BF16)
    x = torch.randn(t, h, device=dev).to(BF16)
    post = torch.rand(t, hc, device=dev)
    comb = torch.softmax(torch.randn(t, hc, hc, device=dev), -1).reshape(t, hc * hc).contiguous()

    def call(i):
        w = sets[i % n_sets]
        if op == "mhc":
            return Fn.mhc_pre(res, *w, 1e-6, 1e-6, 20)
        if op == "mhc_fused":
            return Fn.mhc_post_pre(x, res, post, comb, *w, 1e-6, 1e-6, 20)
        if op == "mhc_unfused":
            nr = Fn.mhc_post(x, res, post, comb)
            return Fn.mhc_pre(nr, *w, 1e-6, 1e-6, 20)
        raise SystemExit(f"unknown op {op}")

    for i in range(3):
        call(i)
    torch.cuda.synchronize()
    if not graph:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            call(i)
        e1.record()
        torch.cuda.synchronize()
        return {"op": op, "T": t, "H": h, "iters": iters, "weight_sets": n_sets, "graph": False,
                "us_per_call": e0.elapsed_time(e1) * 1e3 / iters}
    # a CUDA graph of `iters` calls: launch gaps as inside a captured step, not host-bound
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for i in range(iters):
                call(i)
    torch.cuda.current_stream().wait_stream(side)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return {"op": op, "T": t, "H": h, "iters": iters, "weight_sets": n_sets, "us_per_call": e0.elapsed_time(e1) * 1e3 / iters}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="mhc_fused")
    ap.add_argument("--T", type=int, default=1)
    ap.add_argument("--H", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--sets", type=int, default=100)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--impl", default="ours", help="'reference': time the reference's own shipped Triton kernels against "
                                                   "this library's kernels for the same ops (see bench/ref_ops.py)")
    a, rest = ap.parse_known_args()
    if a.impl == "reference":
        from .ref_ops import main as ref_main
        raise SystemExit(ref_main(rest))
    print(json.dumps(run(a.op, a.T, a.H, a.iters, a.sets, not a.no_graph)))


if __name__ == "__main__":
    main()
