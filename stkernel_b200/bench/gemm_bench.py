"""Dense GEMM microbenchmark: achieved bytes/s (skinny) and FLOP/s (wide) of the tcgen05 kernel
against torch.matmul (cuBLAS), timed as CUDA-graph replays with operands larger than L2 rotated
between calls.

    python -m stkernel_b200.bench.gemm_bench [--out FILE] [--shapes 4096x4096x8192] [--dtypes bf16] [--no-cublas]
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import functional as Fn

PEAKS = {"hbm_gbs": 6549.1, "bf16_tflops": 1613.6}


def load_peaks() -> dict:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}


def graph_time(fns, iters: int = 10) -> float:
    """us per call; `fns` is a list of equivalent closures over distinct operands (rotated so that
    consecutive calls do not find their weights in L2)."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fns[i % len(fns)]()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--shapes", default="", help="TxNxK[,TxNxK...] instead of the default list")
    ap.add_argument("--dtypes", default="bf16,fp8")
    ap.add_argument("--no-cublas", action="store_true", help="time only this library's kernel (profiler captures)")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    peaks = load_peaks()
    rows = []
    shapes = [(1, 2048, 4096), (1, 40960, 1536), (1, 4096, 8192), (8, 4096, 8192), (64, 4096, 8192), (64, 40960, 1536),
              (256, 4096, 8192), (4096, 4096, 8192), (4096, 8192, 8192), (8192, 8192, 8192)]
    if a.shapes:
        shapes = [tuple(int(v) for v in sh.split("x")) for sh in a.shapes.split(",")]
    for dtype in a.dtypes.split(","):
        for (T, N, K) in shapes:
            wbytes = N * K * (1 if dtype == "fp8" else 2)
            copies = max(2, min(8, (256 << 20) // wbytes + 1))
            ws = [Fn.LinearWeight.from_master(torch.randn(N, K, device=dev) * 0.05, dtype, dev) for _ in range(copies)]
            x = torch.randn(T, K, device=dev).to(torch.bfloat16)
            xq = Fn.quant_act(x, "bench") if dtype == "fp8" else x
            outs = [torch.empty(T, N, dtype=torch.bfloat16, device=dev) for _ in range(copies)]
            ours = graph_time([lambda w=w, o=o: Fn.linear(xq, w, out=o) for w, o in zip(ws, outs)])
            if dtype == "bf16" and not a.no_cublas:
                base = graph_time([lambda w=w, o=o: torch.matmul(x, w.w.t(), out=o) for w, o in zip(ws, outs)])
            else:
                base = None
            flops = 2.0 * T * N * K
            byts = wbytes + T * K * (1 if dtype == "fp8" else 2) + T * N * 2
            peak_t = max(flops / (peaks["bf16_tflops"] * (2 if dtype == "fp8" else 1) * 1e12), byts / (peaks["hbm_gbs"] * 1e9)) * 1e6
            rows.append({"dtype": dtype, "T": T, "N": N, "K": K, "ours_us": round(ours, 2),
                         "cublas_us": round(base, 2) if base else None, "tflops": round(flops / ours / 1e6, 1),
                         "gbs": round(byts / ours / 1e3, 1), "roofline_us": round(peak_t, 2),
                         "frac_of_roofline": round(peak_t / ours, 3)})
            print(rows[-1], flush=True)
            del ws, outs
            torch.cuda.empty_cache()
    if a.out:
        with open(a.out, "w") as f:
            f.write(f"# tcgen05 GEMM vs cuBLAS, CUDA-graph timed, peaks ({peaks['src']}): {peaks}\n")
            f.write("# fp8 roofline uses 2x the measured bf16 GEMM peak as its compute bound\n")
            for r in rows:
                f.write(json.dumps(r) + "\n")


if __name__ == "__main__":
    main()
