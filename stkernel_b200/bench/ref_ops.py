"""Per-op comparison against the reference's own shipped kernels on the same GPU.

The reference cannot be installed or served here (it is a set of overlay files for a closed engine image), but four
of its hot ops are self-contained Triton kernels in those files.  This tool runs them **unmodified**: the function
definitions are cut out of the reference's source text by name (the way its own test loads overlay code,
tests/test_logic.py:24-46), written to a scratch module whose only additions are the three imports the overlay takes
from its engine (`torch`, `triton`, `triton.language as tl` standing in for `vllm.triton_utils`), and launched through
the reference's own wrapper code with the same shapes as this library's kernel for the op:

    router gate      overlay/nvidia_model.py:595-667      vs  stk_skinny_linear (+ the router epilogue)
    KV quant+insert  overlay/ops_cache_utils.py:29-218    vs  stk_q_rope_kv_insert (latent-row half)
    indexer-Q        overlay/ops_fused_indexer_q.py:70-172,285-452  vs  stk_indexer_q_prep
    SWA index lists  overlay/sparse_swa_dsv4.py:748-804   vs  stk_swa_indices

    python -m stkernel_b200.bench.ref_ops [--reference DIR] [--tokens 1,6,32,64] [--out FILE]

Both sides are timed the same way: a CUDA graph of `iters` calls, CUDA events around one replay, best of 5.
The reference tree is looked for in --reference, $STK_REFERENCE_DIR and baseline/_ref.
"""
from __future__ import annotations

import argparse
import ast
import importlib.util
import json
import os
import sys
import tempfile
from pathlib import Path
from typing import Callable, Dict, List, Optional

import torch

ROOT = Path(__file__).resolve().parents[2]


def find_reference(explicit: str = "") -> Optional[Path]:
    for cand in (explicit, os.environ.get("STK_REFERENCE_DIR", ""), str(ROOT / "baseline" / "_ref")):
        if cand and (Path(cand) / "overlay" / "ops_cache_utils.py").is_file():
            return Path(cand)
    return None


_HEADER = ("import os\nimport torch\nimport triton\nimport triton.language as tl\n"
           "class _Platform:\n    @staticmethod\n    def is_fp8_fnuz():\n        return False\n"
           "current_platform = _Platform()\nHAS_CUTEDSL = False\n")


def load_defs(ref: Path, relpath: str, names: List[str], tag: str):
    """Module holding the named top-level (or nested-in-`if`) functions and assignments of a reference file, verbatim."""
    src = (ref / relpath).read_text()
    tree = ast.parse(src)
    found: Dict[str, str] = {}
    for node in ast.walk(tree):
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)) and node.name in names and node.name not in found:
            start = min([node.lineno] + [d.lineno for d in node.decorator_list]) - 1
            lines = src.splitlines()[start:node.end_lineno]
            indent = len(lines[0]) - len(lines[0].lstrip())
            found[node.name] = "\n".join(l[indent:] if len(l) >= indent else l for l in lines)
        elif isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name) \
                and node.targets[0].id in names and node.targets[0].id not in found:
            found[node.targets[0].id] = ast.get_source_segment(src, node)
    missing = [n for n in names if n not in found]
    if missing:
        raise RuntimeError(f"{relpath}: not found in the reference: {missing}")
    body = _HEADER + "\n\n".join(found[n] for n in names) + "\n"
    d = Path(tempfile.gettempdir()) / "stk_ref_ops"
    d.mkdir(exist_ok=True)
    path = d / f"ref_{tag}.py"
    path.write_text(body)
    spec = importlib.util.spec_from_file_location(f"stk_ref_{tag}", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def time_graph(fn: Callable[[], None], iters: int = 20) -> float:
    """us per call: a CUDA graph of `iters` calls, best of 5 replays."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
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
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3 / iters)
    return best


def bench_gate(ref: Path, t: int) -> Dict:
    from ..ops import functional as Fn
    dev = torch.device("cuda:0")
    m = load_defs(ref, "overlay/nvidia_model.py",
                  ["_GATE_FUSED_SPLIT_K", "_GATE_FUSED_BLOCK_N", "_GATE_FUSED_BLOCK_K", "_deneb_gate_partial_kernel",
                   "_deneb_fused_gate"], "gate")
    if t > 32:
        return {"op": "router_gate_logits", "tokens": t, "skipped": "the reference kernel serves at most 32 tokens"}
    x = torch.randn(t, 4096, device=dev).to(torch.bfloat16)
    w = (torch.randn(256, 4096, device=dev) * 0.02).to(torch.bfloat16)
    lw = Fn.LinearWeight(w)
    ref_out = m._deneb_fused_gate(x, w)
    ours = Fn.linear(x, lw, out_dtype=torch.float32)
    err = ((ours - ref_out).norm() / ref_out.norm()).item()
    r_us = time_graph(lambda: m._deneb_fused_gate(x, w))
    o_us = time_graph(lambda: Fn.linear(x, lw, out_dtype=torch.float32))
    out = {"op": "router_gate_logits", "tokens": t, "reference_us": r_us, "ours_us": o_us, "rel_diff": err}
    if t <= Fn.SKINNY_MAX_T:
        bias = torch.zeros(256, device=dev)
        out["ours_with_top6_routing_us"] = time_graph(lambda: Fn.gate_route(x, lw, bias, 6, "sigmoid", True, 1.0))
    return out


def bench_kv_insert(ref: Path, t: int) -> Dict:
    from ..ops import cache as C
    from ..ops import functional as Fn
    dev = torch.device("cuda:0")
    m = load_defs(ref, "overlay/ops_cache_utils.py", ["quantize_and_insert_k_kernel", "quantize_and_insert_k_cache"], "kv")
    pages = max(4, (t + 63) // 64 + 1)
    k = torch.randn(t, 512, device=dev).to(torch.bfloat16)
    slots = torch.randperm(pages * 64, device=dev)[:t].to(torch.int64)
    ours_cache = C.PagedCache.allocate(pages, 512, 64, True, "latent", dev)
    ref_cache = torch.zeros_like(ours_cache.buf)
    pos = torch.zeros(t, dtype=torch.int64, device=dev)          # position 0: RoPE is the identity, as in the reference op
    inv = Fn.inv_freq(64, 10000.0, dev)
    m.quantize_and_insert_k_cache(k, ref_cache, slots, block_size=64)
    C.kv_rope_quant_insert(k, pos, slots, inv, ours_cache)
    torch.cuda.synchronize()
    same = float((ref_cache == ours_cache.buf).float().mean())
    r_us = time_graph(lambda: m.quantize_and_insert_k_cache(k, ref_cache, slots, block_size=64))
    o_us = time_graph(lambda: C.kv_rope_quant_insert(k, pos, slots, inv, ours_cache))
    return {"op": "kv_quantize_insert", "tokens": t, "reference_us": r_us, "ours_us": o_us, "identical_bytes": same,
            "note": "ours also applies RoPE to the 64 rope dims (identity at position 0)"}


def bench_indexer_q(ref: Path, t: int) -> Dict:
    from ..ops import cache as C
    from ..ops import functional as Fn
    dev = torch.device("cuda:0")
    m = load_defs(ref, "overlay/ops_fused_indexer_q.py",
                  ["MXFP4_BLOCK_SIZE", "_get_cos_sin", "_fp32x2_to_fp4x2", "_quantize_mxfp4_pair",
                   "_fused_indexer_q_rope_quant_kernel", "_fused_indexer_q_rope_mxfp4_kernel",
                   "fused_indexer_q_rope_quant"], "idxq")
    ih, d, rd = 64, 128, 64
    q = torch.randn(t, ih, d, device=dev).to(torch.bfloat16)
    w = torch.rand(t, ih, device=dev)
    pos = torch.randint(0, 30000, (t,), device=dev, dtype=torch.int64)
    inv = Fn.inv_freq(rd, 10000.0, dev)
    ang = torch.arange(32768, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
    cos_sin = torch.cat([torch.cos(ang), torch.sin(ang)], -1).contiguous()
    sm_scale, head_scale = d ** -0.5, ih ** -0.5
    r_us = time_graph(lambda: m.fused_indexer_q_rope_quant(pos, q, cos_sin, w, sm_scale, head_scale))
    o_us = time_graph(lambda: C.indexer_q_prep(q, w, pos, inv, rd, True))
    return {"op": "indexer_q_rope_quant", "tokens": t, "reference_us": r_us, "ours_us": o_us}


def bench_swa_indices(ref: Path, t: int) -> Dict:
    from ..ops import attention as A
    dev = torch.device("cuda:0")
    m = load_defs(ref, "overlay/sparse_swa_dsv4.py", ["_compute_swa_indices_and_lens_kernel"], "swa")
    window, ctx, page = 128, 32768, 64
    n_pages = ctx // page + 2
    bt = torch.arange(t * n_pages, dtype=torch.int32, device=dev).view(t, n_pages)
    # t decode requests of one token each at position ctx - 1
    qsl = torch.arange(t + 1, dtype=torch.int32, device=dev)
    seq_lens = torch.full((t,), ctx, dtype=torch.int32, device=dev)
    tok_req = torch.arange(t, dtype=torch.int32, device=dev)
    valid = torch.ones(t, dtype=torch.bool, device=dev)
    out_idx = torch.empty(t, window, dtype=torch.int32, device=dev)
    out_len = torch.empty(t, dtype=torch.int32, device=dev)
    positions = torch.full((t,), ctx - 1, dtype=torch.int64, device=dev)

    def ref_call():
        m._compute_swa_indices_and_lens_kernel[(t,)](out_idx, out_idx.stride(0), out_len, window, qsl, seq_lens, tok_req,
                                                     valid, bt, bt.stride(0), page, token_offset=0, TRITON_BLOCK_SIZE=1024)

    ref_call()
    ours_idx, ours_len = A.swa_indices(positions, tok_req, bt, window)
    torch.cuda.synchronize()
    same = bool(torch.equal(out_idx, ours_idx[:, :window]) and torch.equal(out_len, ours_len))
    r_us = time_graph(ref_call)
    o_us = time_graph(lambda: A.swa_indices(positions, tok_req, bt, window))
    return {"op": "swa_index_lists", "tokens": t, "reference_us": r_us, "ours_us": o_us, "identical": same}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="")
    ap.add_argument("--tokens", default="1,6,32,64")
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    ref = find_reference(a.reference)
    if ref is None:
        print(json.dumps({"impl": "reference", "unavailable": "reference overlay sources not found (looked in --reference, "
                                                              "$STK_REFERENCE_DIR, baseline/_ref)"}))
        return 0
    rows = []
    for t in [int(x) for x in a.tokens.split(",")]:
        for fn in (bench_gate, bench_kv_insert, bench_indexer_q, bench_swa_indices):
            try:
                r = fn(ref, t)
                if "reference_us" in r:
                    r["speedup_vs_reference"] = r["reference_us"] / r["ours_us"]
            except Exception as e:                     # a kernel of the reference that does not build here is reported, not hidden
                r = {"op": fn.__name__[6:], "tokens": t, "error": f"{type(e).__name__}: {e}"[-400:]}
            rows.append(r)
            print(json.dumps(r), flush=True)
    if a.out:
        with open(a.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
