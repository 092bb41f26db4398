"""Small-shape checks of the hot kernels against the fp32 PyTorch statements in :mod:`..ops.reference`.

`kernel_self_check()` is what a deployment runs right after the library loads (and what the driver's smoke
hook runs first): every input is drawn on the host and copied over, so the first device launches of the
process are this library's own kernels, and every result is compared on the host.  Returns
{check name: relative error}; raises `AssertionError` on a mismatch.
"""
from __future__ import annotations

from typing import Dict

import torch

BF16, F32 = torch.bfloat16, torch.float32


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / b.norm().clamp(min=1e-12)).item()


def kernel_self_check(device="cuda:0") -> Dict[str, float]:
    from ..ops import attention as A
    from ..ops import cache as C
    from ..ops import functional as Fn
    from ..ops import moe as M
    from ..ops import reference as R
    from ..ops import _lib

    dev = torch.device(device)
    g = torch.Generator().manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=g)
    res: Dict[str, float] = {}

    # dense GEMM, bf16 (tcgen05) at 64 tokens and the weight-streaming kernel at 1 token
    x, w = rn(64, 1024).to(BF16), rn(512, 1024).to(BF16)
    ref = x.float() @ w.float().t()
    lw = Fn.LinearWeight(w.to(dev))
    res["gemm_bf16_t64"] = _rel(Fn.linear(x.to(dev), lw), ref)
    res["skinny_bf16_t1"] = _rel(Fn.linear(x[:1].to(dev), lw), ref[:1])

    # fp8 128x128 block-scaled GEMM against the dequantised product
    wq, ws = R.quant_fp8_block128_weight(rn(512, 1024) * 0.05)
    lw8 = Fn.LinearWeight(wq.to(dev).contiguous(), ws.to(dev).contiguous())
    xq, xs = R.quant_fp8_group128_act(x)
    ref8 = R.dequant_fp8_group128_act(xq, xs) @ R.dequant_fp8_block128_weight(wq, ws).t()
    res["gemm_fp8_t64"] = _rel(Fn.linear(x.to(dev), lw8, out_dtype=F32), ref8)

    # mHC pre-mix (Sinkhorn) + post-mix, one token
    hc, H = 4, 4096
    r0 = rn(1, hc, H).to(BF16)
    fn, base, scale = rn(24, hc * H) * 0.02, rn(24) * 0.1, torch.tensor([1.0, 0.7, 1.3])
    nw = (1 + 0.1 * rn(H)).to(BF16)
    y, post, comb = Fn.mhc_pre(r0.to(dev), fn.to(dev), base.to(dev), scale.to(dev), nw.to(dev), 1e-6, 1e-6, 20)
    yr, pr, cr = R.mhc_pre(r0, fn, base, scale, nw, 1e-6, 1e-6, 20, round_bf16=True)
    res["mhc_pre_y"] = _rel(y, yr)
    res["mhc_pre_comb"] = _rel(comb.view(1, hc, hc), cr)
    xo = rn(1, H).to(BF16)
    res["mhc_post"] = _rel(Fn.mhc_post(xo.to(dev), r0.to(dev), post, comb), R.mhc_post(xo, r0, pr, cr))

    # sparse MLA over paged fp8_ds_mla rows: 8 heads, window + top-k rows, sink logit
    D, Rd, T, W, K, pages = 512, 64, 2, 128, 256, 12
    ccpu = C.PagedCache.allocate(pages, D, Rd, True, "latent", "cpu")
    ccpu.write_rows_cpu(torch.arange(pages * 64), rn(pages * 64, D))
    cg = C.PagedCache(ccpu.buf.to(dev), D, Rd, True, "latent")
    q = rn(T, 8, D).to(BF16)
    swa = torch.randint(0, pages * 64, (T, W), dtype=torch.int32, generator=g)
    swa_l = torch.tensor([W, 9], dtype=torch.int32)
    tk = torch.randint(0, pages * 64, (T, K), dtype=torch.int32, generator=g)
    tk_l = torch.tensor([K, 31], dtype=torch.int32)
    sink = rn(8)
    o = A.sparse_mla(q.to(dev), cg, swa.to(dev), swa_l.to(dev), cg, tk.to(dev), tk_l.to(dev), sink.to(dev), D ** -0.5)
    oref = A.sparse_mla(q, ccpu, swa, swa_l, ccpu, tk, tk_l, sink, D ** -0.5)
    res["sparse_mla"] = _rel(o, oref)

    # routed experts (NVFP4 weights) behind the router, 3 tokens
    E, I, Hm, k = 8, 256, 512, 2
    ec = M.ExpertWeights.from_master(rn(E, 2 * I, Hm) * 0.02, rn(E, Hm, I) * 0.02, "nvfp4", "cpu")
    ew = M.ExpertWeights(*[t.to(dev) for t in (ec.w13, ec.w2, ec.s13, ec.s2, ec.g13, ec.g2)], 0)
    xm = rn(3, Hm).to(BF16)
    ids, wts = M.router(rn(3, E).to(dev), None, k, "sigmoid", True, 1.0)
    om = M.moe_experts(xm.to(dev), ids, wts, ew, 10.0, None)
    d13, d2 = ec.dequant()
    res["moe_nvfp4"] = _rel(om, R.moe_experts(xm, ids.cpu(), wts.cpu(), d13, d2, 10.0))

    torch.cuda.synchronize(dev)
    _lib.check_status()
    limits = {"gemm_bf16_t64": 1e-2, "skinny_bf16_t1": 1e-2, "gemm_fp8_t64": 6e-3, "mhc_pre_y": 5e-3, "mhc_pre_comb": 2e-3,
              "mhc_post": 5e-3, "sparse_mla": 1e-2, "moe_nvfp4": 1.5e-2}
    bad = {n: e for n, e in res.items() if not e <= limits[n]}
    assert not bad, f"kernel self-check failed: {bad}"
    return res
