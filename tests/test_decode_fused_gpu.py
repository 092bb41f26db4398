"""The launches that the decode chain folds into their neighbours, each against the unfused sequence of the same ops:
RMSNorm inside the weight-streaming projection, kv norm inside the cache insert, the router inside the gate projection,
and the all-reduce folded into its producer (projection / MoE combine) and consumer (mHC pre-mix) -- the latter on one
GPU as a one-rank exchange, which runs the same stores, epochs, parities and polls with nothing to add."""
import pytest
import torch

from stkernel_b200.ops import _lib
from stkernel_b200.ops import cache as C
from stkernel_b200.ops import functional as Fn
from stkernel_b200.ops import moe as M
from stkernel_b200.ops import reference as R

pytestmark = pytest.mark.gpu
BF16, F32 = torch.bfloat16, torch.float32


def dev():
    return torch.device("cuda:0")


def rel_err(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / b.norm().clamp(min=1e-12)).item()


def _exchange(words=64 * 2048):
    from stkernel_b200.parallel.symm import LLExchange
    return LLExchange.loopback(dev(), words)


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
@pytest.mark.parametrize("T", [1, 3, 4])
def test_projection_with_rmsnorm_prologue(dtype, T):
    torch.manual_seed(T)
    K, N = 1536, 4096 + 512
    buf = torch.randn(T, K + 512, device=dev()).to(BF16) * 3.0            # a strided view, as the model passes it
    x = buf[:, :K]
    nw = (1 + 0.1 * torch.randn(K, device=dev())).to(BF16)
    lw = Fn.LinearWeight.from_master(torch.randn(N, K, device=dev()) * 0.05, dtype, dev())
    ref = Fn.linear(Fn.rms_norm(x.contiguous(), nw, 1e-6), lw)
    out = Fn.linear(x, lw, norm=(nw, 1e-6))
    assert rel_err(out, ref) < 4e-3
    exact = R.rms_norm(x, nw, 1e-6).to(BF16).float() @ lw.dequant().t()
    assert rel_err(out, exact) < 1e-2


def test_kv_norm_inside_the_cache_insert():
    torch.manual_seed(2)
    T, D, Rd, nh = 3, 512, 64, 8
    inv = Fn.inv_freq(Rd, 10000.0, dev())
    pos = torch.tensor([5, 77, 1234], dtype=torch.int64, device=dev())
    slots = torch.tensor([3, 64 + 9, 130], dtype=torch.int64, device=dev())
    kv = torch.randn(T, D, device=dev()).to(BF16) * 2.0
    w = (1 + 0.1 * torch.randn(D, device=dev())).to(BF16)
    q = torch.randn(T, nh, D, device=dev()).to(BF16)
    c_ref = C.PagedCache.allocate(4, D, Rd, True, "latent", dev())
    c_new = C.PagedCache.allocate(4, D, Rd, True, "latent", dev())
    q_ref = C.q_rope_kv_insert(q.clone(), Fn.rms_norm(kv, w, 1e-6), pos, slots, inv, c_ref, 1e-6)
    q_new = C.q_rope_kv_insert(q.clone(), kv, pos, slots, inv, c_new, 1e-6, kv_norm_w=w)
    assert torch.equal(q_ref, q_new)
    assert torch.equal(c_ref.buf, c_new.buf)
    c_only = C.PagedCache.allocate(4, D, Rd, True, "latent", dev())
    assert C.q_rope_kv_insert(None, kv, pos, slots, inv, c_only, 1e-6, kv_norm_w=w) is None
    assert torch.equal(c_only.buf, c_ref.buf)


@pytest.mark.parametrize("scoring", ["sigmoid", "sqrtsoftplus"])
@pytest.mark.parametrize("T", [1, 4])
@pytest.mark.parametrize("path", ["cluster", "grid"])
def test_router_inside_the_gate_projection(scoring, T, path, monkeypatch):
    """`cluster`: one 16-CTA cluster, logits meet in distributed shared memory; `grid`: K split over independent CTAs,
    the last one to finish routes."""
    monkeypatch.setattr(Fn, "GATE_CLUSTER", path == "cluster")
    if path == "cluster":
        assert Fn._gate_cluster_ok(), "a 16-CTA cluster of the gate kernel must be launchable on this GPU"
    torch.manual_seed(7 + T)
    H, E, k = 4096, 256, 6
    x = torch.randn(T, H, device=dev()).to(BF16)
    wg = Fn.LinearWeight((torch.randn(E, H, device=dev()) * 0.02).to(BF16))
    bias = torch.rand(E, device=dev()) * 0.2 - 0.1
    for rep in range(3):            # the arrival counter must come back to zero
        got = Fn.gate_route(x, wg, bias, k, scoring, True, 2.5)
        assert got is not None
        ids, wts = got
        logits = Fn.linear(x, wg, out_dtype=F32)
        rid, rw = M.router(logits, bias, k, scoring, True, 2.5)
        assert torch.equal(ids, rid) and torch.allclose(wts, rw, rtol=1e-4, atol=1e-6)
    # hash routing
    tid2eid = torch.randint(0, E, (1000, k), dtype=torch.int32, device=dev())
    toks = torch.randint(0, 1000, (T,), dtype=torch.int64, device=dev())
    ids, wts = Fn.gate_route(x, wg, None, k, scoring, True, 1.0, tid2eid, toks)
    rid, rw = M.router(Fn.linear(x, wg, out_dtype=F32), None, k, scoring, True, 1.0, tid2eid, toks)
    assert torch.equal(ids, rid) and torch.allclose(wts, rw, rtol=1e-5, atol=1e-6)
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("T", [6, 8])
def test_fused_launches_at_verify_batch_sizes(T, monkeypatch):
    """Speculative verification runs 6 rows per request: with the weight-streaming limit raised to 8 tokens the norm
    prologue, the folded all-reduce push and the cluster gate serve those steps too."""
    monkeypatch.setattr(Fn, "SKINNY_MAX_T", 8)
    ex = _exchange()
    torch.manual_seed(50 + T)
    K, N = 1536, 4096
    x = torch.randn(T, K, device=dev()).to(BF16) * 2.0
    nw = (1 + 0.1 * torch.randn(K, device=dev())).to(BF16)
    for dtype in ("bf16", "fp8"):
        lw = Fn.LinearWeight.from_master(torch.randn(N, K, device=dev()) * 0.05, dtype, dev())
        xn = R.rms_norm(x, nw, 1e-6).to(BF16)
        if dtype == "fp8":            # above four tokens the activations are quantised per 128 values, as in the GEMM path
            xn = R.dequant_fp8_group128_act(*R.quant_fp8_group128_act(xn))
        exact = xn.float() @ lw.dequant().t()
        for rep in range(3):
            p = Fn.linear(x, lw, norm=(nw, 1e-6), ll=ex)
            assert isinstance(p, Fn.LLPending)
            got = Fn.ll_reduce(p)
        assert rel_err(got, exact) < 1e-2
    H, E, k = 4096, 256, 6
    xg = torch.randn(T, H, device=dev()).to(BF16)
    wg = Fn.LinearWeight((torch.randn(E, H, device=dev()) * 0.02).to(BF16))
    bias = torch.rand(E, device=dev()) * 0.2 - 0.1
    ids, wts = Fn.gate_route(xg, wg, bias, k, "sqrtsoftplus", True, 2.5)
    rid, rw = M.router(xg.float() @ wg.w.float().t(), bias, k, "sqrtsoftplus", True, 2.5)
    assert torch.equal(ids, rid) and torch.allclose(wts, rw, rtol=1e-4, atol=1e-6)
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("T,H", [(1, 4096), (4, 4096), (3, 1024)])
def test_folded_allreduce_push_and_reduce_roundtrip(T, H):
    ex = _exchange()
    torch.manual_seed(T)
    for rep in range(5):            # both parities, epochs advance on the device
        x = torch.randn(T, H, device=dev()).to(BF16)
        out = Fn.ll_reduce(Fn.ll_push(x, ex))
        assert torch.equal(out, x)
    assert ex.counters.tolist() == [5, 5]
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
@pytest.mark.parametrize("T", [1, 2, 4])
def test_projection_pushes_into_the_folded_allreduce(dtype, T):
    ex = _exchange()
    torch.manual_seed(10 + T)
    K, N = 1024, 4096
    x = torch.randn(T, K, device=dev()).to(BF16)
    lw = Fn.LinearWeight.from_master(torch.randn(N, K, device=dev()) * 0.05, dtype, dev())
    ref = Fn.linear(x, lw)
    for rep in range(3):
        p = Fn.linear(x, lw, ll=ex)
        assert isinstance(p, Fn.LLPending) and p.shape == (T, N)
        assert torch.equal(Fn.ll_reduce(p), ref)
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("T,H", [(1, 4096), (4, 4096), (2, 1024)])
def test_mhc_premix_consumes_the_folded_allreduce(T, H):
    """producer (projection with push) -> consumer (post+pre mix that adds the ranks) equals projection -> mix."""
    ex = _exchange()
    torch.manual_seed(20 + T)
    hc, K = 4, 1024
    res = torch.randn(T, hc, H, device=dev()).to(BF16)
    post_old = torch.rand(T, hc, device=dev()) * 2
    comb_old = torch.softmax(torch.randn(T, hc, hc, device=dev()), -1).reshape(T, hc * hc).contiguous()
    fn = torch.randn(24, hc * H, device=dev()) * 0.02
    base = torch.randn(24, device=dev()) * 0.1
    scale = torch.tensor([1.0, 0.7, 1.3], device=dev())
    nw = (1 + 0.1 * torch.randn(H, device=dev())).to(BF16)
    x = torch.randn(T, K, device=dev()).to(BF16)
    lw = Fn.LinearWeight((torch.randn(H, K, device=dev()) * 0.05).to(BF16))
    fa = Fn.linear(x, lw)
    ref_res, ref = Fn.mhc_post_pre(fa, res, post_old, comb_old, fn, base, scale, nw, 1e-6, 1e-6, 20)
    for rep in range(4):
        pend = Fn.linear(x, lw, ll=ex)
        new_res, r = Fn.mhc_post_pre(pend, res, post_old, comb_old, fn, base, scale, nw, 1e-6, 1e-6, 20)
        assert torch.equal(new_res, ref_res)
        for a, b in zip(r, ref):
            assert torch.equal(a, b)
    # and against the fp32 statement of the two ops
    rr = R.mhc_post(fa, res, post_old, comb_old.view(T, hc, hc)).to(BF16)
    assert rel_err(ref_res, rr) < 5e-3
    yr, pr, cr = R.mhc_pre(rr, fn, base, scale, nw, 1e-6, 1e-6, 20, round_bf16=True)
    assert rel_err(ref[0], yr) < 6e-3
    assert torch.allclose(ref[1], pr, atol=2e-3, rtol=2e-3)
    assert torch.allclose(ref[2].view(T, hc, hc), cr, atol=2e-3, rtol=2e-3)
    torch.cuda.synchronize()
    _lib.check_status()


def test_moe_combine_pushes_into_the_folded_allreduce():
    ex = _exchange()
    torch.manual_seed(31)
    T, H, I, E, k = 2, 4096, 2048, 16, 6
    ew = M.ExpertWeights.from_master(torch.randn(E, 2 * I, H) * 0.02, torch.randn(E, H, I) * 0.02, "nvfp4", dev())
    x = torch.randn(T, H, device=dev()).to(BF16)
    ids, w = M.router(torch.randn(T, E, device=dev()), None, k, "sigmoid", True, 1.0)
    shared = torch.randn(T, H, device=dev()).to(BF16)
    ref = M.moe_experts(x, ids, w, ew, 10.0, shared)
    for rep in range(2):
        p = M.moe_experts(x, ids, w, ew, 10.0, shared, ll=ex)
        assert isinstance(p, Fn.LLPending)
        assert torch.equal(Fn.ll_reduce(p), ref)
    torch.cuda.synchronize()
    _lib.check_status()


def test_engine_with_folded_allreduce_and_fused_launches_matches_unfused(monkeypatch):
    """The whole decode step with every fusion on (and the one-rank exchange standing in for tensor parallelism),
    through captured graphs, against the same engine with the separate launches."""
    from stkernel_b200.config import EngineConfig, SchedulerConfig, flash_config
    from stkernel_b200.models.dsv4 import RandomSource, build_model_weights
    from stkernel_b200.runtime.engine import Engine, SamplingParams
    cfg = flash_config(num_layers=3, n_routed_experts=16, vocab_size=4096)
    ec = EngineConfig(model=cfg, sched=SchedulerConfig(max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=256,
                                                       graph_cap=4)).validate()
    weights = build_model_weights(cfg, RandomSource(0), dev(), head_fp8=True)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (300, 17)]
    outs = {}
    for mode in ("unfused", "fused"):
        monkeypatch.setenv("STK_DECODE_FUSE", "1" if mode == "fused" else "0")
        monkeypatch.setenv("STK_LL_LOOPBACK", "1" if mode == "fused" else "0")
        eng = Engine(ec, weights, dev(), max_context=1024)
        # sampled, not greedy: random-init logits are nearly flat, so a greedy arg-max hangs on 1e-3 differences while
        # the seeded Gumbel noise separates the candidates by O(1)
        outs[mode] = eng.generate(prompts, SamplingParams(temperature=1.0, seed=11, max_tokens=12))
        torch.cuda.synchronize()
        _lib.check_status()
        if mode == "fused":
            assert eng.model._ll_loop is not None and eng.model._ll_loop.counters[0].item() > 0
    # The same noise picks the same token unless two candidates are within bf16 rounding of each other; after such a
    # flip the two texts are different continuations, so agreement is measured as the common prefix of each request
    # (the kernels themselves are compared exactly, one by one, in the tests above).
    def prefix(a, b):
        n = 0
        while n < min(len(a), len(b)) and a[n] == b[n]:
            n += 1
        return n
    pre = [prefix(x, y) for x, y in zip(outs["fused"], outs["unfused"])]
    assert min(pre) >= 2 and sum(pre) >= 10, (pre, outs)


@pytest.mark.parametrize("nh", [8, 16, 64])
@pytest.mark.parametrize("T", [1, 3])
def test_decode_attention_kernel_matches_reference(nh, T):
    """The register-resident decode kernel against the fp32 statement on the CPU: window + top-k rows with masked
    entries and short lists, sink, inverse RoPE of the output, and q normalised + rotated on load."""
    from stkernel_b200.ops import attention as A
    torch.manual_seed(40 + nh + T)
    D, Rd, W, K, n_pages = 512, 64, 128, 2048, 48
    ccpu = C.PagedCache.allocate(n_pages, D, Rd, True, "latent", "cpu")
    ccpu.write_rows_cpu(torch.arange(n_pages * 64), torch.randn(n_pages * 64, D))
    cg = C.PagedCache(ccpu.buf.to(dev()), D, Rd, True, "latent")
    q_raw = (torch.randn(T, nh, D) * 2.5).to(BF16)
    pos = torch.tensor([4000, 17, 33000][:T], dtype=torch.int64)
    inv = Fn.inv_freq(Rd, 10000.0, "cpu")
    swa = torch.randint(0, n_pages * 64, (T, W), dtype=torch.int32)
    swa_l = torch.tensor([W, 5, 77][:T], dtype=torch.int32)
    tk = torch.randint(0, n_pages * 64, (T, K), dtype=torch.int32)
    tk[0, 3] = -1
    tk_l = torch.tensor([K, 0, 700][:T], dtype=torch.int32)
    sink = torch.randn(nh)
    scale = D ** -0.5
    q_cpu = Fn.q_norm_rope(q_raw.clone(), pos, inv, Rd, 1e-6)
    ref = A.sparse_mla(q_cpu, ccpu, swa, swa_l, ccpu, tk, tk_l, sink, scale, inv_rope=(pos, inv))
    g = lambda x: x.to(dev())
    assert A.USE_DECODE_MLA
    out = A.sparse_mla(g(q_raw), cg, g(swa), g(swa_l), cg, g(tk), g(tk_l), g(sink), scale, inv_rope=(g(pos), g(inv)),
                       q_prep=(g(pos), g(inv), 1e-6))
    assert rel_err(out, ref) < 1.2e-2
    # q already prepared, window only, no inverse rotation
    ref2 = A.sparse_mla(q_cpu, ccpu, swa, swa_l, None, None, None, sink, scale)
    out2 = A.sparse_mla(g(q_cpu.to(BF16)), cg, g(swa), g(swa_l), None, None, None, g(sink), scale)
    assert rel_err(out2, ref2) < 1.2e-2
    # and against the tensor-core kernel on the same inputs
    A.USE_DECODE_MLA = False
    try:
        tc = A.sparse_mla(g(q_cpu.to(BF16)), cg, g(swa), g(swa_l), cg, g(tk), g(tk_l), g(sink), scale, inv_rope=(g(pos), g(inv)))
    finally:
        A.USE_DECODE_MLA = True
    assert rel_err(out, tc) < 1.2e-2
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("nh", [8, 64])
def test_decode_attention_inserts_the_tokens_own_row(nh):
    """Pure-decode step: the attention kernel builds, stores and attends to each token's own latent row.  The cache
    bytes must equal the stand-alone insert's, and the output the attention over that cache."""
    from stkernel_b200.ops import attention as A
    torch.manual_seed(50 + nh)
    D, Rd, W, K, n_pages, T = 512, 64, 128, 512, 40, 3
    base = C.PagedCache.allocate(n_pages, D, Rd, True, "latent", "cpu")
    base.write_rows_cpu(torch.arange(n_pages * 64), torch.randn(n_pages * 64, D))
    inv = Fn.inv_freq(Rd, 10000.0, dev())
    pos = torch.tensor([4000, 130, 77], dtype=torch.int64, device=dev())
    q_raw = (torch.randn(T, nh, D, device=dev()) * 2.0).to(BF16)
    kv_raw = (torch.randn(T, D, device=dev()) * 1.5).to(BF16)
    kv_w = (1 + 0.1 * torch.randn(D, device=dev())).to(BF16)
    swa = torch.randperm(n_pages * 64)[:T * W].view(T, W).to(torch.int32).to(dev())
    swa_l = torch.tensor([W, W, 78], dtype=torch.int32, device=dev())
    own = torch.stack([swa[i, int(swa_l[i]) - 1] for i in range(T)]).to(torch.int64)      # last window entry = own slot
    tk = torch.randint(0, n_pages * 64, (T, K), dtype=torch.int32, device=dev())
    tk_l = torch.tensor([K, 40, 0], dtype=torch.int32, device=dev())
    sink = torch.randn(nh, device=dev())
    scale = D ** -0.5
    # separate launches: insert, then attention
    c_ref = C.PagedCache(base.buf.to(dev()), D, Rd, True, "latent")
    C.q_rope_kv_insert(None, kv_raw, pos, own, inv, c_ref, 1e-6, kv_norm_w=kv_w)
    ref = A.sparse_mla(q_raw.clone(), c_ref, swa, swa_l, c_ref, tk, tk_l, sink, scale, inv_rope=(pos, inv), q_prep=(pos, inv, 1e-6))
    # one launch
    c_new = C.PagedCache(base.buf.to(dev()), D, Rd, True, "latent")
    out = A.sparse_mla(q_raw.clone(), c_new, swa, swa_l, c_new, tk, tk_l, sink, scale, inv_rope=(pos, inv), q_prep=(pos, inv, 1e-6),
                       kv_insert=(kv_raw, kv_w, own))
    torch.cuda.synchronize()
    assert torch.equal(c_new.buf, c_ref.buf)
    assert rel_err(out, ref) < 2e-3
    # a token without a slot (padding row) inserts nothing
    c_pad = C.PagedCache(base.buf.to(dev()), D, Rd, True, "latent")
    none = torch.full((T,), -1, dtype=torch.int64, device=dev())
    A.sparse_mla(q_raw.clone(), c_pad, swa, swa_l, c_pad, tk, tk_l, sink, scale, inv_rope=(pos, inv), q_prep=(pos, inv, 1e-6),
                 kv_insert=(kv_raw, kv_w, none))
    torch.cuda.synchronize()
    assert torch.equal(c_pad.buf.cpu(), base.buf)
    _lib.check_status()
