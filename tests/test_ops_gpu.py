"""Each sm_100a kernel against the PyTorch fp32 statement of the same op."""
import pytest
import torch

from stkernel_b200.ops import _lib
from stkernel_b200.ops import attention as A
from stkernel_b200.ops import cache as C
from stkernel_b200.ops import functional as Fn
from stkernel_b200.ops import moe as M
from stkernel_b200.ops import reference as R
from stkernel_b200.ops import sampling as S

pytestmark = pytest.mark.gpu
BF16, F32 = torch.bfloat16, torch.float32


def dev():
    return torch.device("cuda:0")


def rel_err(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / b.norm().clamp(min=1e-12)).item()


@pytest.mark.parametrize("T", [1, 8, 64, 256, 1000])
@pytest.mark.parametrize("N,K", [(512, 1024), (2048, 4096), (384, 576)])
def test_gemm_bf16(T, N, K):
    torch.manual_seed(T + N)
    x = torch.randn(T, K, device=dev()).to(BF16)
    w = torch.randn(N, K, device=dev()).to(BF16)
    ref = x.float() @ w.float().t()
    out = Fn.linear(x, Fn.LinearWeight(w))
    assert rel_err(out, ref) < 1e-2
    out32 = Fn.linear(x, Fn.LinearWeight(w), out_dtype=F32)
    assert rel_err(out32, ref) < 2e-3


@pytest.mark.parametrize("T,N,K", [(512, 512, 256), (700, 1000, 1024), (1024, 4160, 4096), (4096, 2048, 8192)])
def test_gemm_bf16_wide_tile(T, N, K):
    """Large bf16 problems: one CTA per 256 weight rows x 256 tokens (two accumulators), ragged edges included."""
    torch.manual_seed(T + N + K)
    x = (torch.randn(T, K, device=dev()) * 0.5).to(BF16)
    w = (torch.randn(N, K, device=dev()) * 0.5).to(BF16)
    ref = x.float() @ w.float().t()
    out = Fn.linear(x, Fn.LinearWeight(w))
    assert rel_err(out, ref) < 1e-2
    out32 = Fn.linear(x, Fn.LinearWeight(w), out_dtype=F32)
    assert rel_err(out32, ref) < 2e-3
    # element-wise, not only in norm: a misplaced tile would hide in a relative norm of random data
    assert (out32 - ref).abs().max().item() < 0.05 * ref.abs().max().item()
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("splits", [1, 2, 5])
def test_gemm_bf16_splitk_matches(splits):
    torch.manual_seed(1)
    x = torch.randn(8, 4096, device=dev()).to(BF16)
    w = torch.randn(256, 4096, device=dev()).to(BF16)
    ref = x.float() @ w.float().t()
    out = Fn.linear(x, Fn.LinearWeight(w), out_dtype=F32, splits=splits)
    assert rel_err(out, ref) < 2e-3


@pytest.mark.parametrize("T", [1, 6, 64, 128, 700])
@pytest.mark.parametrize("N,K", [(512, 1024), (2048, 4096), (1536, 7168)])
def test_gemm_fp8_block(T, N, K):
    torch.manual_seed(T)
    x = torch.randn(T, K, device=dev()).to(BF16)
    w = torch.randn(N, K, device=dev()) * 0.05
    lw = Fn.LinearWeight.from_master(w, "fp8", dev())
    xq, xs = R.quant_fp8_group128_act(x)
    ref = R.dequant_fp8_group128_act(xq, xs) @ lw.dequant().t()
    if T <= 4:                        # the CUDA-core weight-streaming kernel keeps the activations unquantised
        ref = x.float() @ lw.dequant().t()
    out = Fn.linear(x, lw, out_dtype=F32)
    assert rel_err(out, ref) < 2e-3
    # and against the unquantised product within fp8 error
    assert rel_err(out, x.float() @ w.t()) < 6e-2


def test_quant_act_matches_reference():
    x = (torch.randn(37, 640, device=dev()) * 3).to(BF16)
    qa = Fn.quant_act(x)
    q, s = R.quant_fp8_group128_act(x)
    assert torch.equal(qa.q.view(torch.uint8)[:37], q.view(torch.uint8))
    assert torch.allclose(qa.scale[:, :37].t(), s)


def test_rmsnorm_and_pair():
    x = torch.randn(9, 1536, device=dev()).to(BF16)
    w = (1 + 0.1 * torch.randn(1536, device=dev())).to(BF16)
    y = Fn.rms_norm(x, w, 1e-6)
    assert rel_err(y, R.rms_norm(x, w, 1e-6)) < 5e-3
    x1 = torch.randn(9, 512, device=dev()).to(BF16)
    w1 = torch.ones(512, device=dev()).to(BF16)
    a, b, qa = Fn.rms_norm_pair(x, w, x1, w1, 1e-6, quant0=True)
    assert rel_err(a, R.rms_norm(x, w, 1e-6)) < 5e-3
    assert rel_err(b, R.rms_norm(x1, w1, 1e-6)) < 5e-3
    deq = R.dequant_fp8_group128_act(qa.q[:9], qa.scale[:, :9].t())
    assert rel_err(deq, a) < 4e-2


def test_swiglu_clamp():
    gu = (torch.randn(5, 512, device=dev()) * 8).to(BF16)
    a = Fn.swiglu_clamp(gu, 10.0)
    assert rel_err(a, R.swiglu_clamp(gu[:, :256], gu[:, 256:], 10.0)) < 5e-3


@pytest.mark.parametrize("T,H", [(1, 4096), (7, 4096), (33, 256), (300, 4096), (700, 1024)])
def test_mhc_pre_post_head(T, H):
    torch.manual_seed(0)
    hc = 4
    res = torch.randn(T, hc, H, device=dev()).to(BF16)
    fn = torch.randn(24, hc * H, device=dev()) * 0.02
    base = torch.randn(24, device=dev()) * 0.1
    scale = torch.tensor([1.0, 0.7, 1.3], device=dev())
    nw = (1 + 0.1 * torch.randn(H, device=dev())).to(BF16)
    y, post, comb = Fn.mhc_pre(res, fn, base, scale, nw, 1e-6, 1e-6, 20)
    yr, pr, cr = R.mhc_pre(res, fn, base, scale, nw, 1e-6, 1e-6, 20, round_bf16=True)
    assert rel_err(y, yr) < 5e-3
    assert torch.allclose(post, pr, atol=1e-4, rtol=1e-4)
    assert torch.allclose(comb.view(T, hc, hc), cr, atol=1e-4, rtol=1e-3)
    # combine matrix is (nearly) doubly stochastic after Sinkhorn
    assert torch.allclose(comb.view(T, hc, hc).sum(1), torch.ones(T, hc, device=dev()), atol=1e-3)
    x = torch.randn(T, H, device=dev()).to(BF16)
    out = Fn.mhc_post(x, res, post, comb)
    assert rel_err(out, R.mhc_post(x, res, pr, cr)) < 5e-3
    hfn = torch.randn(hc, hc * H, device=dev()) * 0.02
    hb = torch.randn(hc, device=dev()) * 0.1
    hs = torch.tensor([0.9], device=dev())
    hh = Fn.hc_head(res, hfn, hb, hs, 1e-6, 1e-6)
    assert rel_err(hh, R.hc_head(res, hfn, hb, hs, 1e-6, 1e-6)) < 5e-3


@pytest.mark.parametrize("T,H", [(1, 4096), (5, 4096), (16, 1024), (40, 512)])
def test_mhc_post_pre_fused(T, H):
    """Post-mix of one sub-block fused into the next pre-mix (one cluster launch for T <= 16) against the two
    reference ops run back to back in fp32 (streams rounded to bf16 in between, as the unfused path stores them)."""
    torch.manual_seed(1)
    hc = 4
    res = torch.randn(T, hc, H, device=dev()).to(BF16)
    x = torch.randn(T, H, device=dev()).to(BF16)
    post_old = torch.rand(T, hc, device=dev()) * 2
    comb_old = torch.softmax(torch.randn(T, hc, hc, device=dev()), -1).reshape(T, hc * hc).contiguous()
    fn = torch.randn(24, hc * H, device=dev()) * 0.02
    base = torch.randn(24, device=dev()) * 0.1
    scale = torch.tensor([1.0, 0.7, 1.3], device=dev())
    nw = (1 + 0.1 * torch.randn(H, device=dev())).to(BF16)
    new_res, r = Fn.mhc_post_pre(x, res, post_old, comb_old, fn, base, scale, nw, 1e-6, 1e-6, 20)
    ref_res = R.mhc_post(x, res, post_old, comb_old.view(T, hc, hc)).to(BF16)
    assert rel_err(new_res, ref_res) < 5e-3
    yr, pr, cr = R.mhc_pre(ref_res, fn, base, scale, nw, 1e-6, 1e-6, 20, round_bf16=True)
    assert rel_err(r[0], yr) < 6e-3
    assert torch.allclose(r[1], pr, atol=2e-3, rtol=2e-3)
    assert torch.allclose(r[2].view(T, hc, hc), cr, atol=2e-3, rtol=2e-3)


def _rope_setup(T, R_):
    pos = torch.randint(0, 100000, (T,), device=dev(), dtype=torch.int64)
    inv = Fn.inv_freq(R_, 10000.0, dev())
    ang = pos.float()[:, None] * inv[None]
    return pos, inv, torch.cos(ang), torch.sin(ang)


def test_q_norm_rope():
    T, nh, D, R_ = 5, 8, 512, 64
    q = torch.randn(T, nh, D, device=dev()).to(BF16)
    pos, inv, cos, sin = _rope_setup(T, R_)
    ref = R.rms_norm(q, None, 1e-6)
    ref = torch.cat([ref[..., :D - R_], R.apply_rope_interleaved(ref[..., D - R_:], cos, sin)], -1)
    out = Fn.q_norm_rope(q.clone(), pos, inv, R_, 1e-6)
    assert rel_err(out, ref) < 6e-3


@pytest.mark.parametrize("fp8", [True, False])
def test_kv_insert_gather_roundtrip(fp8):
    T, D, R_ = 70, 512, 64
    kv = torch.randn(T, D, device=dev()).to(BF16)
    pos, inv, cos, sin = _rope_setup(T, R_)
    cache = C.PagedCache.allocate(4, D, R_, fp8, "latent", dev())
    slots = torch.randperm(4 * 64, device=dev())[:T].to(torch.int64)
    slots[3] = -1
    C.kv_rope_quant_insert(kv, pos, slots, inv, cache)
    rows = C.kv_gather_dequant(cache, slots)
    roped = torch.cat([kv.float()[:, :D - R_], R.apply_rope_interleaved(kv[:, D - R_:], cos, sin).to(BF16).float()], 1)
    ref = R.kv_fake_quant(roped, R_) if fp8 else roped.to(BF16).float()
    ref[3] = 0
    assert rel_err(rows, ref) < 4e-3
    # byte-exact against the CPU writer of the same format
    cpu = C.PagedCache.allocate(4, D, R_, fp8, "latent", "cpu")
    cpu.write_rows_cpu(slots.cpu(), roped.cpu())
    same = (cpu.buf == cache.buf.cpu()).float().mean().item()
    assert same > 0.999


@pytest.mark.parametrize("ratio,c,kind,fp8", [(4, 2, "latent", True), (4, 2, "indexer", True), (128, 1, "latent", False)])
def test_compress_windows_matches_cpu(ratio, c, kind, fp8):
    torch.manual_seed(3)
    D = 512 if kind == "latent" else 128
    R_ = 64
    ring = 2 * ratio if c == 2 else ratio
    # two requests: a 300-token prefill chunk starting at 0 and a decode token at position 2*ratio-1 with state
    lens = [300, 1]
    starts = [0, 2 * ratio - 1]
    T = sum(lens)
    kvs = torch.randn(T, 2 * c * D)
    ape = torch.randn(ratio, c * D) * 0.1
    nw = (1 + 0.1 * torch.randn(D)).to(BF16)
    inv = Fn.inv_freq(R_, 10000.0, "cpu")
    qs = torch.tensor([0, 300, 301], dtype=torch.int32)
    tok_req, positions, first, last = A.token_maps(qs, torch.tensor([0, 1], dtype=torch.int32),
                                                   torch.tensor(starts, dtype=torch.int32), 2, T)
    state = torch.randn(2, ring, 2 * c * D)
    bt = torch.tensor([[0, 1], [2, 3]], dtype=torch.int32)
    cpu_cache = C.PagedCache.allocate(4, D, R_, fp8, kind, "cpu")
    st_cpu = state.clone()
    C.compress_windows(kvs, ape, nw, inv, positions, tok_req, first, last, st_cpu, bt, cpu_cache, ratio, c, 1e-6)
    g = lambda t: t.to(dev())
    gpu_cache = C.PagedCache.allocate(4, D, R_, fp8, kind, dev())
    st_gpu = g(state.clone())
    C.compress_windows(g(kvs), g(ape), g(nw), g(inv), g(positions), g(tok_req), g(first), g(last), st_gpu, g(bt),
                       gpu_cache, ratio, c, 1e-6)
    n_win = 300 // ratio
    slots = torch.cat([torch.arange(n_win), torch.tensor([2 * 64 + 1])])
    a, sa = cpu_cache.read_rows_cpu(slots)
    gc = C.PagedCache(gpu_cache.buf.cpu(), D, R_, fp8, kind)
    b, sb = gc.read_rows_cpu(slots)
    if sa is not None:
        a, b = a * sa[:, None], b * sb[:, None]
    assert a.abs().sum() > 0
    assert rel_err(b, a) < 3e-2
    assert torch.allclose(st_gpu.cpu(), st_cpu)


def test_indexer_q_prep():
    T, ih, d, R_ = 6, 64, 128, 64
    q = torch.randn(T, ih, d, device=dev()).to(BF16)
    w = torch.randn(T, ih, device=dev())
    pos, inv, cos, sin = _rope_setup(T, R_)
    qq, wf = C.indexer_q_prep(q, w, pos, inv, R_, True)
    rq, rw = R.indexer_q_prepare(q, w, cos, sin, R_, True)
    # compare dequantised operands (scale folded into the weights)
    assert rel_err(qq.float() * wf[..., None], rq * rw[..., None]) < 2e-2


def _fill_indexer_cache(S, d, fp8):
    k = torch.randn(S, d, device=dev())
    cache = C.PagedCache.allocate((S + 63) // 64 + 1, d, 64, fp8, "indexer", "cpu")
    cache.write_rows_cpu(torch.arange(S), k.cpu())
    return k, C.PagedCache(cache.buf.to(dev()), d, 64, fp8, "indexer"), cache


@pytest.mark.parametrize("T", [3, 131, 300])
def test_indexer_scores_tensor_core_matches_cuda_core(T):
    """tcgen05 scorer (K block stationary, q tiles by TMA, head sum in the TMEM lane) against the CUDA-core scorer and
    the CPU reference: two requests with scattered pages, causal n_valid, a padded token (request -1)."""
    torch.manual_seed(17)
    ih, d, S = 64, 128, 1000
    n_pages = 2 * ((S + 63) // 64) + 3
    cache = C.PagedCache.allocate(n_pages, d, 64, True, "indexer", "cpu")
    perm = torch.randperm(n_pages - 1)[:2 * ((S + 63) // 64)] + 1
    bt_cpu = perm.view(2, -1).to(torch.int32)
    for req in range(2):
        k = torch.randn(S, d)
        slots = bt_cpu[req].long()[torch.arange(S) // 64] * 64 + torch.arange(S) % 64
        cache.write_rows_cpu(slots, k)
    gcache = C.PagedCache(cache.buf.to(dev()), d, 64, True, "indexer")
    bt = bt_cpu.to(dev()).contiguous()
    q = torch.randn(T, ih, d, device=dev()).to(BF16)
    w = torch.rand(T, ih, device=dev())
    split = T // 3                                          # request 0: first third, request 1: the rest
    tok_req = torch.cat([torch.zeros(split, dtype=torch.int32), torch.ones(T - split, dtype=torch.int32)]).to(dev())
    pos = torch.cat([torch.arange(split) + 900, torch.arange(T - split) * 9 + 5]).to(dev())
    tok_req[-1] = -1
    inv = Fn.inv_freq(64, 10000.0, dev())
    qq, wf = C.indexer_q_prep(q, w, pos, inv, 64, True)
    nv = A.compressed_valid(pos, 4)
    nv[-1] = 0
    assert int(nv.max()) <= S
    assert A.USE_TENSOR_CORE_INDEXER
    before = A.tc_indexer_calls
    tc = A.indexer_scores(qq, wf, gcache, bt, tok_req, nv, S, tag="idx_tc_test").clone()
    assert A.tc_indexer_calls == before + 1
    A.USE_TENSOR_CORE_INDEXER = False
    try:
        cc = A.indexer_scores(qq, wf, gcache, bt, tok_req, nv, S, tag="idx_cc_test").clone()
    finally:
        A.USE_TENSOR_CORE_INDEXER = True
    checked = 0
    for i in range(T):
        n = int(nv[i])
        if n:
            assert rel_err(tc[i, :n], cc[i, :n]) < 1e-3, i
            checked += 1
    assert checked >= T // 2
    sub = [0, max(0, split - 1), min(T - 2, split)]
    ref = A.indexer_scores(qq[sub].cpu(), wf[sub].cpu(), cache, bt_cpu, tok_req[sub].cpu(), nv[sub].cpu(), S)
    for j, i in enumerate(sub):
        n = int(nv[i])
        if n:
            assert rel_err(tc[i, :n], ref[j, :n]) < 2e-3


@pytest.mark.parametrize("fp8", [True, False])
def test_indexer_scores_and_topk(fp8):
    torch.manual_seed(5)
    T, ih, d, S, K = 5, 64, 128, 700, 64
    k, gcache, ccache = _fill_indexer_cache(S, d, fp8)
    q = torch.randn(T, ih, d, device=dev()).to(BF16)
    w = torch.rand(T, ih, device=dev())
    pos = torch.tensor([S * 4 - 1, 100, 3, 2000, 1023], device=dev(), dtype=torch.int64)
    inv = Fn.inv_freq(64, 10000.0, dev())
    qq, wf = C.indexer_q_prep(q, w, pos, inv, 64, fp8)
    bt = torch.arange(gcache.num_pages, dtype=torch.int32, device=dev())[None].contiguous()
    tok_req = torch.zeros(T, dtype=torch.int32, device=dev())
    nv = A.compressed_valid(pos, 4)
    scores = A.indexer_scores(qq, wf, gcache, bt, tok_req, nv, S)
    ref = A.indexer_scores(qq.cpu(), wf.cpu(), ccache, bt.cpu(), tok_req.cpu(), nv.cpu(), S)
    for i in range(T):
        n = int(nv[i])
        if n:
            assert rel_err(scores[i, :n], ref[i, :n]) < 2e-3
    top = A.topk_rows(scores, nv, K)
    for i in range(T):
        n = int(nv[i])
        got = top[i][top[i] >= 0].cpu()
        assert got.numel() == min(n, K)
        assert got.unique().numel() == got.numel()
        if n > K:
            thr = torch.topk(scores[i, :n], K).values.min()
            assert (scores[i, got.to(dev()).long()] >= thr).all()
        elif n > 0:
            assert torch.equal(got.sort().values, torch.arange(n, dtype=torch.int32))


def test_topk_large_with_ties():
    T, S, K = 3, 40000, 2048
    scores = torch.randn(T, S, device=dev())
    scores[1] = torch.randint(0, 50, (S,), device=dev()).float()      # heavy ties
    nv = torch.tensor([S, S, 5000], dtype=torch.int32, device=dev())
    top = A.topk_rows(scores, nv, K)
    for i in range(T):
        got = top[i].long()
        assert (got >= 0).all() and got.unique().numel() == K
        n = int(nv[i])
        assert (got < n).all()
        thr = torch.topk(scores[i, :n], K).values.min()
        assert (scores[i, got] >= thr).all()
        assert torch.isclose(scores[i, got].sum(), torch.topk(scores[i, :n], K).values.sum(), rtol=1e-4)


@pytest.mark.parametrize("nh,D,R_,fp8", [(64, 512, 64, True), (8, 512, 64, True), (4, 80, 16, False)])
def test_sparse_mla_matches_reference(nh, D, R_, fp8):
    torch.manual_seed(7)
    T, W, K = 4, 128, 512 if D == 512 else 16
    n_pages = 24
    rows = torch.randn(n_pages * 64, D)
    ccpu = C.PagedCache.allocate(n_pages, D, R_, fp8, "latent", "cpu")
    ccpu.write_rows_cpu(torch.arange(n_pages * 64), rows)
    cg = C.PagedCache(ccpu.buf.to(dev()), D, R_, fp8, "latent")
    q = torch.randn(T, nh, D, device=dev()).to(BF16)
    swa_slots = torch.randint(0, n_pages * 64, (T, W), dtype=torch.int32, device=dev())
    swa_lens = torch.tensor([W, 5, 1, 77], dtype=torch.int32, device=dev())
    topk_slots = torch.randint(0, n_pages * 64, (T, K), dtype=torch.int32, device=dev())
    topk_slots[0, 3] = -1
    topk_lens = torch.tensor([K, 0, K // 2, 9], dtype=torch.int32, device=dev())
    sink = torch.randn(nh, device=dev())
    out = A.sparse_mla(q, cg, swa_slots, swa_lens, cg, topk_slots, topk_lens, sink, D ** -0.5)
    ref = A.sparse_mla(q.cpu(), ccpu, swa_slots.cpu(), swa_lens.cpu(), ccpu, topk_slots.cpu(), topk_lens.cpu(),
                       sink.cpu(), D ** -0.5)
    assert rel_err(out, ref) < 1e-2
    out2 = A.sparse_mla(q, cg, swa_slots, swa_lens, None, None, None, sink, D ** -0.5)
    ref2 = A.sparse_mla(q.cpu(), ccpu, swa_slots.cpu(), swa_lens.cpu(), None, None, None, sink.cpu(), D ** -0.5)
    assert rel_err(out2, ref2) < 1e-2


@pytest.mark.parametrize("nh", [64, 8])
def test_sparse_mla_direct_output_matches_split_path(nh):
    """Steps with many tokens take the single-split kernel that writes the final rows itself (sink merge, normalisation,
    inverse RoPE in its epilogue); compare with the fp32 reference and with the partial + combine path."""
    torch.manual_seed(9)
    D, R_, T, W, K = 512, 64, 320, 128, 256
    n_pages = 24
    rows = torch.randn(n_pages * 64, D)
    ccpu = C.PagedCache.allocate(n_pages, D, R_, True, "latent", "cpu")
    ccpu.write_rows_cpu(torch.arange(n_pages * 64), rows)
    cg = C.PagedCache(ccpu.buf.to(dev()), D, R_, True, "latent")
    q = torch.randn(T, nh, D, device=dev()).to(BF16)
    swa_slots = torch.randint(0, n_pages * 64, (T, W), dtype=torch.int32, device=dev())
    swa_lens = torch.randint(0, W + 1, (T,), dtype=torch.int32, device=dev())
    topk_slots = torch.randint(0, n_pages * 64, (T, K), dtype=torch.int32, device=dev())
    topk_slots[0, 3] = -1
    topk_lens = torch.randint(0, K + 1, (T,), dtype=torch.int32, device=dev())
    swa_lens[1] = 0
    topk_lens[1] = 0                      # a token without any key: only the sink has mass, output zero
    sink = torch.randn(nh, device=dev())
    pos = torch.randint(0, 50000, (T,), device=dev(), dtype=torch.int64)
    inv = Fn.inv_freq(R_, 10000.0, dev())
    assert A.MLA_DIRECT_OUT
    out = A.sparse_mla(q, cg, swa_slots, swa_lens, cg, topk_slots, topk_lens, sink, D ** -0.5, inv_rope=(pos, inv))
    A.MLA_DIRECT_OUT = False
    try:
        split = A.sparse_mla(q, cg, swa_slots, swa_lens, cg, topk_slots, topk_lens, sink, D ** -0.5, inv_rope=(pos, inv))
    finally:
        A.MLA_DIRECT_OUT = True
    assert rel_err(out, split) < 4e-3
    assert float(out[1].float().abs().max()) == 0.0
    sub = slice(0, 6)
    ref = A.sparse_mla(q[sub].cpu(), ccpu, swa_slots[sub].cpu(), swa_lens[sub].cpu(), ccpu, topk_slots[sub].cpu(),
                       topk_lens[sub].cpu(), sink.cpu(), D ** -0.5, inv_rope=(pos[sub].cpu(), inv.cpu()))
    assert rel_err(out[sub], ref) < 1.2e-2


@pytest.mark.parametrize("scoring", ["sigmoid", "sqrtsoftplus"])
def test_router(scoring):
    T, E, k = 33, 256, 6
    logits = torch.randn(T, E, device=dev())
    bias = (torch.rand(E, device=dev()) * 0.2 - 0.1)
    ids, w = M.router(logits, bias, k, scoring, True, 2.5)
    rid, rw = R.route(logits, bias, k, scoring, True, 2.5)
    assert torch.equal(ids.sort(-1).values, rid.sort(-1).values)
    assert torch.allclose(w.sum(-1), rw.sum(-1), rtol=1e-4)
    tid2eid = torch.randint(0, E, (1000, k), dtype=torch.int32, device=dev())
    toks = torch.randint(0, 1000, (T,), device=dev())
    ids2, w2 = M.router(logits, None, k, scoring, True, 1.0, tid2eid, toks)
    assert torch.equal(ids2, tid2eid[toks])
    rid2, rw2 = R.route(logits, None, k, scoring, True, 1.0, tid2eid[toks])
    assert torch.allclose(w2, rw2, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("T,H,I,E", [(1, 4096, 2048, 16), (7, 4096, 2048, 16), (5, 256, 128, 8)])
def test_moe_experts_nvfp4(T, H, I, E):
    torch.manual_seed(11)
    k = 2 if E == 8 else 6
    w13 = torch.randn(E, 2 * I, H) * 0.02
    w2 = torch.randn(E, H, I) * 0.02
    ew = M.ExpertWeights.from_master(w13, w2, "nvfp4", dev())
    x = torch.randn(T, H, device=dev()).to(BF16)
    logits = torch.randn(T, E, device=dev())
    ids, w = M.router(logits, None, k, "sigmoid", True, 1.0)
    shared = torch.randn(T, H, device=dev()).to(BF16)
    out = M.moe_experts(x, ids, w, ew, 10.0, shared)
    d13, d2 = ew.dequant()
    ref = R.moe_experts(x, ids, w, d13, d2, 10.0) + shared.float()
    assert rel_err(out, ref) < 1.5e-2
    # expert-parallel slice: only experts [E/2, E) are local
    ew_hi = M.ExpertWeights(ew.w13[E // 2:], ew.w2[E // 2:], ew.s13[E // 2:], ew.s2[E // 2:], ew.g13[E // 2:],
                            ew.g2[E // 2:], E // 2)
    out_hi = M.moe_experts(x, ids, w, ew_hi, 10.0)
    ref_hi = R.moe_experts(x, ids, w, d13[E // 2:], d2[E // 2:], 10.0, E // 2)
    assert rel_err(out_hi, ref_hi) < 1.5e-2


def test_moe_experts_sliced_along_the_intermediate_dimension():
    """Decode steps under tensor parallelism: every rank holds 1/tp of every expert's intermediate rows; the ranks'
    partial results add up to the whole experts' output."""
    torch.manual_seed(12)
    T, H, I, E, k, tp = 2, 4096, 2048, 16, 6, 8
    w13 = torch.randn(E, 2 * I, H) * 0.02
    w2 = torch.randn(E, H, I) * 0.02
    x = torch.randn(T, H, device=dev()).to(BF16)
    ids, w = M.router(torch.randn(T, E, device=dev()), None, k, "sigmoid", True, 1.0)
    il = I // tp
    total = torch.zeros(T, H)
    ref = torch.zeros(T, H)
    for r in range(tp):
        sl = slice(r * il, (r + 1) * il)
        w13_r = torch.cat([w13[:, :I][:, sl], w13[:, I:][:, sl]], 1).contiguous()
        w2_r = w2[:, :, sl].contiguous()
        ew = M.ExpertWeights.from_master(w13_r, w2_r, "nvfp4", dev())
        out = M.moe_experts(x, ids, w, ew, 10.0, None, E)
        d13, d2 = ew.dequant()
        ref += R.moe_experts(x, ids, w, d13, d2, 10.0).float().cpu()
        total += out.float().cpu()
    assert rel_err(total, ref) < 1.5e-2
    full = R.moe_experts(x, ids, w, w13.to(dev()), w2.to(dev()), 10.0).float().cpu()
    assert rel_err(total, full) < 0.25          # NVFP4 quantisation of the weights
    torch.cuda.synchronize()
    _lib.check_status()


def test_gumbel_argmax_and_coupling():
    B, N, V = 3, 5, 129280
    logits = torch.randn(B * (N + 1), V, device=dev())
    temp = torch.tensor([0.6, 0.0, 1.0], device=dev())
    seed = torch.tensor([1, 2 ** 40 + 7, 3], device=dev(), dtype=torch.int64)
    pos = torch.tensor([10, 2000, 5], device=dev(), dtype=torch.int64)
    tok, proc = S.gumbel_argmax(logits, temp, seed, pos, rows_per_request=N + 1, want_processed=True)
    rtok, rproc = S.gumbel_argmax(logits.cpu(), temp.cpu(), seed.cpu(), pos.cpu(), rows_per_request=N + 1,
                                  want_processed=True)
    assert torch.equal(tok.cpu(), rtok)
    assert torch.allclose(proc.cpu(), rproc, rtol=1e-5, atol=1e-5)
    # same (seed, pos) => same noise: sampling identical logits twice gives identical tokens
    tok2, _ = S.gumbel_argmax(logits, temp, seed, pos, rows_per_request=N + 1)
    assert torch.equal(tok, tok2)
    ver = tok.view(B, N + 1)
    draft = ver[:, :N].clone()
    draft[0, 2] = (draft[0, 2] + 1) % V
    acc, em = S.coupled_accept(ver, draft)
    assert acc.tolist() == [2, N, N]
    assert em[0].tolist()[:3] == ver[0].tolist()[:3] and (em[0, 3:] == -1).all()


def test_markov_topk_bias():
    B, V, Rk = 2, 129280, 256
    base = torch.randn(B, V, device=dev()).to(BF16)
    w2 = (torch.randn(V, Rk, device=dev()) * 0.02).to(BF16)
    emb = torch.randn(B, Rk, device=dev()).to(BF16)
    out = S.markov_topk_bias(base, w2, emb, 512)
    ref = R.markov_bias_topk(base, w2, emb, 512)
    fin = torch.isfinite(ref)
    assert torch.equal(torch.isfinite(out), fin) or (torch.isfinite(out).sum(-1) == 512).all()
    assert (torch.isfinite(out).sum(-1) == 512).all()
    both = fin & torch.isfinite(out)
    assert torch.allclose(out[both], ref[both], rtol=1e-3, atol=1e-3)
    dense = S.markov_topk_bias(base, w2, emb, 0)
    assert torch.allclose(dense, R.markov_bias_topk(base, w2, emb, 0), rtol=1e-3, atol=1e-3)


def test_swa_indices_and_slots():
    pos = torch.tensor([0, 5, 200, -1], device=dev(), dtype=torch.int64)
    tok_req = torch.tensor([0, 1, 1, -1], dtype=torch.int32, device=dev())
    bt = torch.tensor([[3, 4, 5, 6], [7, 8, 9, 10]], dtype=torch.int32, device=dev())
    s, l = A.swa_indices(pos, tok_req, bt, 128)
    rs, rl = A.swa_indices(pos.cpu(), tok_req.cpu(), bt.cpu(), 128)
    assert torch.equal(s.cpu(), rs) and torch.equal(l.cpu(), rl)
    topk = torch.tensor([[0, 65, -1, 130], [1, 2, 3, 4]], dtype=torch.int32, device=dev())
    sl, ln = A.topk_to_slots(topk, bt, tok_req[:2].contiguous(), 256)
    rsl, rln = A.topk_to_slots(topk.cpu(), bt.cpu(), tok_req[:2].cpu(), 256)
    assert torch.equal(sl.cpu(), rsl) and torch.equal(ln.cpu(), rln)


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
@pytest.mark.parametrize("T", [1, 40, 300])
def test_gemm_grouped_block_diagonal(dtype, T):
    torch.manual_seed(2)
    G, Ng, K = 4, 256, 512
    x = torch.randn(T, G * K, device=dev()).to(BF16)
    ws = [torch.randn(Ng, K, device=dev()) * 0.05 for _ in range(G)]
    lws = [Fn.LinearWeight.from_master(w, dtype, dev()) for w in ws]
    stacked = Fn.LinearWeight(torch.cat([l.w for l in lws], 0).contiguous(),
                              torch.cat([l.scale for l in lws], 0).contiguous() if dtype == "fp8" else None)
    out = Fn.linear(x, stacked, out_dtype=F32, groups=G)
    for g in range(G):
        xg = x[:, g * K:(g + 1) * K]
        if dtype == "fp8" and T > 4:
            xq, xs = R.quant_fp8_group128_act(xg)
            ref = R.dequant_fp8_group128_act(xq, xs) @ lws[g].dequant().t()
        else:
            ref = xg.float() @ lws[g].dequant().t()
        assert rel_err(out[:, g * Ng:(g + 1) * Ng], ref) < 3e-3


@pytest.mark.parametrize("T,N,K", [(64, 4096, 8192), (100, 384, 1024), (128, 4096, 2048), (256, 4096, 8192), (300, 640, 2048)])
def test_gemm_splitk_wide_tiles(T, N, K):
    torch.manual_seed(3)
    x = torch.randn(T, K, device=dev()).to(BF16)
    w = torch.randn(N, K, device=dev()).to(BF16)
    ref = x.float() @ w.float().t()
    for splits in (2, 4):
        assert rel_err(Fn.linear(x, Fn.LinearWeight(w), splits=splits), ref) < 1e-2


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
@pytest.mark.parametrize("T", [1, 3, 4])
@pytest.mark.parametrize("N,K", [(2048, 4096), (40960, 1536), (4096, 8192), (176, 256)])
def test_skinny_linear(dtype, T, N, K):
    torch.manual_seed(T)
    x = torch.randn(T, K, device=dev()).to(BF16)
    w = torch.randn(N, K, device=dev()) * 0.05
    lw = Fn.LinearWeight.from_master(w, dtype, dev())
    ref = x.float() @ lw.dequant().t()
    out = Fn.linear(x, lw, out_dtype=F32)          # T <= 4 routes to the weight-streaming kernel
    assert rel_err(out, ref) < 2e-3
    out16 = Fn.linear(x, lw)
    assert rel_err(out16, ref) < 1e-2


def test_skinny_linear_grouped():
    G, Ng, K, T = 8, 1024, 4096, 2
    x = torch.randn(T, G * K, device=dev()).to(BF16)
    w = torch.randn(G * Ng, K, device=dev()) * 0.05
    lw = Fn.LinearWeight.from_master(w, "fp8", dev())
    out = Fn.linear(x, lw, out_dtype=F32, groups=G)
    wd = lw.dequant().view(G, Ng, K)
    ref = torch.einsum("tgk,gnk->tgn", x.float().view(T, G, K), wd).reshape(T, G * Ng)
    assert rel_err(out, ref) < 2e-3


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
def test_skinny_swiglu(dtype):
    T, I, K = 2, 2048, 4096
    x = torch.randn(T, K, device=dev()).to(BF16)
    w = torch.randn(2 * I, K, device=dev()) * 0.03
    lw = Fn.LinearWeight.from_master(w, dtype, dev())
    act = Fn.linear_swiglu(x, lw, 10.0)
    gu = x.float() @ lw.dequant().t()
    ref = R.swiglu_clamp(gu[:, :I], gu[:, I:], 10.0)
    assert rel_err(act, ref) < 1e-2


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
@pytest.mark.parametrize("T", [5, 6, 8])
@pytest.mark.parametrize("N,K", [(2048, 4096), (16160, 1536), (4096, 8192), (176, 256), (576, 4096)])
def test_skinny_mma_linear_five_to_eight_tokens(dtype, T, N, K, monkeypatch):
    """Five to eight tokens: the warp-level tensor-core stream (fp8 activations quantised per 128 values inside the
    kernel, exactly like the GEMM path)."""
    monkeypatch.setattr(Fn, "SKINNY_MAX_T", 8)
    torch.manual_seed(T + N)
    buf = torch.randn(T, K + 256, device=dev()).to(BF16) * 2.0        # a strided view
    x = buf[:, :K]
    w = torch.randn(N, K, device=dev()) * 0.05
    lw = Fn.LinearWeight.from_master(w, dtype, dev())
    before = _lib.launch_count
    out = Fn.linear(x, lw, out_dtype=F32)
    if Fn._skinny_ok(x, T, K, dtype == "fp8", N):   # (the largest fp8 case at 8 tokens exceeds the staging area)
        assert _lib.launch_count == before + 1      # one kernel: no separate quantisation, no split-K reduction
    if dtype == "fp8":
        xq, xs = R.quant_fp8_group128_act(x.contiguous())
        ref = R.dequant_fp8_group128_act(xq, xs) @ lw.dequant().t()
    else:
        ref = x.float() @ lw.dequant().t()
    assert rel_err(out, ref) < 2e-3
    assert rel_err(Fn.linear(x, lw), ref) < 1e-2
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("T", [9, 16, 33, 64])
@pytest.mark.parametrize("N,K", [(256, 4096), (512, 4096), (1024, 1536)])
def test_skinny_mma_narrow_weights_up_to_64_tokens(T, N, K, monkeypatch):
    """The router gate at decode batch sizes: the bf16 weight (<= 4 MB) is streamed once per group of eight tokens
    instead of through a mostly empty tensor-core tile with split-K (an option: STK_SKINNY_NARROW=1)."""
    monkeypatch.setattr(Fn, "SKINNY_NARROW", True)
    torch.manual_seed(T * 7 + N)
    x = torch.randn(T, K, device=dev()).to(BF16)
    lw = Fn.LinearWeight((torch.randn(N, K, device=dev()) * 0.05).to(BF16))
    assert Fn._skinny_ok(x, T, K, False, N, N)
    before = _lib.launch_count
    out = Fn.linear(x, lw, out_dtype=F32)
    assert _lib.launch_count == before + 1
    ref = x.float() @ lw.dequant().t()
    assert rel_err(out, ref) < 2e-3
    assert (out - ref).abs().max().item() < 0.02 * ref.abs().max().item()
    nw = (1 + 0.1 * torch.randn(K, device=dev())).to(BF16)
    xn = R.rms_norm(x, nw, 1e-6).to(BF16)
    assert rel_err(Fn.linear(x, lw, norm=(nw, 1e-6)), xn.float() @ lw.dequant().t()) < 1e-2
    # fp8 weights at these batch sizes stay on the tensor-core tile
    lw8 = Fn.LinearWeight.from_master(torch.randn(N, K, device=dev()) * 0.05, "fp8", dev())
    assert not Fn._skinny_ok(x, T, K, True, N, N)
    ref8 = R.dequant_fp8_group128_act(*R.quant_fp8_group128_act(x)) @ lw8.dequant().t()
    assert rel_err(Fn.linear(x, lw8, out_dtype=F32), ref8) < 2e-3
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
def test_skinny_mma_grouped_and_swiglu(dtype, monkeypatch):
    monkeypatch.setattr(Fn, "SKINNY_MAX_T", 8)
    torch.manual_seed(9)
    G, Ng, K, T = 8, 1024, 512, 6
    x = torch.randn(T, G * K, device=dev()).to(BF16)
    lw = Fn.LinearWeight.from_master(torch.randn(G * Ng, K, device=dev()) * 0.05, dtype, dev())
    out = Fn.linear(x, lw, out_dtype=F32, groups=G)
    wd = lw.dequant().view(G, Ng, K)
    if dtype == "fp8":
        xf = torch.cat([R.dequant_fp8_group128_act(*R.quant_fp8_group128_act(x[:, g * K:(g + 1) * K].contiguous()))
                        for g in range(G)], 1)
    else:
        xf = x.float()
    ref = torch.einsum("tgk,gnk->tgn", xf.view(T, G, K), wd).reshape(T, G * Ng)
    assert rel_err(out, ref) < 2e-3
    I, K2 = 2048, 4096
    x2 = torch.randn(T, K2, device=dev()).to(BF16)
    lw2 = Fn.LinearWeight.from_master(torch.randn(2 * I, K2, device=dev()) * 0.03, dtype, dev())
    act = Fn.linear_swiglu(x2, lw2, 10.0)
    assert act is not None
    x2f = R.dequant_fp8_group128_act(*R.quant_fp8_group128_act(x2)) if dtype == "fp8" else x2.float()
    gu = x2f @ lw2.dequant().t()
    assert rel_err(act, R.swiglu_clamp(gu[:, :I], gu[:, I:], 10.0)) < 1e-2
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("T,E,k", [(64, 16, 6), (700, 16, 6), (300, 32, 2), (2048, 8, 2)])
def test_moe_grouped_gemm_nvfp4(T, E, k):
    """Batches beyond a handful of pairs go through the tcgen05 grouped GEMM."""
    torch.manual_seed(13)
    H, I = 1024, 512
    w13 = torch.randn(E, 2 * I, H) * 0.03
    w2 = torch.randn(E, H, I) * 0.03
    ew = M.ExpertWeights.from_master(w13, w2, "nvfp4", dev())
    x = torch.randn(T, H, device=dev()).to(BF16)
    logits = torch.randn(T, E, device=dev())
    logits[:, 0] -= 100.0                               # expert 0 never selected: an empty group
    ids, w = M.router(logits, None, k, "sigmoid", True, 1.0)
    out = M.moe_experts(x, ids, w, ew, 10.0, None, E)
    d13, d2 = ew.dequant()
    ref = R.moe_experts(x, ids, w, d13, d2, 10.0)
    assert rel_err(out, ref) < 1.5e-2
    M.USE_GROUPED_GEMM = False
    try:
        out2 = M.moe_experts(x, ids, w, ew, 10.0, None, E)
    finally:
        M.USE_GROUPED_GEMM = True
    assert rel_err(out, out2) < 1.5e-2


def test_topk_candidates_and_markov_chain_match_cpu():
    """The drafter's sampling path: two-level candidate selection over the full vocabulary and the one-launch
    sequential Markov sampling against their CPU statements."""
    torch.manual_seed(21)
    B, N, V, Rk, K = 3, 5, 129280, 256, 512
    base = (torch.randn(B * N, V, device=dev()) * 3).to(BF16)
    ci, cv = S.topk_candidates(base, K)
    ri, rv = S.topk_candidates(base.cpu(), K)
    assert ci.shape == (B * N, K) and int(ci.min()) >= 0 and int(ci.max()) < V
    # same value multiset (ties at the threshold may pick different ids of equal value)
    assert torch.equal(cv.sort(-1).values.cpu(), rv.sort(-1).values)
    assert torch.equal(base.float().gather(1, ci.long()), cv)
    w1 = (torch.randn(V, Rk, device=dev()) * 0.3).to(BF16)
    w2 = (torch.randn(V, Rk, device=dev()) * 0.3).to(BF16)
    anchors = torch.randint(0, V, (B,), device=dev())
    temp = torch.tensor([0.6, 0.0, 1.0], device=dev())
    seed = torch.tensor([11, 2 ** 41 + 5, 3], device=dev(), dtype=torch.int64)
    pos = torch.tensor([100, 32768, 7], device=dev(), dtype=torch.int64)
    got = S.markov_chain(ci.view(B, N, K), cv.view(B, N, K), anchors, w1, w2, temp, seed, pos)
    ref = S.markov_chain(ci.view(B, N, K).cpu(), cv.view(B, N, K).cpu(), anchors.cpu(), w1.cpu(), w2.cpu(), temp.cpu(),
                         seed.cpu(), pos.cpu())
    assert got.shape == (B, N)
    assert torch.equal(got[:, 0].cpu(), ref[:, 0])                       # first position: same inputs on both sides
    assert (got.cpu() == ref).float().mean().item() >= 0.8              # later ones depend on earlier draws
    # every drawn token is one of its position's candidates
    for b in range(B):
        for i in range(N):
            assert int(got[b, i]) in set(ci.view(B, N, K)[b, i].tolist())
