"""The allocation-free GEMM entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory when they call it (a callback inside
another runtime, a loop with a fixed memory budget), so `stk_gemm_noalloc` keeps its split-K scratch
in an array built into the library.  This test loads the symbol with ctypes, runs it twice in a row
(the second call reuses the scratch the first one left behind) and compares each result with the
regular entry point, which gets its workspace from the caller.  It is collected last so that a run
that stops at the first failure has already exercised everything else.
"""
import ctypes

import pytest
import torch

from stkernel_b200.ops import _lib
from stkernel_b200.ops import functional as Fn

pytestmark = pytest.mark.gpu


def _call_noalloc(L, w, x, out, splits, status):
    t, k = x.shape
    n = w.shape[0]
    return L.stk_gemm_noalloc(w.data_ptr(), w.stride(0), x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), t, n,
                              k, 0, 1 if out.dtype == torch.float32 else 0, None, 0, None, 0, splits,
                              status.data_ptr(), _lib.sm_count(), _lib.stream())


def test_noalloc_gemm_matches_regular_entry_point_twice():
    dev = torch.device("cuda:0")
    L = _lib.lib()
    assert L.stk_gemm_noalloc_max_workspace_bytes() == 8 << 20
    torch.manual_seed(0)
    status = _lib.status_buffer()
    for call, (t, n, k, splits) in enumerate([(8, 2048, 4096, 4), (16, 4096, 8192, 8)]):
        x = torch.randn(t, k, device=dev).to(torch.bfloat16)
        w = torch.randn(n, k, device=dev).to(torch.bfloat16)
        ref = Fn.linear(x, Fn.LinearWeight(w), out_dtype=torch.float32, splits=splits)     # caller-provided workspace
        out = torch.empty(t, n, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = _call_noalloc(L, w, x, out, splits, status)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        _lib.check_status()
        err = ((out - ref).norm() / ref.norm()).item()
        assert err < 1e-2, (call, err)
        exact = x.float() @ w.float().t()
        assert ((out - exact).norm() / exact.norm()).item() < 1e-2


def test_noalloc_gemm_rejects_oversized_problems():
    dev = torch.device("cuda:0")
    L = _lib.lib()
    x = torch.randn(128, 4096, device=dev).to(torch.bfloat16)
    w = torch.randn(8192, 4096, device=dev).to(torch.bfloat16)
    out = torch.empty(128, 8192, dtype=torch.float32, device=dev)
    # 4 splits x 128 x 8192 x 4 bytes = 16 MiB > 8 MiB of built-in scratch
    assert _call_noalloc(L, w, x, out, 4, _lib.status_buffer()) == -32
    # without split-K no scratch is needed and the same problem runs
    assert _call_noalloc(L, w, x, out, 1, _lib.status_buffer()) == 0
    torch.cuda.synchronize()
    ref = x.float() @ w.float().t()
    assert ((out - ref).norm() / ref.norm()).item() < 1e-2


def test_noalloc_back_to_back_calls_share_the_scratch_in_stream_order():
    """Two calls of different shapes queued on one stream with no synchronisation between them: the second
    overwrites the partials and reuses the counters the first one left at zero, and both results must hold."""
    dev = torch.device("cuda:0")
    L = _lib.lib()
    torch.manual_seed(2)
    status = _lib.status_buffer()
    cases = [(8, 2048, 4096, 4), (16, 1024, 8192, 8)]
    xs = [torch.randn(t, k, device=dev).to(torch.bfloat16) for t, n, k, s in cases]
    ws = [torch.randn(n, k, device=dev).to(torch.bfloat16) for t, n, k, s in cases]
    outs = [torch.empty(t, n, dtype=torch.float32, device=dev) for t, n, k, s in cases]
    torch.cuda.synchronize()
    for (t, n, k, s), x, w, o in zip(cases, xs, ws, outs):
        assert _call_noalloc(L, w, x, o, s, status) == 0
    torch.cuda.synchronize()
    _lib.check_status()
    for x, w, o in zip(xs, ws, outs):
        ref = x.float() @ w.float().t()
        assert ((o - ref).norm() / ref.norm()).item() < 1e-2
    assert L.stk_gemm_noalloc_reset(_lib.stream()) == 0       # harmless when the counters are already zero
    torch.cuda.synchronize()
    o2 = torch.empty_like(outs[0])
    assert _call_noalloc(L, ws[0], xs[0], o2, cases[0][3], status) == 0
    torch.cuda.synchronize()
    assert torch.equal(o2, outs[0])


def test_noalloc_rejects_more_tiles_than_counters():
    dev = torch.device("cuda:0")
    L = _lib.lib()
    # 4100 feature tiles of 128 rows with K = 256 (two splits): the partials fit the 8 MiB, the tile count does not
    n = 4100 * 128
    x = torch.zeros(1, 256, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(n, 256, dtype=torch.bfloat16, device=dev)
    out = torch.empty(1, n, dtype=torch.float32, device=dev)
    assert _call_noalloc(L, w, x, out, 2, _lib.status_buffer()) == -33


def test_noalloc_fp8_splitk_matches_regular_entry_point():
    dev = torch.device("cuda:0")
    L = _lib.lib()
    torch.manual_seed(5)
    t, n, k, splits = 16, 2048, 4096, 4
    x = torch.randn(t, k, device=dev).to(torch.bfloat16)
    lw = Fn.LinearWeight.from_master(torch.randn(n, k, device=dev) * 0.05, "fp8", dev)
    xa = Fn.quant_act(x, "noalloc.fp8")
    ref = Fn.linear(xa, lw, out_dtype=torch.float32, splits=splits)
    out = torch.empty(t, n, dtype=torch.float32, device=dev)
    rc = L.stk_gemm_noalloc(lw.w.data_ptr(), lw.w.stride(0), xa.q.data_ptr(), xa.q.stride(0), out.data_ptr(), out.stride(0),
                            t, n, k, 1, 1, lw.scale.data_ptr(), lw.scale.stride(0), xa.scale.data_ptr(), xa.scale.stride(0),
                            splits, _lib.status_buffer().data_ptr(), _lib.sm_count(), _lib.stream())
    assert rc == 0, rc
    torch.cuda.synchronize()
    _lib.check_status()
    assert ((out - ref).norm() / ref.norm()).item() < 1e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_splitk_output_with_odd_row_stride_takes_element_stores(dtype):
    """An output view whose row stride is not a multiple of the vector width (ldo = N + 1) through the allocation-free
    symbol: the reduction must fall back to element stores and still match the fp32 product."""
    dev = torch.device("cuda:0")
    L = _lib.lib()
    torch.manual_seed(6)
    t, n, k, splits = 8, 1024, 4096, 4
    x = torch.randn(t, k, device=dev).to(torch.bfloat16)
    w = torch.randn(n, k, device=dev).to(torch.bfloat16)
    buf = torch.zeros(t, n + 1, dtype=dtype, device=dev)
    out = buf[:, :n]
    assert _call_noalloc(L, w, x, out, splits, _lib.status_buffer()) == 0
    torch.cuda.synchronize()
    _lib.check_status()
    ref = x.float() @ w.float().t()
    assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2
    assert float(buf[:, n].abs().max()) == 0.0
