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
