"""Guard paths on the GPU: a bounded wait that runs out reports a status and leaves the context usable;
out-of-range ids and padding rows are skipped and reported, never dereferenced.  Nothing here faults,
traps or hangs: the timeout is a local flag that nothing sets, with a budget of a few milliseconds, and the
bad ids exercise the checks that the source audit (`fleet/audit_guards.py`) proves are in the kernels."""
import pytest
import torch

from stkernel_b200.ops import _lib
from stkernel_b200.ops import attention as A
from stkernel_b200.ops import cache as C
from stkernel_b200.ops import functional as Fn
from stkernel_b200.ops import moe as M

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def dev():
    return torch.device("cuda:0")


def _expect_status(code: int):
    torch.cuda.synchronize()
    with pytest.raises(_lib.KernelError, match=f"device status {code}"):
        _lib.check_status()
    _lib.check_status()                                   # cleared: the next check passes


def test_bounded_wait_times_out_with_status_and_context_survives():
    flag = torch.zeros(4, dtype=torch.int32, device=dev())      # nothing ever writes this flag
    _lib.call("stk_flag_timeout_probe", flag, 1, 20000, _lib.status_buffer(), _lib.stream())
    _expect_status(4)                                           # local flag wait timed out
    # the same wait passes when the flag is already there
    flag.fill_(1)
    _lib.call("stk_flag_timeout_probe", flag, 1, 20000, _lib.status_buffer(), _lib.stream())
    torch.cuda.synchronize()
    _lib.check_status()
    # the context is intact: a real kernel still runs and is right
    x = torch.randn(8, 256, device=dev()).to(BF16)
    w = torch.ones(256, device=dev()).to(BF16)
    y = Fn.rms_norm(x, w, 1e-6)
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    assert (y.float() - ref).abs().max().item() < 3e-2


def test_embedding_rejects_out_of_range_token_ids():
    V, H, hc = 100, 64, 4
    emb = torch.randn(V, H, device=dev()).to(BF16)
    ids = torch.tensor([3, V, -1, 99], device=dev(), dtype=torch.int64)
    out = Fn.embed_hc(ids, emb, hc, V)
    _expect_status(3)                                           # index out of range, reported not dereferenced
    assert torch.equal(out[0, 0], emb[3]) and torch.equal(out[3, 2], emb[99])
    assert out[1].abs().sum().item() == 0 and out[2].abs().sum().item() == 0


def test_cache_insert_skips_padding_and_rejects_bad_slots():
    T, D, R_ = 6, 512, 64
    cache = C.PagedCache.allocate(2, D, R_, True, "latent", dev())
    before = cache.buf.clone()
    kv = torch.randn(T, D, device=dev()).to(BF16)
    pos = torch.arange(T, device=dev())
    inv = Fn.inv_freq(R_, 10000.0, dev())
    slots = torch.full((T,), -1, device=dev(), dtype=torch.int64)           # all padding: nothing is written
    C.kv_rope_quant_insert(kv, pos, slots, inv, cache)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(cache.buf, before)
    slots[2] = cache.num_slots + 5                                           # past the pool
    slots[4] = 7
    C.kv_rope_quant_insert(kv, pos, slots, inv, cache)
    _expect_status(3)
    rows = C.kv_gather_dequant(cache, torch.tensor([7, -1], device=dev(), dtype=torch.int64))
    assert rows[0].abs().sum().item() > 0 and rows[1].abs().sum().item() == 0


def test_router_hash_table_and_expert_ids_are_bounded():
    T, E, k = 5, 16, 2
    logits = torch.randn(T, E, device=dev())
    table = torch.randint(0, E, (50, k), dtype=torch.int32, device=dev())
    table[7, 1] = E + 3                                                      # corrupt table entry
    toks = torch.tensor([1, 7, 50, -2, 3], device=dev())                      # 50 and -2 are outside the table
    ids, w = M.router(logits, None, k, "sigmoid", True, 1.0, table, toks)
    torch.cuda.synchronize()
    assert int(ids.min()) >= 0 and int(ids.max()) < E                        # every emitted id is a valid expert
    assert torch.isfinite(w).all()
    # experts outside the local range are skipped by the expert kernels
    H, I = 256, 128
    ew = M.ExpertWeights.from_master(torch.randn(E, 2 * I, H) * 0.02, torch.randn(E, H, I) * 0.02, "nvfp4", dev())
    x = torch.randn(T, H, device=dev()).to(BF16)
    bad = ids.clone()
    bad[0, 0] = E + 9
    bad[1, 1] = -4
    out = M.moe_experts(x, bad, w, ew, 10.0)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    _lib.status_buffer().zero_()


def test_index_builders_handle_padding_and_empty_rows():
    # padding tokens (request -1, position -1) get empty windows; a zero-length top-k row stays empty
    positions = torch.tensor([5, -1, 0, 130], device=dev(), dtype=torch.int64)
    tok_req = torch.tensor([0, -1, 1, 0], device=dev(), dtype=torch.int32)
    table = torch.full((2, 4), -1, dtype=torch.int32, device=dev())
    table[0, :3] = torch.tensor([2, 0, 1])
    table[1, 0] = 3
    slots, lens = A.swa_indices(positions, tok_req, table, 128)
    torch.cuda.synchronize()
    assert lens.tolist() == [6, 0, 1, 128]
    assert int(slots[0, 0]) == 2 * 64 + 0 and int(slots[2, 0]) == 3 * 64
    assert (slots[1] == -1).all()
    nv = A.compressed_valid(positions, 4)
    assert nv.tolist() == [1, 0, 0, 32]
    scores = torch.randn(4, 64, device=dev())
    out = torch.full((4, 8), -7, dtype=torch.int32, device=dev())
    A.topk_rows(scores, nv, 8, out=out)
    torch.cuda.synchronize()
    assert (out[1] == -1).all() and (out[2] == -1).all()
    assert int((out[0] >= 0).sum()) == 1 and int((out[3] >= 0).sum()) == 8
    _lib.check_status()
