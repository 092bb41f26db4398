"""Expert-parallel MoE layer over NVLink peer memory (distinct tokens per rank).

`EpMoE.forward(x, ids, weights, experts, shared)` runs route -> dispatch -> grouped FC1 (+SwiGLU) ->
grouped FC2 -> return -> combine with this library's kernels only (`csrc/ep_moe.cu`,
`csrc/moe_grouped.cu`): token rows travel once over NVLink, straight into their final row of the owner's
expert-sorted matrix; the FC1 kernel starts an expert as soon as its rows have landed; results travel
back once.  `forward_nccl` is the baseline the microbenchmark compares against: all_to_all_single for
dispatch and combine around the same grouped GEMMs.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.moe import ExpertWeights
from .symm import SymmetricHeap

BF16 = torch.bfloat16
I32 = torch.int32


def pick_bt(avg_rows: float) -> int:
    return 16 if avg_rows <= 8 else 32 if avg_rows <= 24 else 64 if avg_rows <= 48 else 128


class EpMoE:
    def __init__(self, comm, num_experts: int, topk: int, hidden: int, inter: int, max_tokens: int, limit: float = 10.0,
                 cap_factor: Optional[float] = None, spin_budget: int = 4_000_000):
        self.comm, self.world, self.rank = comm, comm.world_size, comm.rank
        self.E, self.topk, self.H, self.I, self.limit = num_experts, topk, hidden, inter, limit
        self.e_local = num_experts // self.world
        self.max_pairs = max_tokens * topk
        worst = self.world * self.max_pairs
        # worst case: every pair of every rank lands here; a cap factor trades memory for a checked limit
        self.cap_rows = worst if cap_factor is None else min(worst, int(cap_factor * self.max_pairs) + 128)
        L = _lib.lib()
        L.stk_ep_region_bytes.restype = ctypes.c_longlong
        nbytes = L.stk_ep_region_bytes(self.world, self.E, self.e_local, hidden, ctypes.c_longlong(self.cap_rows),
                                       ctypes.c_longlong(self.max_pairs))
        self.heap = SymmetricHeap(comm, int(nbytes))
        self.ctx = (ctypes.c_ubyte * L.stk_ep_ctx_size())()
        bases = (ctypes.c_longlong * self.world)(*self.heap.bases)
        if L.stk_ep_ctx_fill(self.ctx, bases, self.rank, self.world, self.E, topk, hidden, ctypes.c_longlong(self.cap_rows),
                             ctypes.c_longlong(self.max_pairs), spin_budget) != 0:
            raise RuntimeError("expert-parallel context rejected")
        L.stk_ep_ctx_offset.restype = ctypes.c_longlong
        self.off_xs = L.stk_ep_ctx_offset(self.ctx, 0)
        self.off_arrived = L.stk_ep_ctx_offset(self.ctx, 1)
        dev = comm.device
        self.offsets = torch.zeros(self.e_local + 1, dtype=I32, device=dev)
        self.dest_base = torch.zeros(self.E, dtype=I32, device=dev)
        self.cursor = torch.zeros(self.E, dtype=I32, device=dev)
        self.act = torch.zeros(self.cap_rows + 256, inter, dtype=torch.float16, device=dev)
        self.y = torch.empty(self.cap_rows + 256, hidden, dtype=BF16, device=dev)
        self.spin_budget = spin_budget
        comm.barrier()

    def forward(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ew: ExpertWeights,
                shared: Optional[torch.Tensor] = None, bt: Optional[int] = None) -> torch.Tensor:
        t, h = x.shape
        n_pairs = t * self.topk
        assert n_pairs <= self.max_pairs and h == self.H and ids.dtype == I32 and ew.is_fp4
        st, status = _lib.stream(), _lib.status_buffer()
        ctx = self.ctx
        _lib.call("stk_ep_route", ctx, ids, n_pairs, self.offsets, self.dest_base, self.cursor, status, st)
        _lib.call("stk_ep_dispatch", ctx, x, x.stride(0), ids, n_pairs, self.dest_base, self.cursor, status, st)
        if bt is None:
            bt = pick_bt(n_pairs * self.world / self.E)
        xs = ctypes.c_void_p(self.heap.local + self.off_xs)
        arrived = ctypes.c_void_p(self.heap.local + self.off_arrived)
        rows = self.cap_rows + 256
        _lib.call("stk_moe_grouped_ep", xs, rows, ew.w13, ew.s13, ew.g13, self.offsets, self.e_local, self.I, h, self.act, 1,
                  float(self.limit), bt, status, _lib.sm_count(), arrived, self.spin_budget, st)
        _lib.call("stk_moe_grouped", self.act, rows, ew.w2, ew.s2, ew.g2, self.offsets, self.e_local, h, self.I, self.y, 0,
                  0.0, bt, status, _lib.sm_count(), st)
        _lib.call("stk_ep_return", ctx, self.y, self.offsets, min(self.cap_rows, self.world * n_pairs), status, st)
        out = torch.empty(t, h, dtype=BF16, device=x.device)
        _lib.call("stk_ep_combine", ctx, weights, ids, shared, shared.stride(0) if shared is not None else 0, out,
                  out.stride(0), t, status, st)
        return out

    # ---- baseline: NCCL all-to-all around the same grouped GEMMs ----------------------------------
    def forward_nccl(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ew: ExpertWeights,
                     shared: Optional[torch.Tensor] = None, bt: Optional[int] = None) -> torch.Tensor:
        t, h = x.shape
        k, w, el = self.topk, self.world, self.e_local
        dev = x.device
        flat = ids.reshape(-1).long()
        order = torch.argsort(flat, stable=True)                     # pairs sorted by global expert = by owner, expert
        counts_e = torch.bincount(flat, minlength=self.E)
        send_counts = counts_e.view(w, el).sum(1)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.comm.group)
        counts_all = torch.empty(w, self.E, dtype=counts_e.dtype, device=dev)
        dist.all_gather_into_tensor(counts_all.view(-1), counts_e, group=self.comm.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()          # host sync: part of what the baseline costs
        send_x = x.index_select(0, order // k).to(torch.float16)
        recv_x = torch.empty(sum(rc), h, dtype=torch.float16, device=dev)
        dist.all_to_all_single(recv_x, send_x, rc, sc, group=self.comm.group)
        # received rows are (source, expert)-ordered; the grouped GEMM wants expert-major
        mine = counts_all[:, self.rank * el:(self.rank + 1) * el]    # [src, local expert]
        src_expert = torch.repeat_interleave(torch.arange(el, device=dev).repeat(w), mine.reshape(-1))
        perm = torch.argsort(src_expert, stable=True)
        n = recv_x.shape[0]
        xs = torch.zeros(n + 256, h, dtype=torch.float16, device=dev)
        xs[:n] = recv_x.index_select(0, perm)
        offsets = torch.zeros(el + 1, dtype=I32, device=dev)
        offsets[1:] = mine.sum(0).cumsum(0).to(I32)
        if bt is None:
            bt = pick_bt(t * k * w / self.E)
        act = torch.zeros(n + 256, self.I, dtype=torch.float16, device=dev)
        y = torch.empty(n + 256, h, dtype=BF16, device=dev)
        st, status = _lib.stream(), _lib.status_buffer()
        _lib.call("stk_moe_grouped", xs, n + 256, ew.w13, ew.s13, ew.g13, offsets, el, self.I, h, act, 1, float(self.limit), bt,
                  status, _lib.sm_count(), st)
        _lib.call("stk_moe_grouped", act, n + 256, ew.w2, ew.s2, ew.g2, offsets, el, h, self.I, y, 0, 0.0, bt, status,
                  _lib.sm_count(), st)
        back = torch.empty(n, h, dtype=BF16, device=dev)
        back[perm] = y[:n]
        ret = torch.empty(t * k, h, dtype=BF16, device=dev)
        dist.all_to_all_single(ret, back, sc, rc, group=self.comm.group)
        pairs = torch.empty(t * k, h, dtype=BF16, device=dev)
        pairs[order] = ret
        out = (pairs.view(t, k, h).float() * weights.view(t, k, 1)).sum(1)
        if shared is not None:
            out = out + shared.float()
        return out.to(BF16)

    def close(self) -> None:
        self.heap.close()
