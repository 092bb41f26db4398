"""Tensor-parallel communicator: one rank per GPU.

`all_reduce` picks, per call, between this library's own kernels over symmetric
peer memory (one-shot for small messages, two-shot reduce-scatter + all-gather
for large ones; see :mod:`.symm`) and the NCCL path kept as the measured baseline
and as the fallback when the symmetric heap is unavailable or a kernel reported
a bounded-wait timeout.  Takes the place of the reference's device communicator
and its one-shot all-reduce hook (overlay/cuda_communicator.py:255-327,
overlay/dsv4_oneshot_shim.py:136-162).
"""
from __future__ import annotations

import os

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


class Communicator:
    def __init__(self, group: Optional[dist.ProcessGroup] = None, device=None, use_symm: bool = True,
                 oneshot_max_bytes: int = 512 * 1024, cpu_group: Optional[dist.ProcessGroup] = None,
                 fuse_gemm: bool = True, ag_bytes: int = 0):
        self.group = group if group is not None else dist.group.WORLD
        self.world_size = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.oneshot_max_bytes = oneshot_max_bytes
        self.cpu_group = cpu_group
        self.symm = None
        self.fuse_gemm = fuse_gemm
        self.disabled_reason: Optional[str] = None
        self.calls = {"oneshot": 0, "twoshot": 0, "nccl": 0}
        # sequence-parallel all-gather / reduce-scatter through this library's kernels (STK_OWN_GATHER_SCATTER=0: NCCL)
        self.own_gather_scatter = os.environ.get("STK_OWN_GATHER_SCATTER", "1") != "0"
        if use_symm and self.device.type == "cuda" and self.world_size > 1:
            try:
                from .symm import SymmetricAllReduce
                self.symm = SymmetricAllReduce(self, max_bytes=64 << 20, user_bytes=2 * ag_bytes)
                self.symm.self_test()
            except Exception as e:  # fail closed onto NCCL, permanently
                self.symm = None
                self.disabled_reason = f"{type(e).__name__}: {e}"

        if self.device.type == "cuda" and self.world_size > 1:
            self._warm_up_nccl()

    def _warm_up_nccl(self) -> None:
        """NCCL sets up its point-to-point and ring connections at the first use of each collective kind (seconds for
        all-to-all on 8 GPUs): pay that at start-up, not inside the first large prefill step."""
        w = self.world_size
        x = torch.zeros(w * 8, dtype=torch.bfloat16, device=self.device)
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x, group=self.group)
        big = torch.empty(w * x.numel(), dtype=x.dtype, device=self.device)
        dist.all_gather_into_tensor(big, x, group=self.group)
        small = torch.empty(x.numel() // w, dtype=x.dtype, device=self.device)
        dist.reduce_scatter_tensor(small, x, group=self.group)
        dist.all_reduce(x, group=self.group)
        torch.cuda.synchronize(self.device)

    # ---- collectives -------------------------------------------------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return x
        if self.symm is not None and self.symm.eligible(x):
            out = self.symm.all_reduce(x)
            if out is not None:
                return out
        self.calls["nccl"] += 1
        dist.all_reduce(x, group=self.group)
        return x

    def all_gather_last_dim(self, x: torch.Tensor) -> torch.Tensor:
        """[T, n] per rank -> [T, n * world] (rank-major along the last dim)."""
        if self.world_size == 1:
            return x
        self.calls["nccl"] += 1
        parts = torch.empty(self.world_size * x.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(parts, x.contiguous(), group=self.group)
        return parts.view(self.world_size, x.shape[0], x.shape[1]).permute(1, 0, 2).reshape(x.shape[0], -1)

    def all_gather_dim0(self, x: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return x
        if self.symm is not None and x.is_cuda and self.own_gather_scatter:
            out = self.symm.all_gather(x.contiguous())
            if out is not None:
                return out
        self.calls["nccl"] += 1
        out = torch.empty(self.world_size * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def all_gatherv_dim0(self, x: torch.Tensor, sizes: Sequence[int]) -> torch.Tensor:
        """Ragged all-gather along dim 0 (`sizes[r]` rows from rank r)."""
        if self.world_size == 1:
            return x
        self.calls["nccl"] += 1
        outs = [torch.empty(s, *x.shape[1:], dtype=x.dtype, device=x.device) for s in sizes]
        dist.all_gather(outs, x.contiguous(), group=self.group)
        return torch.cat(outs, 0)

    def reduce_scatter_dim0(self, x: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return x
        assert x.shape[0] % self.world_size == 0
        n = x.shape[0] // self.world_size
        if self.symm is not None and x.is_cuda and self.own_gather_scatter:
            out = self.symm.reduce_scatter(x.contiguous())
            if out is not None:
                return out
        self.calls["nccl"] += 1
        if not x.is_cuda:
            # gloo has no reduce-scatter: sum everywhere, keep this rank's rows
            y = x.contiguous().clone()
            dist.all_reduce(y, group=self.group)
            return y[self.rank * n:(self.rank + 1) * n].contiguous()
        out = torch.empty(n, *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
        return out

    def reduce_scatterv_dim0(self, x: torch.Tensor, sizes: Sequence[int]) -> torch.Tensor:
        if self.world_size == 1:
            return x
        self.calls["nccl"] += 1
        chunks = list(torch.split(x.contiguous(), list(sizes), 0))
        out = torch.empty_like(chunks[self.rank])
        dist.reduce_scatter(out, chunks, group=self.group)
        return out

    def broadcast(self, x: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world_size > 1:
            dist.broadcast(x, src=dist.get_global_rank(self.group, src), group=self.group)
        return x

    def send(self, x: torch.Tensor, dst: int) -> None:
        dist.send(x, dst=dist.get_global_rank(self.group, dst), group=self.group)

    def recv(self, x: torch.Tensor, src: int) -> torch.Tensor:
        dist.recv(x, src=dist.get_global_rank(self.group, src), group=self.group)
        return x

    def all_to_all_dim0(self, x: torch.Tensor, in_sizes: Sequence[int], out_sizes: Sequence[int]) -> torch.Tensor:
        """Expert-parallel dispatch/combine baseline: ragged all-to-all along dim 0."""
        self.calls["nccl"] += 1
        out = torch.empty(sum(out_sizes), *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), list(out_sizes), list(in_sizes), group=self.group)
        return out

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier(group=self.group)

    def all_gather_object(self, obj) -> List:
        g = self.cpu_group if self.cpu_group is not None else self.group
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=g)
        return out
