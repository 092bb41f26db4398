"""Symmetric peer memory (CUDA IPC over NVLink) and the all-reduce kernels that use it.

Bootstrap mirrors the reference's one-shot shim (overlay/dsv4_oneshot_shim.py:62-122): exchange
handles with ``all_gather_object``, run a lock-step self-test against the library collective, and
on any failure fall back to NCCL permanently.  The data path differs: kernels store directly into
peer HBM and spin (bounded) on epoch flags; a timed-out wait sets a device status word that the
host reads after the step, upon which this path disables itself.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib

_MB = 1 << 20


class LLExchange:
    """Receive slots + epoch counters of the all-reduce that is folded into its producer and consumer kernels
    (csrc/symm.cuh, `LLAr`): a row-parallel layer's kernel stores its partial result into every rank's slot, the
    next kernel adds the ranks.  `ctx` is the descriptor the kernels take by value.

    `words` = capacity per source rank in 8-byte words (two bf16 values each): rows x hidden / 2."""

    def __init__(self, bases: List[int], counters: torch.Tensor, words: int, rank: int, world: int,
                 spin_budget: int = 16_000_000, keep=None):
        L = _lib.lib()
        self.ctx = (ctypes.c_ubyte * L.stk_ll_ctx_size())()
        arr = (ctypes.c_longlong * world)(*bases)
        rc = L.stk_ll_ctx_fill(self.ctx, arr, ctypes.c_void_p(counters.data_ptr()), words, rank, world, spin_budget)
        if rc != 0:
            raise RuntimeError(f"folded all-reduce context rejected ({rc})")
        self.words, self.rank, self.world = words, rank, world
        self.counters = counters
        self._keep = keep

    @staticmethod
    def loopback(device, words: int) -> "LLExchange":
        """A one-rank exchange over local memory: the same kernels and protocol with nothing to add (tests, and the
        single-GPU stand-in for one rank of a group)."""
        buf = torch.zeros(2 * words, dtype=torch.int64, device=device)
        return LLExchange([buf.data_ptr()], torch.zeros(2, dtype=torch.int32, device=device), words, 0, 1, keep=buf)

    def fits(self, t: int, h: int) -> bool:
        return h % 2 == 0 and t * h // 2 <= self.words


def region_layout(world: int, oneshot_bytes: int, twoshot_bytes: int, gemm_bytes: int = 2 * _MB,
                  ll_words: int = 0) -> dict:
    """Byte offsets of the symmetric region (identical on every rank)."""
    off = 0
    lay = {}
    lay["off_flags"] = off
    off += 1 * _MB
    lay["off_epochs"] = off
    off += 256 * 1024
    lay["off_oneshot"] = off
    off += 2 * world * oneshot_bytes
    lay["off_rs"] = off
    chunk = (twoshot_bytes + world - 1) // world
    chunk = (chunk + 15) // 16 * 16
    off += 2 * world * chunk
    off = (off + 255) // 256 * 256
    lay["off_ag"] = off
    off += 2 * twoshot_bytes
    off = (off + 255) // 256 * 256
    lay["off_gemm"] = off
    lay["gemm_bytes"] = gemm_bytes
    off += 2 * world * gemm_bytes
    off = (off + 255) // 256 * 256
    lay["off_ll"] = off
    lay["ll_words"] = ll_words
    off += 2 * world * ll_words * 8
    lay["off_user"] = (off + 255) // 256 * 256
    lay["oneshot_bytes"] = oneshot_bytes
    lay["twoshot_bytes"] = twoshot_bytes
    return lay


class SymmetricHeap:
    """One cudaMalloc'd region per rank, mapped into every peer."""

    def __init__(self, comm, nbytes: int):
        self.comm = comm
        self.nbytes = nbytes
        L = _lib.lib()
        p = ctypes.c_void_p()
        if L.stk_symm_alloc(ctypes.c_longlong(nbytes), ctypes.byref(p)) != 0:
            raise RuntimeError("symmetric allocation failed")
        self.local = p.value
        h = (ctypes.c_ubyte * 64)()
        if L.stk_symm_export(ctypes.c_void_p(self.local), h) != 0:
            raise RuntimeError("cudaIpcGetMemHandle failed")
        handles = comm.all_gather_object(bytes(h))
        self.bases: List[int] = []
        self._opened: List[int] = []
        for r, hb in enumerate(handles):
            if r == comm.rank:
                self.bases.append(self.local)
                continue
            q = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(hb)
            if L.stk_symm_import(buf, ctypes.byref(q)) != 0:
                raise RuntimeError(f"cudaIpcOpenMemHandle failed for rank {r}")
            self.bases.append(q.value)
            self._opened.append(q.value)

    def close(self) -> None:
        L = _lib.lib()
        for q in self._opened:
            L.stk_symm_close(ctypes.c_void_p(q))
        self._opened = []
        if self.local:
            L.stk_symm_free(ctypes.c_void_p(self.local))
            self.local = 0


class SymmetricAllReduce:
    ONESHOT_BLOCKS = 8
    TWOSHOT_BLOCKS = 128

    LL_ROWS, LL_HIDDEN = 64, 8192            # the folded all-reduce holds up to 64 rows of 8192 values per rank

    def __init__(self, comm, max_bytes: int = 64 * _MB, oneshot_bytes: int = 2 * _MB, spin_budget: int = 16_000_000,
                 user_bytes: int = 0):
        self.comm = comm
        self.world = comm.world_size
        if self.world > 8:
            raise RuntimeError("symmetric all-reduce supports at most 8 ranks")
        self.layout = region_layout(self.world, oneshot_bytes, max_bytes, ll_words=self.LL_ROWS * self.LL_HIDDEN // 2)
        self.heap = SymmetricHeap(comm, self.layout["off_user"] + user_bytes)
        L = _lib.lib()
        self.ctx = (ctypes.c_ubyte * L.stk_symm_ctx_size())()
        bases = (ctypes.c_longlong * self.world)(*self.heap.bases)
        lay = self.layout
        rc = L.stk_symm_ctx_fill(self.ctx, bases, comm.rank, self.world, lay["off_flags"], lay["off_epochs"],
                                 lay["off_oneshot"], lay["oneshot_bytes"], lay["off_rs"], lay["off_ag"],
                                 lay["twoshot_bytes"], lay["off_gemm"], lay["gemm_bytes"], spin_budget)
        if rc != 0:
            raise RuntimeError("symmetric context rejected")
        self.oneshot_max = min(comm.oneshot_max_bytes, oneshot_bytes)
        self.twoshot_max = max_bytes
        self.enabled = True
        self.ag_capacity = (user_bytes // 2) // 256 * 256        # two gathered-activation buffers, used alternately
        self._ag_calls = 0
        self.ll_counters = torch.zeros(2, dtype=torch.int32, device=comm.device)
        self.ll = LLExchange([b + lay["off_ll"] for b in self.heap.bases], self.ll_counters, lay["ll_words"], comm.rank,
                             self.world, spin_budget=spin_budget)
        comm.barrier()

    def eligible(self, x: torch.Tensor) -> bool:
        n = x.numel() * x.element_size()
        return (self.enabled and x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and n % 16 == 0
                and x.data_ptr() % 16 == 0 and 0 < n <= self.twoshot_max)

    def all_reduce(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """In-place sum over ranks; returns None when this path is disabled."""
        if not self.enabled:
            return None
        n = x.numel() * x.element_size()
        L = _lib.lib()
        st = _lib.status_buffer()
        if n <= self.oneshot_max:
            # the block count is fixed per kernel kind: all blocks then share one epoch sequence
            rc = L.stk_oneshot_allreduce(self.ctx, x.data_ptr(), x.data_ptr(), n, self.ONESHOT_BLOCKS, st.data_ptr(),
                                         _lib.stream())
            self.comm.calls["oneshot"] += 1
        else:
            rc = L.stk_twoshot_allreduce(self.ctx, x.data_ptr(), x.data_ptr(), n, self.TWOSHOT_BLOCKS, st.data_ptr(),
                                         _lib.stream())
            self.comm.calls["twoshot"] += 1
        if rc != 0:
            raise _lib.KernelError(f"symmetric all-reduce launch returned {rc}")
        _lib.launch_count += 1
        return x

    def reduce_scatter(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """x [world * n, ...] bf16 -> this rank's [n, ...] summed over ranks (own kernel over the two-shot staging
        area); None when this path does not apply."""
        nbytes = x.numel() * x.element_size()
        if (not self.enabled or x.dtype != torch.bfloat16 or not x.is_contiguous() or nbytes > self.twoshot_max
                or x.data_ptr() % 16
                or nbytes % (16 * self.world) or x.shape[0] % self.world):
            return None
        out = torch.empty(x.shape[0] // self.world, *x.shape[1:], dtype=x.dtype, device=x.device)
        rc = _lib.lib().stk_symm_reduce_scatter(self.ctx, x.data_ptr(), out.data_ptr(), nbytes, self.TWOSHOT_BLOCKS,
                                                 _lib.status_buffer().data_ptr(), _lib.stream())
        if rc != 0:
            raise _lib.KernelError(f"symmetric reduce-scatter launch returned {rc}")
        _lib.launch_count += 1
        self.comm.calls["own_rs"] = self.comm.calls.get("own_rs", 0) + 1
        return out

    def all_gather(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """x [n, ...] -> [world * n, ...] rank-major (own kernel); None when this path does not apply."""
        nbytes = x.numel() * x.element_size()
        if (not self.enabled or not x.is_contiguous() or nbytes % 16 or nbytes * self.world > self.twoshot_max
                or nbytes == 0 or x.data_ptr() % 16):
            return None
        out = torch.empty(self.world * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        rc = _lib.lib().stk_symm_all_gather(self.ctx, x.data_ptr(), out.data_ptr(), nbytes, self.TWOSHOT_BLOCKS,
                                             _lib.status_buffer().data_ptr(), _lib.stream())
        if rc != 0:
            raise _lib.KernelError(f"symmetric all-gather launch returned {rc}")
        _lib.launch_count += 1
        self.comm.calls["own_ag"] = self.comm.calls.get("own_ag", 0) + 1
        return out

    def self_test(self) -> None:
        """Lock-step comparison with the library collective at a few sizes; raises on mismatch."""
        dev = self.comm.device
        for numel in (4096 * 6, 4096 * 256, 4096 * 2048):
            if numel * 2 > self.twoshot_max:
                continue
            g = torch.Generator(device=dev).manual_seed(1234 + self.comm.rank)
            x = torch.randn(numel, device=dev, generator=g).to(torch.bfloat16)
            ref = x.float()
            dist.all_reduce(ref, group=self.comm.group)
            for _ in range(3):          # repeated calls exercise both parities
                y = x.clone()
                self.all_reduce(y)
            torch.cuda.synchronize()
            _lib.check_status()
            err = (y.float() - ref).abs().max().item()
            tol = 0.02 * ref.abs().max().item() + 1e-3
            ok = torch.tensor([1 if err <= tol else 0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.comm.group)
            if int(ok.item()) != 1:
                self.enabled = False
                raise RuntimeError(f"symmetric all-reduce self-test diverged at {numel} elements (err {err})")

    def gemm_ctx(self, t: int, n: int):
        """Context for the GEMM-fused all-reduce, or None when the output does not fit its slots."""
        if not self.enabled or t * n * 2 > self.layout["gemm_bytes"] or t > 128 or n % 128:
            return None
        return self.ctx

    AG_BLOCKS = 32

    def ag_gemm(self, x_shard: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """All-gather of row shards fused with a column-parallel GEMM: every rank holds x_shard [T/world, K]
        (bf16) and weight [N_local, K] (bf16); returns x_full @ weight.T as [T, N_local].

        The shard is pushed into every rank's gathered matrix over NVLink (each row crosses a link once);
        the tcgen05 GEMM starts with the tiles of its own shard and waits, tile by tile, only for the shards
        it is about to read.  Two gathered buffers alternate by call, so a rank may start the next push while
        a slower peer still reads the previous one."""
        rows, k = x_shard.shape
        t = rows * self.world
        n = weight.shape[0]
        nbytes = rows * k * 2
        if not (self.enabled and x_shard.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x_shard.is_contiguous()
                and weight.is_contiguous() and nbytes % 16 == 0 and t * k * 2 <= self.ag_capacity):
            raise ValueError("ag_gemm: unsupported operands or gathered matrix larger than the reserved buffers")
        parity = self._ag_calls & 1
        self._ag_calls += 1
        off = self.layout["off_user"] + parity * self.ag_capacity
        st = _lib.status_buffer()
        _lib.call("stk_symm_ag_push", self.ctx, x_shard, nbytes, off, self.AG_BLOCKS, st, _lib.stream())
        if out is None:
            out = torch.empty(t, n, dtype=torch.bfloat16, device=x_shard.device)
        import ctypes as _ct
        _lib.call("stk_gemm_gated", weight, k, _ct.c_void_p(self.heap.local + off), k, out, out.stride(0), t, n, k, 0, 0,
                  None, 0, None, 0, st, _lib.sm_count(), self.ctx, rows, _lib.stream())
        return out

    def ll_exchange(self, t: int, h: int) -> Optional[LLExchange]:
        """The folded all-reduce for a [t, h] activation, or None when this path is off or the slots are too small."""
        if not self.enabled or not self.ll.fits(t, h):
            return None
        return self.ll

    def disable(self, reason: str) -> None:
        self.enabled = False
        self.comm.disabled_reason = reason
