"""Hybrid paged KV manager.

Several cache *groups* share one page-id space per group kind:

* ``swa``   — every layer's sliding-window latent cache (64-token pages).  Only the
  pages that still intersect a request's window are kept; older ones are released
  as the request advances, so SWA memory is O(window), not O(context).
* ``c4``    — compressed latent cache + indexer-K cache of every ratio-4 layer
  (one row per 4 tokens).
* ``c128``  — compressed latent cache of every ratio-128 layer.
* compressor *state* rows (raw value/gate rows of the open window) live in a
  dense per-request-row tensor owned by each layer.

Each group has a free list and a per-request block table row
(``[max_requests, max_pages]`` int32, -1 = no page) that lives on the device at a
fixed address, so captured CUDA graphs keep working while tables change.
This is the engine-side counterpart of the KV specs and slot mappings the
reference builds on (overlay/attention.py:743-759,836-849,
overlay/sparse_swa_dsv4.py:87-111).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..config import ModelConfig
from ..ops.cache import PAGE, PagedCache
from .planning import dcp_owner


class OutOfPages(RuntimeError):
    pass


@dataclass
class GroupTable:
    """Free list + device block table of one cache group."""
    name: str
    num_pages: int
    max_requests: int
    max_pages_per_req: int
    device: torch.device
    rows_per_token: float            # 1 for swa, 1/ratio for compressed groups
    # Decode context parallel: logical page lp of every request is stored by rank lp % dcp_size only.  The other
    # ranks map it to one shared scratch page past the pool (`trash`), so kernels that write a compressed row through
    # the table need no owner test, and nothing ever reads that page.
    dcp_rank: int = 0
    dcp_size: int = 1
    table_host: torch.Tensor = field(init=False)
    table_dev: torch.Tensor = field(init=False)
    free: List[int] = field(init=False)
    dirty: bool = field(default=True, init=False)
    on_pressure: Optional[Callable[[], bool]] = field(default=None, init=False)

    def __post_init__(self) -> None:
        self.table_host = torch.full((self.max_requests, self.max_pages_per_req), -1, dtype=torch.int32)
        if self.device.type == "cuda":
            self.table_host = self.table_host.pin_memory()
        self.table_np = self.table_host.numpy()          # host truth; never read by an async copy
        # upload snapshots: the DMA of step k may run while the host already edits the table for step
        # k+1, so rows are copied into one of two pinned snapshots and uploaded from there
        self.snap = [torch.full_like(self.table_host, -1) for _ in range(2)]
        if self.device.type == "cuda":
            self.snap = [t.pin_memory() for t in self.snap]
        self.snap_np = [t.numpy() for t in self.snap]
        self.table_dev = torch.full((self.max_requests, self.max_pages_per_req), -1, dtype=torch.int32,
                                    device=self.device)
        self.free = list(range(self.num_pages - 1, -1, -1))
        # owners per physical page: a request row, and any number of prefix-cache entries sharing it
        self.ref = [0] * self.num_pages
        # resident logical pages of each row form one interval [lo, hi)
        self.lo = [0] * self.max_requests
        self.hi = [0] * self.max_requests
        self.dirty_rows = set()
        self.trash = self.num_pages if self.dcp_size > 1 else -2          # physical id of the scratch page

    def owns(self, logical: int) -> bool:
        return self.dcp_size == 1 or dcp_owner(logical * PAGE, self.dcp_size, PAGE) == self.dcp_rank

    def local_table(self) -> torch.Tensor:
        """[max_requests, ceil(max_pages / dcp)] block table over this rank's own pages only: column l is logical
        page l * dcp_size + dcp_rank.  Row r of that local numbering is global row
        ((r // PAGE) * dcp_size + dcp_rank) * PAGE + r % PAGE."""
        return self.table_dev[:, self.dcp_rank::self.dcp_size].contiguous()

    def ensure(self, row: int, first_logical: int, last_logical: int) -> None:
        """Make logical pages [first, last] of request `row` resident (the resident set stays an interval)."""
        if last_logical >= self.max_pages_per_req:
            raise OutOfPages(f"{self.name}: request needs logical page {last_logical} >= {self.max_pages_per_req}")
        first_logical = max(first_logical, 0)
        if self.hi[row] == self.lo[row]:
            self.lo[row] = self.hi[row] = first_logical
        t = self.table_np[row]
        start = max(self.hi[row], first_logical)
        if first_logical < self.lo[row]:
            raise OutOfPages(f"{self.name}: page {first_logical} of row {row} was already released")
        for lp in range(start, last_logical + 1):
            if self.owns(lp):
                while not self.free and self.on_pressure is not None and self.on_pressure():
                    pass                                   # cached prefixes give pages back, oldest first
                if not self.free:
                    # the pages taken so far stay with the row (the interval below covers them): nothing leaks
                    raise OutOfPages(f"{self.name}: pool of {self.num_pages} pages exhausted")
                t[lp] = self.free.pop()
                self.ref[int(t[lp])] = 1
            else:
                t[lp] = self.trash
            self.hi[row] = lp + 1
            self.dirty = True
            self.dirty_rows.add(row)

    def release_before(self, row: int, logical: int) -> None:
        t = self.table_np[row]
        end = min(max(logical, 0), self.hi[row])
        for lp in range(self.lo[row], end):
            self.unref(int(t[lp]))
            t[lp] = -1
        if end > self.lo[row]:
            self.lo[row] = end
            self.dirty = True
            self.dirty_rows.add(row)

    def unref(self, page: int) -> None:
        if page == self.trash:
            return
        self.ref[page] -= 1
        if self.ref[page] == 0:
            self.free.append(page)

    def share(self, row: int, first_logical: int, last_logical: int) -> List[int]:
        """Physical pages of logical pages [first, last] of `row`, each with one more owner."""
        t = self.table_np[row]
        pages = [int(t[lp]) for lp in range(first_logical, last_logical + 1)]
        if any(pg < 0 for pg in pages):
            raise OutOfPages(f"{self.name}: cannot share a page that is not resident")
        for pg in pages:
            if pg != self.trash:
                self.ref[pg] += 1
        return pages

    def adopt(self, row: int, first_logical: int, pages: List[int]) -> None:
        """Map shared physical pages as logical pages [first, first + len) of an empty row."""
        assert self.hi[row] == self.lo[row], "adopt needs a row without resident pages"
        t = self.table_np[row]
        for i, pg in enumerate(pages):
            t[first_logical + i] = pg
            if pg != self.trash:
                self.ref[pg] += 1
        self.lo[row], self.hi[row] = first_logical, first_logical + len(pages)
        self.dirty = True
        self.dirty_rows.add(row)

    def release_all(self, row: int) -> None:
        self.release_before(row, self.max_pages_per_req)
        self.lo[row] = self.hi[row] = 0

    def sync(self, parity: int = 0) -> None:
        """Upload the rows that changed since the last step (through pinned snapshot `parity`, which
        the caller guarantees is no longer being read by an earlier upload)."""
        if self.dirty:
            snap, snap_np = self.snap[parity], self.snap_np[parity]
            if len(self.dirty_rows) * 4 >= self.max_requests:
                snap_np[:] = self.table_np
                self.table_dev.copy_(snap, non_blocking=True)
            else:
                for r in self.dirty_rows:
                    snap_np[r] = self.table_np[r]
                    self.table_dev[r].copy_(snap[r], non_blocking=True)
            self.dirty_rows.clear()
            self.dirty = False

    @property
    def pages_in_use(self) -> int:
        return self.num_pages - len(self.free)

    def held(self, row: int) -> int:
        """Pool pages behind the resident logical pages of `row` (with context parallelism: this rank's only)."""
        n, r = self.dcp_size, self.dcp_rank
        below = lambda x: (x - r + n - 1) // n if x > r else 0         # logical pages < x that this rank stores
        return below(self.hi[row]) - below(self.lo[row])


class KVManager:
    """Owns the group tables, the per-layer cache tensors and the request-row allocator."""

    def __init__(self, cfg: ModelConfig, device, max_requests: int, max_model_len: int, swa_pages: int,
                 c4_pages: int, c128_pages: int = 0, max_chunk: int = 4096, layers: Optional[List[int]] = None,
                 extra_swa_layers: int = 0, spec_tokens: int = 0, dcp_rank: int = 0, dcp_size: int = 1):
        """dcp_size > 1: the ratio-4 caches (compressed latent rows and indexer keys, the part of the KV that grows
        with the context) are dealt page by page over the ranks; `c4_pages` is then this rank's pool.  The
        sliding-window and ratio-128 caches stay replicated (a window, and 1/32 of the ratio-4 rows)."""
        self.cfg = cfg
        self.dcp_rank, self.dcp_size = dcp_rank, dcp_size
        self.device = torch.device(device)
        self.max_requests = max_requests
        fp8 = cfg.kv_cache_dtype == "fp8_ds_mla"
        D, Rd = cfg.head_dim, cfg.qk_rope_head_dim
        # the block table spans the whole context; SWA residency is bounded by window + chunk
        pages_ctx = (max_model_len + PAGE - 1) // PAGE + 1
        self.swa = GroupTable("swa", swa_pages, max_requests, pages_ctx, self.device, 1.0)
        self.c4 = GroupTable("c4", max(c4_pages, 1), max_requests, (max_model_len // 4) // PAGE + 2, self.device, 0.25,
                             dcp_rank, dcp_size)
        self.c128 = GroupTable("c128", max(c128_pages, 1), max_requests, (max_model_len // 128) // PAGE + 2,
                               self.device, 1 / 128)
        self.layers = layers if layers is not None else list(range(cfg.num_hidden_layers))
        self.model_has_c4 = any(cfg.layer_kind(l) == "c4a" for l in range(cfg.num_hidden_layers))
        self.model_has_c128 = any(cfg.layer_kind(l) == "c128a" for l in range(cfg.num_hidden_layers))
        self.swa_cache: Dict[int, PagedCache] = {}
        self.comp_cache: Dict[int, PagedCache] = {}
        self.idx_cache: Dict[int, PagedCache] = {}
        self.comp_state: Dict[int, torch.Tensor] = {}
        self.idx_state: Dict[int, torch.Tensor] = {}
        n_total = cfg.num_hidden_layers + extra_swa_layers
        # Speculative verification writes up to `spec_tokens` raw compressor rows past the accepted
        # prefix; the rings are widened so that those writes never land on a row that a window
        # closing after the rollback still needs.
        ring4 = 8 if spec_tokens == 0 else 32
        ring128 = 128 if spec_tokens == 0 else 160
        for li in list(self.layers) + list(range(cfg.num_hidden_layers, n_total)):
            self.swa_cache[li] = PagedCache.allocate(swa_pages, D, Rd, fp8, "latent", self.device)
            kind = cfg.layer_kind(li) if li < cfg.num_hidden_layers else "swa"
            if kind == "c4a":
                n4 = self.c4.num_pages + (1 if dcp_size > 1 else 0)          # + the scratch page
                self.comp_cache[li] = PagedCache.allocate(n4, D, Rd, fp8, "latent", self.device)
                self.idx_cache[li] = PagedCache.allocate(n4, cfg.index_head_dim, Rd, fp8, "indexer", self.device,
                                                         fp4=cfg.indexer_dtype == "mxfp4")
                self.comp_state[li] = torch.zeros(max_requests, ring4, 2 * 2 * D, dtype=torch.float32, device=self.device)
                self.idx_state[li] = torch.zeros(max_requests, ring4, 2 * 2 * cfg.index_head_dim, dtype=torch.float32,
                                                 device=self.device)
            elif kind == "c128a":
                self.comp_cache[li] = PagedCache.allocate(self.c128.num_pages, D, Rd, fp8, "latent", self.device)
                self.comp_state[li] = torch.zeros(max_requests, ring128, 2 * D, dtype=torch.float32, device=self.device)
        self.free_rows = list(range(max_requests - 1, -1, -1))
        self.spec_tokens = spec_tokens
        # ratio-4 pages promised to admitted requests for their whole context (allocated page by page as they grow):
        # admission counts the part not yet allocated as taken, so a pool smaller than max_requests x max_model_len
        # makes requests wait instead of running out of pages in the middle of a step
        self.reserved: Dict[int, int] = {}

    # ---- request rows -------------------------------------------------------
    def alloc_row(self) -> int:
        if not self.free_rows:
            raise OutOfPages("no free request row")
        return self.free_rows.pop()

    def free_row(self, row: int) -> None:
        for g in (self.swa, self.c4, self.c128):
            g.release_all(row)
        self.reserved.pop(row, None)
        self.free_rows.append(row)

    def reserve(self, row: int, context: int) -> None:
        """Promise request `row` the ratio-4 pages of a context of `context` tokens."""
        self.reserved[row] = self.admit_needs(0, context)[1]

    def promised(self) -> int:
        """Ratio-4 pages promised to running requests and not allocated yet."""
        return sum(max(0, need - self.c4.held(row)) for row, need in self.reserved.items())

    # ---- per-step residency ---------------------------------------------------
    def prepare(self, row: int, start_pos: int, n_tokens: int, lookback: Optional[int] = None) -> None:
        """Make resident what a step that appends positions [start, start+n) to request `row` touches,
        and release SWA pages that have left the window."""
        cfg = self.cfg
        W = cfg.sliding_window if lookback is None else lookback
        end = start_pos + n_tokens                 # exclusive
        lo = max(0, start_pos - W + 1)
        self.swa.release_before(row, lo // PAGE)
        self.swa.ensure(row, lo // PAGE, (end - 1) // PAGE)
        # by the kinds of the whole model, not of this pipeline stage's layers: every stage keeps the same tables, so
        # their schedulers and prefix caches decide alike
        if self.model_has_c4:
            n_rows = end // 4
            if n_rows > 0:
                self.c4.ensure(row, 0, (n_rows - 1) // PAGE)
        if self.model_has_c128:
            n_rows = end // 128
            if n_rows > 0:
                self.c128.ensure(row, 0, (n_rows - 1) // PAGE)

    def admit_needs(self, n_tokens: int, context: int) -> Tuple[int, int]:
        """(sliding-window pages, ratio-4 pages) a new request of this size must find free."""
        c4 = ((context + (2 * self.spec_tokens + 1 if self.spec_tokens else 0)) // 4) // PAGE + 1
        return (min(n_tokens, context) + self.cfg.sliding_window) // PAGE + 2, -(-c4 // self.dcp_size)

    def fits(self, context: int) -> bool:
        """Whether a request of this context could ever be admitted (its ratio-4 pages fit the whole pool)."""
        return self.admit_needs(0, context)[1] <= self.c4.num_pages

    def can_admit(self, n_tokens: int, context: int) -> bool:
        need_swa, need_c4 = self.admit_needs(n_tokens, context)
        return (bool(self.free_rows) and len(self.swa.free) >= need_swa
                and len(self.c4.free) - self.promised() >= need_c4)

    def sync(self, parity: int = 0) -> None:
        for g in (self.swa, self.c4, self.c128):
            g.sync(parity)

    def bytes_allocated(self) -> int:
        n = 0
        for d in (self.swa_cache, self.comp_cache, self.idx_cache):
            n += sum(c.buf.numel() for c in d.values())
        for d in (self.comp_state, self.idx_state):
            n += sum(t.numel() * 4 for t in d.values())
        return n


def size_pools(cfg: ModelConfig, max_requests: int, max_context: int, max_chunk: int, dcp_size: int = 1,
               pool_tokens: Optional[int] = None) -> Dict[str, int]:
    """Pages needed so that `max_requests` sequences of `max_context` tokens fit (no prefix sharing); with decode
    context parallelism `c4_pages` is one rank's share (every dcp_size-th page of each request, rounded up).
    pool_tokens: cap the compressed pools at this many context tokens over all requests together (plus the partial
    pages every request may leave open); admission then makes requests wait for room."""
    swa = max_requests * ((cfg.sliding_window + PAGE - 1) // PAGE + 2) + (max_chunk + PAGE - 1) // PAGE + 2
    c4 = max_requests * -(-((max_context // 4 + PAGE - 1) // PAGE + 1) // dcp_size)
    c128 = max_requests * ((max_context // 128 + PAGE - 1) // PAGE + 1)
    if pool_tokens is not None:
        c4 = min(c4, -(-(pool_tokens // 4) // (PAGE * dcp_size)) + max_requests)
        c128 = min(c128, -(-(pool_tokens // 128) // PAGE) + 2 * max_requests + 1)
    return {"swa_pages": swa, "c4_pages": c4, "c128_pages": c128}


def kv_bytes_per_context_token(cfg: ModelConfig, layers: Optional[List[int]] = None, dcp_size: int = 1) -> float:
    """Bytes of compressed KV (latent + indexer-K rows of the ratio-4 layers, latent rows of the ratio-128 layers) that
    one token of context costs a rank: the quantity that turns a memory budget into `pool_tokens`."""
    fp8 = cfg.kv_cache_dtype == "fp8_ds_mla"
    D, Rd, di = cfg.head_dim, cfg.qk_rope_head_dim, cfg.index_head_dim
    latent = PagedCache.page_bytes(D, Rd, fp8, "latent") / PAGE
    index = PagedCache.page_bytes(di, Rd, fp8, "indexer", fp4=cfg.indexer_dtype == "mxfp4") / PAGE
    total = 0.0
    for li in (layers if layers is not None else range(cfg.num_hidden_layers)):
        kind = cfg.layer_kind(li)
        if kind == "c4a":
            total += (latent + index) / 4 / dcp_size
        elif kind == "c128a":
            total += latent / 128
    return total


def memory_pool_tokens(cfg: ModelConfig, utilization: float, free_bytes: int, total_bytes: int, min_tokens: int,
                       layers: Optional[List[int]] = None, dcp_size: int = 1) -> int:
    """Context tokens the compressed pools may hold when this process may use `utilization` of the device's memory:
    that share minus what is taken already (the weights; other tenants of a shared GPU count too), divided by the
    bytes one token costs, but never less than one request of `min_tokens` (launchers/start-hy4-tp4.sh:16-30 GPU_MEM)."""
    budget = utilization * total_bytes - (total_bytes - free_bytes)
    per_token = kv_bytes_per_context_token(cfg, layers, dcp_size)
    return max(min_tokens, int(budget / max(per_token, 1e-9)))
