"""Automatic prefix caching over the hybrid paged KV.

A prompt is cut into blocks of `block` tokens; a hash chain over the blocks keys the state the engine holds
after computing them: the compressed pages (ratio-4 latent + indexer-K), the sliding-window pages of the
last `window` tokens, and a copy of the compressors' ring rows (the raw rows a window that straddles the cut
still needs).  A new request whose prompt starts with a cached chain adopts those pages (they are
reference-counted, never copied) and starts its prefill at the cut.  `block` is 256 tokens, so that the cut
falls on a page boundary of the sliding-window and ratio-4 groups (64 rows, 64 x 4 tokens) and on a window
boundary of the ratio-128 compressor.  A ratio-128 page spans 8192 tokens, so a cut usually falls inside one:
the full pages before it are shared like the others, and the rows of the partial page are copied into the entry
and, on adoption, into a fresh page of the adopting request (at most 63 rows per ratio-128 layer).

Entries are dropped least-recently-used when a pool runs low, longest prefixes of a chain first (an entry is
only reachable through its ancestors, so every touch of an entry also refreshes them), and all at once by `reset()` — the
`/reset_prefix_cache` endpoint the reference's supervisor calls daily when idle
(launchers/dsv4-tp4-supervisor.sh:117-132).  The reference relies on its engine's prefix cache for
multi-turn chat; this is the equivalent for the hybrid cache layout (overlay/attention.py:743-759 lists the
same groups).
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops.cache import PAGE
from .kv import KVManager

BLOCK = 256


@dataclass
class Entry:
    pos: int                                  # tokens covered
    c4_pages: List[int]
    swa_first: int                            # first logical SWA page held
    swa_pages: List[int]
    comp_state: Dict[int, torch.Tensor] = field(default_factory=dict)     # layer -> ring rows
    idx_state: Dict[int, torch.Tensor] = field(default_factory=dict)
    c128_pages: List[int] = field(default_factory=list)                   # full ratio-128 pages (shared)
    c128_tail: Dict[int, torch.Tensor] = field(default_factory=dict)      # layer -> bytes of the partial page
    c128_part: bool = False                                               # rows past the shared pages exist


def chain_hashes(tokens: Sequence[int], block: int = BLOCK, limit: Optional[int] = None) -> List[bytes]:
    """Hash of every full block prefix: h[i] covers tokens[0 : (i+1)*block]."""
    out: List[bytes] = []
    prev = b""
    n = (len(tokens) if limit is None else min(limit, len(tokens))) // block
    for i in range(n):
        h = hashlib.blake2b(prev, digest_size=16)
        h.update(struct.pack(f"<{block}q", *tokens[i * block:(i + 1) * block]))
        prev = h.digest()
        out.append(prev)
    return out


class PrefixCache:
    def __init__(self, kv: KVManager, max_entries: int = 512, block: int = BLOCK):
        self.kv = kv
        self.block = block
        self.max_entries = max_entries
        self.entries: "OrderedDict[bytes, Entry]" = OrderedDict()
        cfg = kv.cfg
        self.c128_layers = [l for l in kv.layers if cfg.layer_kind(l) == "c128a"]     # this stage's: their bytes are copied
        # decisions follow the whole model, so that every pipeline stage keeps and finds the same entries
        self.has_c128 = kv.model_has_c128
        self.enabled = block % (4 * PAGE) == 0 and block % 128 == 0
        self.window_pages = (cfg.sliding_window + PAGE - 1) // PAGE
        self.hits = 0
        self.hit_tokens = 0
        self.queries = 0

    # ---- lookup --------------------------------------------------------------------------------
    def match(self, prompt: Sequence[int]) -> Tuple[int, Optional[Entry]]:
        """Longest cached prefix that leaves at least one prompt token to compute."""
        if not self.enabled or not self.entries:
            return 0, None
        self.queries += 1
        best: Optional[Entry] = None
        hit: List[bytes] = []
        for h in chain_hashes(prompt, self.block, limit=len(prompt) - 1):
            e = self.entries.get(h)
            if e is None:
                break
            best = e
            hit.append(h)
        self._touch(hit)
        return (best.pos, best) if best is not None else (0, None)

    def _touch(self, chain: Sequence[bytes]) -> None:
        """Refresh a chain so that its longest prefix is the oldest of it and its root the newest: eviction then
        takes leaves first and never strands an entry behind a missing ancestor."""
        for h in reversed(chain):
            if h in self.entries:
                self.entries.move_to_end(h)

    def adopt(self, row: int, e: Entry) -> None:
        """Give request row `row` the cached state (pages shared, ring rows copied)."""
        kv = self.kv
        kv.c4.adopt(row, 0, e.c4_pages)
        kv.swa.adopt(row, e.swa_first, e.swa_pages)
        for li, st in e.comp_state.items():
            kv.comp_state[li][row].copy_(st)
        for li, st in e.idx_state.items():
            kv.idx_state[li][row].copy_(st)
        if self.has_c128:
            if e.c128_pages:
                kv.c128.adopt(row, 0, e.c128_pages)
            if e.c128_part:
                lp = len(e.c128_pages)
                kv.c128.ensure(row, lp, lp)                        # a page of its own for the rows past the shared ones
                pg = int(kv.c128.table_np[row][lp])
                for li, tail in e.c128_tail.items():
                    kv.comp_cache[li].buf[pg].copy_(tail)
        self.hits += 1
        self.hit_tokens += e.pos

    # ---- registration ----------------------------------------------------------------------------
    def offer(self, row: int, prompt: Sequence[int], pos: int) -> bool:
        """Called when request `row` has exactly `pos` prompt tokens computed; keeps the state if `pos` is a
        block boundary that is not cached yet."""
        if not self.enabled or pos <= 0 or pos % self.block or pos > len(prompt):
            return False
        hashes = chain_hashes(prompt, self.block, limit=pos)
        key = hashes[-1]
        if key in self.entries:
            self._touch(hashes)
            return False
        kv = self.kv
        n_c4_pages = (pos // 4) // PAGE
        last_swa = pos // PAGE - 1
        first_swa = max(0, last_swa - self.window_pages + 1)
        if first_swa < kv.swa.lo[row] or last_swa >= kv.swa.hi[row] or n_c4_pages > kv.c4.hi[row]:
            return False                                        # window pages already released: nothing to keep
        while len(self.entries) >= self.max_entries:
            self.evict_one()
        e = Entry(pos, kv.c4.share(row, 0, n_c4_pages - 1) if n_c4_pages else [], first_swa,
                  kv.swa.share(row, first_swa, last_swa))
        for li, st in kv.comp_state.items():
            e.comp_state[li] = st[row].clone()
        for li, st in kv.idx_state.items():
            e.idx_state[li] = st[row].clone()
        if self.has_c128:
            rows = pos // 128
            full, part = rows // PAGE, rows % PAGE
            if full > kv.c128.hi[row] or (part and full >= kv.c128.hi[row]):
                self._drop(e)
                return False
            e.c128_pages = kv.c128.share(row, 0, full - 1) if full else []
            e.c128_part = bool(part)
            if part:
                pg = int(kv.c128.table_np[row][full])
                for li in self.c128_layers:
                    e.c128_tail[li] = kv.comp_cache[li].buf[pg].clone()
        self.entries[key] = e
        self._touch(hashes)
        return True

    # ---- eviction ------------------------------------------------------------------------------
    def _drop(self, e: Entry) -> None:
        for pg in e.c4_pages:
            self.kv.c4.unref(pg)
        for pg in e.swa_pages:
            self.kv.swa.unref(pg)
        for pg in e.c128_pages:
            self.kv.c128.unref(pg)

    def evict_one(self) -> bool:
        if not self.entries:
            return False
        _, e = self.entries.popitem(last=False)
        self._drop(e)
        return True

    def make_room(self, need_swa: int, need_c4: int) -> None:
        """Drop least-recently-used entries until the pools have the requested free pages (or none are left)."""
        while (len(self.kv.swa.free) < need_swa or len(self.kv.c4.free) < need_c4) and self.evict_one():
            pass

    def reset(self) -> int:
        n = len(self.entries)
        while self.evict_one():
            pass
        return n
