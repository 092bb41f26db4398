"""Pure index math of the scheduler and the parallel layouts (no tensors, no process groups).

* `split_indexer_prefill_chunks`: packs the requests of a prefill step into indexer work items under
  two budgets at once -- gathered-K workspace rows and the fp32 logits buffer -- sub-chunking a single
  oversized request along its queries (budget rule of overlay/indexer.py `split_indexer_prefill_chunks`,
  exercised by tests/test_logic.py:103-148 in the reference);
* `sp_gather_sizes`: how a large step's rows are ceil-split over the TP ranks when indexer scoring is
  sequence-parallel (the split rule of overlay/attention.py `_indexer_sp_owned_ranges`);
* decode-context-parallel helpers: interleaved ownership of KV positions and the merge of per-rank
  top-k candidates into the global top-k (the DCP merge of probes/sai_probe.py:1872-2618);
* pipeline stage layer ranges (overlay/nvidia_model.py:1623-1648) and the IndexCache compute/reuse pattern.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

Range = Tuple[int, int]


# ---------------------------------------------------------------------------------------
# indexer prefill chunks
# ---------------------------------------------------------------------------------------
def split_indexer_prefill_chunks(seq_lens: Sequence[int], query_lens: Sequence[int], workspace_rows: int,
                                 logits_bytes: int, request_offset: int = 0) -> List[Tuple[slice, slice]]:
    """-> [(request slice, query slice)].  A multi-request item satisfies sum(seq) <= workspace_rows and
    sum(query) * sum(seq) * 4 <= logits_bytes; its query slice spans all queries of those requests
    (relative to the first request of the item).  A request that cannot share is emitted alone, and when
    its own q * n exceeds the logits budget its queries are cut into the largest equal-budget pieces
    (never below one row)."""
    max_elems = max(1, logits_bytes // 4)
    out: List[Tuple[slice, slice]] = []
    n_req = len(seq_lens)
    i = 0
    while i < n_req:
        n, q, j = 0, 0, i
        while j < n_req:
            n2, q2 = n + seq_lens[j], q + query_lens[j]
            if j > i and (n2 > workspace_rows or q2 * n2 > max_elems):
                break
            n, q, j = n2, q2, j + 1
        reqs = slice(i + request_offset, j + request_offset)
        if j - i == 1 and q * n > max_elems and n > 0:
            step = max(1, max_elems // n)
            for a in range(0, q, step):
                out.append((reqs, slice(a, min(q, a + step))))
        else:
            out.append((reqs, slice(0, q)))
        i = j
    return out


# ---------------------------------------------------------------------------------------
# sequence-parallel indexer scoring
# ---------------------------------------------------------------------------------------
def sp_gather_sizes(prefill_chunk: Range, tp_size: int) -> List[int]:
    """Rows each rank contributes for one large chunk (for the ragged all-gather of its top-k rows)."""
    a, b = prefill_chunk
    shard = -(-(b - a) // tp_size)
    return [max(0, min(b, a + (r + 1) * shard) - min(b, a + r * shard)) for r in range(tp_size)]


# ---------------------------------------------------------------------------------------
# decode context parallel
# ---------------------------------------------------------------------------------------
def _clamp(x, lo: int, hi: int):
    return x.clamp(lo, hi) if hasattr(x, "clamp") else max(lo, min(hi, x))


# The four functions below take Python ints or integer tensors (the model calls them on whole steps at once).
def dcp_owner(row, dcp_size: int, interleave: int = 1):
    """Rank that stores compressed-KV row `row` (rows dealt round-robin in groups of `interleave`)."""
    return (row // interleave) % dcp_size


def dcp_local_rows(n_rows, dcp_size: int, rank: int, interleave: int = 1):
    """How many of the first n_rows live on `rank`: whole rounds, plus the rank's part of the open round."""
    span = interleave * dcp_size
    return (n_rows // span) * interleave + _clamp(n_rows % span - rank * interleave, 0, interleave)


def dcp_local_index(row, dcp_size: int, interleave: int = 1):
    """Index of global row `row` inside its owner's local cache."""
    g = row // interleave
    return (g // dcp_size) * interleave + row % interleave


def dcp_global_row(local, dcp_size: int, rank: int, interleave: int = 1):
    return ((local // interleave) * dcp_size + rank) * interleave + local % interleave


def merge_topk_candidates(per_rank: Sequence[Sequence[Tuple[float, int]]], k: int) -> List[int]:
    """Global top-k row ids from each rank's local top-k (score, global row) lists; ties to the lower row.
    The plain statement of what `models.dsv4.dcp_merge_candidates` does on whole steps with tensor sorts."""
    allc = [c for lst in per_rank for c in lst]
    allc.sort(key=lambda c: (-c[0], c[1]))
    return [row for _, row in allc[:k]]


# ---------------------------------------------------------------------------------------
# pipeline stages, IndexCache pattern
# ---------------------------------------------------------------------------------------
def pp_layer_range(num_layers: int, pp_size: int, rank: int) -> Range:
    """Contiguous layers of a stage; earlier stages take the remainder (the last stage also runs the head)."""
    base, rem = divmod(num_layers, pp_size)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def index_cache_pattern(compress_ratios: Sequence[int], num_layers: int, freq: int) -> List[Optional[bool]]:
    """Per layer: True = computes its own top-k (F), False = reuses the previous F layer's (S), None = no
    indexer.  Counted over C4A layers only; the first C4A layer always computes."""
    out: List[Optional[bool]] = []
    ordinal = 0
    for i in range(num_layers):
        if (compress_ratios[i] if i < len(compress_ratios) else 0) != 4:
            out.append(None)
            continue
        out.append(freq <= 1 or ordinal % freq == 0)
        ordinal += 1
    return out
