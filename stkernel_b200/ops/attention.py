"""Indexer scoring / top-k, per-step index metadata and sparse MLA attention."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from . import reference as R
from .cache import PAGE, PagedCache
from .scratch import scratch
from .functional import cpu_act_dtype

BF16 = torch.bfloat16
F32 = torch.float32
I32 = torch.int32
# The tcgen05 sparse-MLA kernel serves fp8_ds_mla rows of the production shape; other shapes (and
# this switch set to False, for A/B checks) use the split-row CUDA-core kernel.
USE_TENSOR_CORE_MLA = True
USE_TENSOR_CORE_INDEXER = True
tc_indexer_calls = 0     # launches of the tcgen05 scorer (tests check that the path they mean to cover ran)
MLA_DIRECT_OUT = True     # single-split steps: final rows written by the attention kernel itself
# optional int64[8] device tensor receiving stage timestamps (ns) of CTA (0, 0) of the tcgen05 kernel
MLA_TRACE = None


# ---- metadata -------------------------------------------------------------------
def token_maps(query_start: torch.Tensor, req_rows: torch.Tensor, start_pos: torch.Tensor, n_req: int, t_padded: int,
               block_table: Optional[torch.Tensor] = None):
    """-> (tok_req i32 [T], positions i64 [T], first_pos i32 [T], last_pos i32 [T][, slot_mapping i64 [T]]);
    padding tokens get request -1 / position -1 / slot -1.  With a block table the destination slot of
    every token's own row is returned as well."""
    dev = query_start.device
    if dev.type != "cuda":
        tok_req = torch.full((t_padded,), -1, dtype=I32)
        positions = torch.full((t_padded,), -1, dtype=torch.int64)
        first = torch.zeros(t_padded, dtype=I32)
        last = torch.full((t_padded,), -1, dtype=I32)
        for i in range(n_req):
            a, b = int(query_start[i]), int(query_start[i + 1])
            tok_req[a:b] = int(req_rows[i])
            positions[a:b] = int(start_pos[i]) + torch.arange(b - a)
            first[a:b] = int(start_pos[i])
            last[a:b] = int(start_pos[i]) + (b - a) - 1
        if block_table is None:
            return tok_req, positions, first, last
        sm = torch.full((t_padded,), -1, dtype=torch.int64)
        ok = tok_req >= 0
        if ok.any():
            sm[ok] = _slots_from_bt(block_table, tok_req[ok].long(), positions[ok]).to(torch.int64)
        return tok_req, positions, first, last, sm
    tok_req = scratch("meta.tok_req", (t_padded,), I32, dev)
    positions = scratch("meta.positions", (t_padded,), torch.int64, dev)
    first = scratch("meta.first", (t_padded,), I32, dev)
    last = scratch("meta.last", (t_padded,), I32, dev)
    sm = scratch("meta.slot_mapping", (t_padded,), torch.int64, dev) if block_table is not None else None
    _lib.call("stk_token_maps", query_start, req_rows, start_pos, n_req, tok_req, positions, first, last, block_table,
              block_table.stride(0) if block_table is not None else 0, sm, t_padded, _lib.stream())
    if block_table is None:
        return tok_req, positions, first, last
    return tok_req, positions, first, last, sm


def _slots_from_bt(block_table, req, p):
    page = block_table[req, p // PAGE]
    return torch.where(page >= 0, page * PAGE + p % PAGE, torch.full_like(page, -1))


def swa_indices(positions: torch.Tensor, tok_req: torch.Tensor, block_table: torch.Tensor, window: int,
                tag: str = "swa") -> Tuple[torch.Tensor, torch.Tensor]:
    """Per token the SWA-cache slots of positions [pos-W+1, pos] (-1 padded) and their count."""
    t = positions.shape[0]
    dev = positions.device
    if dev.type != "cuda":
        slots = torch.full((t, window), -1, dtype=I32)
        lens = torch.zeros(t, dtype=I32)
        for i in range(t):
            pos, req = int(positions[i]), int(tok_req[i])
            if pos < 0 or req < 0:
                continue
            lo = max(0, pos - window + 1)
            p = torch.arange(lo, pos + 1)
            slots[i, :p.numel()] = _slots_from_bt(block_table, req, p).to(I32)
            lens[i] = p.numel()
        return slots, lens
    slots = scratch(f"{tag}.slots", (t, window), I32, dev)
    lens = scratch(f"{tag}.lens", (t,), I32, dev)
    _lib.call("stk_swa_indices", positions, tok_req, block_table, block_table.stride(0), slots, window, lens, t, window,
              _lib.stream())
    return slots, lens


def swa_indices_noncausal(tok_req: torch.Tensor, prefix_len: torch.Tensor, seq_len: torch.Tensor,
                          block_table: torch.Tensor, window: int, width: int, tag: str = "swa_nc"):
    """DSpark draft block: every query of a request sees positions [prefix-W, seq_len)."""
    t = tok_req.shape[0]
    dev = tok_req.device
    if dev.type != "cuda":
        slots = torch.full((t, width), -1, dtype=I32)
        lens = torch.zeros(t, dtype=I32)
        for i in range(t):
            req = int(tok_req[i])
            if req < 0:
                continue
            lo = max(0, int(prefix_len[req]) - window)
            n = int(seq_len[req]) - lo
            if n > width:
                lo += n - width
                n = width
            p = torch.arange(lo, lo + n)
            slots[i, :n] = _slots_from_bt(block_table, req, p).to(I32)
            lens[i] = n
        return slots, lens
    slots = scratch(f"{tag}.slots", (t, width), I32, dev)
    lens = scratch(f"{tag}.lens", (t,), I32, dev)
    _lib.call("stk_swa_indices_noncausal", tok_req, prefix_len, seq_len, block_table, block_table.stride(0), slots,
              width, lens, t, window, _lib.stream())
    return slots, lens


def compressed_valid(positions: torch.Tensor, ratio: int, tag: str = "nvalid") -> torch.Tensor:
    t = positions.shape[0]
    if not positions.is_cuda:
        return torch.where(positions >= 0, (positions + 1) // ratio, torch.zeros_like(positions)).to(I32)
    out = scratch(tag, (t,), I32, positions.device)
    _lib.call("stk_compressed_valid", positions, out, t, ratio, _lib.stream())
    return out


def c128_indices(positions, tok_req, block_table, ratio: int, cap: int, tag: str = "c128"):
    t = positions.shape[0]
    dev = positions.device
    if dev.type != "cuda":
        slots = torch.full((t, cap), -1, dtype=I32)
        lens = torch.zeros(t, dtype=I32)
        for i in range(t):
            pos, req = int(positions[i]), int(tok_req[i])
            if pos < 0 or req < 0:
                continue
            nv = (pos + 1) // ratio
            lo = max(0, nv - cap)
            j = torch.arange(lo, nv)
            slots[i, :j.numel()] = _slots_from_bt(block_table, req, j).to(I32)
            lens[i] = j.numel()
        return slots, lens
    slots = scratch(f"{tag}.slots", (t, cap), I32, dev)
    lens = scratch(f"{tag}.lens", (t,), I32, dev)
    _lib.call("stk_c128_indices", positions, tok_req, block_table, block_table.stride(0), slots, cap, lens, t, ratio,
              cap, _lib.stream())
    return slots, lens


# ---- indexer -----------------------------------------------------------------------
def indexer_scores(q: torch.Tensor, w: torch.Tensor, kcache: PagedCache, block_table: torch.Tensor,
                   tok_req: torch.Tensor, n_valid: torch.Tensor, max_rows: int, tag: str = "idx") -> torch.Tensor:
    """q [T, ih, d] (fp8 or bf16), w [T, ih] folded weights -> scores fp32 [T, ld] (entries >= n_valid[t] undefined)."""
    t, ih, d = q.shape
    ld = max(4, (max_rows + 3) // 4 * 4)
    if not q.is_cuda:
        if hasattr(q, "dequant"):                # MXFP4 operand (ops.cache.Mxfp4Rows): both sides dequantise exactly
            q = q.dequant()
        scores = torch.full((t, ld), float("-inf"), dtype=F32)
        for i in range(t):
            nv, req = int(n_valid[i]), int(tok_req[i])
            if nv <= 0 or req < 0:
                continue
            s = torch.arange(nv)
            rows, sc = kcache.read_rows_cpu(_slots_from_bt(block_table, req, s))
            scores[i, :nv] = R.indexer_scores(q[i:i + 1].to(F32), w[i:i + 1], rows, sc)[0]
        return scores
    scores = scratch(f"{tag}.scores", (t, ld), F32, q.device)
    if (USE_TENSOR_CORE_INDEXER and q.dtype != BF16 and kcache.fp8 and ih == 64 and d == 128 and q.is_contiguous()
            and kcache.page_stride % 16 == 0):
        # tcgen05 scorer: K block stationary in shared memory, q tiles streamed by TMA, one cache row per epilogue thread
        global tc_indexer_calls
        tc_indexer_calls += 1
        _lib.call("stk_indexer_scores_tc", q, w, kcache.buf, kcache.page_stride, kcache.num_pages, block_table,
                  block_table.stride(0), tok_req, n_valid, scores, ld, t, max_rows, ih, d, _lib.status_buffer(),
                  _lib.stream())
        return scores
    _lib.call("stk_indexer_scores", q, w, kcache.buf, kcache.page_stride, 1 if kcache.fp8 else 0, block_table,
              block_table.stride(0), tok_req, n_valid, scores, ld, t, max_rows, ih, d,
              1 if q.dtype != BF16 else 0, _lib.stream())
    return scores


def topk_rows(scores: torch.Tensor, n_valid: torch.Tensor, k: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Indices of the k largest valid scores per row, -1 padded.  The order inside a row is unspecified."""
    t = scores.shape[0]
    if not scores.is_cuda:
        r = R.topk_rows(scores, n_valid, k)
        if out is not None:
            out[:t, :k] = r
            return out
        return r
    if out is None:
        out = torch.empty(t, k, dtype=I32, device=scores.device)
    _lib.call("stk_topk_rows", scores, scores.stride(0), n_valid, out, out.stride(0), t, k, _lib.stream())
    return out


def topk_to_slots(topk: torch.Tensor, block_table: torch.Tensor, tok_req: torch.Tensor, max_rows: int,
                  tag: str = "topk") -> Tuple[torch.Tensor, torch.Tensor]:
    """Local compressed indices -> physical slots of the compressed cache (+ count of valid entries)."""
    t, k = topk.shape[0], topk.shape[1]
    if not topk.is_cuda:
        slots = torch.full((t, k), -1, dtype=I32)
        lens = torch.zeros(t, dtype=I32)
        for i in range(t):
            req = int(tok_req[i])
            if req < 0:
                continue
            idx = topk[i].long()
            ok = idx >= 0
            s = _slots_from_bt(block_table, req, idx.clamp(min=0))
            slots[i] = torch.where(ok, s, torch.full_like(s, -1)).to(I32)
            lens[i] = int((slots[i] >= 0).sum())
        return slots, lens
    slots = scratch(f"{tag}.slots", (t, k), I32, topk.device)
    lens = scratch(f"{tag}.lens", (t,), I32, topk.device)
    _lib.call("stk_topk_to_slots", topk, k, topk.stride(0), block_table, block_table.stride(0), tok_req, slots, k, lens,
              t, max_rows, _lib.status_buffer(), _lib.stream())
    return slots, lens


# ---- attention ------------------------------------------------------------------------
USE_DECODE_MLA = True          # register-resident kernel for decode-sized steps (False: always the tensor-core kernel)
MLA_DECODE_MAX_T = 8


def sparse_mla(q: torch.Tensor, swa_cache: PagedCache, swa_slots: torch.Tensor, swa_lens: torch.Tensor,
               comp_cache: Optional[PagedCache], topk_slots: Optional[torch.Tensor], topk_lens: Optional[torch.Tensor],
               sink: torch.Tensor, scale: float, inv_rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
               q_prep: Optional[Tuple[torch.Tensor, torch.Tensor, float]] = None,
               kv_insert: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    """q [T, nh, D] bf16 -> out [T, nh, D] bf16 attending to the SWA rows then the top-k rows.

    Only the first swa_lens[t] / topk_lens[t] entries of each list are read; -1 entries inside that
    range are masked.  inv_rope = (positions, inv_freq): also apply the inverse RoPE to the output's
    rope dims (fused into the split-merge kernel on the tensor-core path).
    q_prep = (positions, inv_freq, eps): q is the raw projection output; its per-head weightless RMSNorm and RoPE are
    applied here (inside the decode kernel when it serves the step, else by the stand-alone op first).
    kv_insert = (raw kv [T, D], kv norm weight [D], slots int64 [T]): pure-decode steps only (one token per request) and
    only together with q_prep on the decode kernel -- the kernel builds each token's own latent row (norm, RoPE,
    quantise), writes it into the window cache at its slot and attends to it, so no insert launch precedes it."""
    t, nh, d = q.shape
    decode_kernel = (q.is_cuda and USE_DECODE_MLA and t <= MLA_DECODE_MAX_T and swa_cache.fp8 and d == 512
                     and swa_cache.rope_dim == 64 and nh % 8 == 0 and q.stride(0) % 8 == 0 and q.stride(1) == d
                     and (comp_cache is None or comp_cache.fp8)
                     and swa_slots.shape[1] + (topk_slots.shape[1] if topk_slots is not None else 0) <= 4096)
    if q_prep is not None and not decode_kernel:
        from .functional import q_norm_rope
        q = q_norm_rope(q, q_prep[0], q_prep[1], swa_cache.rope_dim, q_prep[2])
    if kv_insert is not None and not (decode_kernel and q_prep is not None):
        raise ValueError("kv_insert needs the decode attention kernel with q_prep")
    if decode_kernel:
        max_rows = swa_slots.shape[1] + (topk_slots.shape[1] if topk_slots is not None else 0)
        S = _lib.query("stk_mla_decode_splits", t, nh, max_rows, _lib.sm_count())
        assert S > 0
        ws = scratch("mla.dpartial", (t * S * nh * 516,), F32, q.device)
        out = torch.empty(t, nh, d, dtype=BF16, device=q.device)
        pos = q_prep[0] if q_prep is not None else (inv_rope[0] if inv_rope is not None else None)
        inv = q_prep[1] if q_prep is not None else (inv_rope[1] if inv_rope is not None else None)
        _lib.call("stk_sparse_mla_decode", q, q.stride(0), swa_cache.buf, swa_cache.page_stride, swa_cache.num_slots,
                  comp_cache.buf if comp_cache is not None else None,
                  comp_cache.page_stride if comp_cache is not None else 0,
                  comp_cache.num_slots if comp_cache is not None else 0, swa_slots, swa_slots.stride(0), swa_slots.shape[1],
                  swa_lens, topk_slots, topk_slots.stride(0) if topk_slots is not None else 0,
                  topk_slots.shape[1] if topk_slots is not None else 0, topk_lens, sink, out, out.stride(0), ws,
                  S, t, nh, float(scale), 1 if q_prep is not None else 0, float(q_prep[2]) if q_prep is not None else 0.0,
                  pos, inv, 1 if inv_rope is not None else 0,
                  kv_insert[0] if kv_insert is not None else None, kv_insert[0].stride(0) if kv_insert is not None else 0,
                  kv_insert[1] if kv_insert is not None else None, kv_insert[2] if kv_insert is not None else None,
                  _lib.status_buffer(), _lib.stream())
        return out
    if not q.is_cuda:
        out = torch.zeros(t, nh, d, dtype=F32)
        for i in range(t):
            sl = swa_slots[i, :int(swa_lens[i])].long()
            rows = [swa_cache.read_rows_cpu(sl)[0]]
            valid = [sl >= 0]
            if topk_slots is not None:
                tl = topk_slots[i, :int(topk_lens[i])].long()
                rows.append(comp_cache.read_rows_cpu(tl)[0])
                valid.append(tl >= 0)
            rr = torch.cat(rows)[None]
            vv = torch.cat(valid)[None]
            out[i] = R.sparse_mla(q[i:i + 1], rr, vv, sink, scale)[0]
        out = out.to(cpu_act_dtype())
        if inv_rope is not None:
            from .functional import q_norm_rope
            out = q_norm_rope(out, inv_rope[0], inv_rope[1], swa_cache.rope_dim, 0.0, norm=False, inverse=True)
        return out
    max_rows = swa_slots.shape[1] + (topk_slots.shape[1] if topk_slots is not None else 0)
    cc = comp_cache if comp_cache is not None else swa_cache
    if USE_TENSOR_CORE_MLA and swa_cache.fp8 and d == 512 and swa_cache.rope_dim == 64 and nh <= 64 and q.stride(0) % 8 == 0:
        # tcgen05 kernel: one 64-row key block per CTA while the SMs are not full (a block is a serial chain of
        # gather -> QK^T -> softmax -> PV, so at decode sizes more, shorter CTAs finish sooner)
        n_splits = max(1, min((max_rows + 63) // 64, (2 * _lib.sm_count()) // max(t, 1)))
        if n_splits == 1 and MLA_DIRECT_OUT:
            # enough tokens to fill the GPU: the kernel writes the final rows itself (no fp32 partials, no combine pass)
            out = torch.empty(t, nh, d, dtype=BF16, device=q.device)
            _lib.call("stk_sparse_mla_tc_out", q, q.stride(0), swa_cache.buf, swa_cache.page_stride, cc.buf, cc.page_stride,
                      swa_slots, swa_slots.stride(0), swa_lens, topk_slots,
                      topk_slots.stride(0) if topk_slots is not None else 0, topk_lens, t, nh, d, swa_cache.rope_dim,
                      max_rows, float(scale), out, out.stride(0), sink,
                      inv_rope[0] if inv_rope is not None else None, inv_rope[1] if inv_rope is not None else None,
                      _lib.status_buffer(), _lib.stream())
            return out
        ws = scratch("mla.partial", (t * n_splits * nh * (d + 2),), F32, q.device)
        out = torch.empty(t, nh, d, dtype=BF16, device=q.device)
        _lib.call("stk_sparse_mla_tc", q, q.stride(0), swa_cache.buf, swa_cache.page_stride, cc.buf, cc.page_stride,
                  swa_slots, swa_slots.stride(0), swa_lens, topk_slots,
                  topk_slots.stride(0) if topk_slots is not None else 0, topk_lens, ws, n_splits, t, nh, d,
                  swa_cache.rope_dim, max_rows, float(scale), _lib.status_buffer(), MLA_TRACE, _lib.stream())
        _lib.call("stk_sparse_mla_combine", ws, sink, out, out.stride(0), t, nh, d, n_splits,
                  inv_rope[0] if inv_rope is not None else None, inv_rope[1] if inv_rope is not None else None,
                  swa_cache.rope_dim, _lib.stream())
        return out
    n_splits = _lib.query("stk_sparse_mla_pick_splits", t, max_rows)
    ws = scratch("mla.partial", (t * n_splits * nh * (d + 2),), F32, q.device)
    out = torch.empty(t, nh, d, dtype=BF16, device=q.device)
    _lib.call("stk_sparse_mla", q, q.stride(0), swa_cache.buf, swa_cache.page_stride, swa_cache.data_bytes, cc.buf,
              cc.page_stride, cc.data_bytes, 1 if swa_cache.fp8 else 0, swa_slots, swa_slots.stride(0), swa_lens,
              topk_slots, topk_slots.stride(0) if topk_slots is not None else 0, topk_lens, sink, out, out.stride(0), ws,
              n_splits, t, nh, d, swa_cache.rope_dim, max_rows, float(scale), _lib.stream())
    if inv_rope is not None:
        from .functional import q_norm_rope
        out = q_norm_rope(out, inv_rope[0], inv_rope[1], swa_cache.rope_dim, 0.0, norm=False, inverse=True)
    return out
