"""Paged-cache ops: latent-row insert/gather, KV compressor, indexer-K / indexer-Q producers.

A cache is a ``[num_pages, page_stride]`` uint8 tensor of 64-row pages:

* latent rows, ``fp8_ds_mla``: ``[64 x (nope + 2R) data][64 x 8 scale bytes][pad]``
  (overlay/ops_cache_utils.py:29-152); ``bf16``: ``[64 x 2D]``.
* indexer-K rows, fp8: ``[64 x d][64 x fp32 scale][pad]`` (132 B/row for d = 128,
  overlay/attention.py:1000-1009); bf16: ``[64 x 2d]``.

Page strides are padded to a multiple of 576 bytes like the reference's pools.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..config import KV_SCALE_BYTES
from . import _lib
from . import reference as R
from .scratch import scratch


def Fn_act():
    from .functional import cpu_act_dtype
    return cpu_act_dtype()

BF16 = torch.bfloat16
F32 = torch.float32
FP8 = torch.float8_e4m3fn
PAGE = 64


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class PagedCache:
    buf: torch.Tensor          # uint8 [num_pages, page_stride]
    dim: int                   # row width D (or indexer d)
    rope_dim: int
    fp8: bool
    kind: str                  # "latent" | "indexer"
    fp4: bool = False          # indexer rows as MXFP4: dim/2 bytes of e2m1 pairs + dim/32 ue8m0 bytes (reference path only)

    @property
    def num_pages(self) -> int:
        return self.buf.shape[0]

    @property
    def page_stride(self) -> int:
        return self.buf.shape[1]

    @property
    def num_slots(self) -> int:
        return self.num_pages * PAGE

    @property
    def data_bytes(self) -> int:
        if self.kind == "latent":
            return (self.dim - self.rope_dim) + 2 * self.rope_dim if self.fp8 else 2 * self.dim
        if self.fp4:
            return self.dim // 2
        return self.dim if self.fp8 else 2 * self.dim

    @staticmethod
    def page_bytes(dim: int, rope_dim: int, fp8: bool, kind: str, fp4: bool = False) -> int:
        if fp4:
            assert kind == "indexer" and dim % 32 == 0
            return _round_up(PAGE * (dim // 2 + dim // 32), 576)
        if kind == "latent":
            raw = PAGE * ((dim - rope_dim) + 2 * rope_dim + KV_SCALE_BYTES) if fp8 else PAGE * 2 * dim
        else:
            raw = PAGE * (dim + 4) if fp8 else PAGE * 2 * dim
        return _round_up(raw, 576)

    @staticmethod
    def allocate(num_pages: int, dim: int, rope_dim: int, fp8: bool, kind: str, device, fp4: bool = False) -> "PagedCache":
        if fp4 and torch.device(device).type == "cuda":
            raise NotImplementedError("MXFP4 indexer rows are served by the reference (CPU) path only; no GPU kernel reads them")
        stride = PagedCache.page_bytes(dim, rope_dim, fp8, kind, fp4)
        return PagedCache(torch.zeros(num_pages, stride, dtype=torch.uint8, device=device), dim, rope_dim, fp8, kind, fp4)

    # ---- CPU row access (reference path) ----------------------------------
    def write_rows_cpu(self, slots: torch.Tensor, rows: torch.Tensor) -> None:
        """rows [n, dim] fp32 (already roped); slot < 0 skipped."""
        keep = slots >= 0
        slots, rows = slots[keep].long(), rows[keep]
        if slots.numel() == 0:
            return
        page, r = slots // PAGE, slots % PAGE
        db = self.data_bytes
        if self.kind == "latent":
            if self.fp8:
                q, rope, sc = R.kv_row_quant(rows, self.rope_dim)
                nope = self.dim - self.rope_dim
                data = torch.cat([q.view(torch.uint8), rope.contiguous().view(torch.uint8).view(-1, 2 * self.rope_dim)], 1)
                for i in range(slots.numel()):
                    self.buf[page[i], r[i] * db:(r[i] + 1) * db] = data[i]
                    o = PAGE * db + r[i] * KV_SCALE_BYTES
                    self.buf[page[i], o:o + KV_SCALE_BYTES] = sc[i]
            else:
                data = rows.to(BF16).contiguous().view(torch.uint8).view(-1, db)
                for i in range(slots.numel()):
                    self.buf[page[i], r[i] * db:(r[i] + 1) * db] = data[i]
        else:
            if self.fp4:
                packed, sb = R.quant_mxfp4(rows.to(F32))
                nsb = self.dim // 32
                for i in range(slots.numel()):
                    self.buf[page[i], r[i] * db:(r[i] + 1) * db] = packed[i]
                    o = PAGE * db + r[i] * nsb
                    self.buf[page[i], o:o + nsb] = sb[i]
            elif self.fp8:
                q, sc = R.indexer_k_quant(rows)
                scb = sc.to(F32).contiguous().view(torch.uint8).view(-1, 4)
                for i in range(slots.numel()):
                    self.buf[page[i], r[i] * db:(r[i] + 1) * db] = q[i].view(torch.uint8)
                    o = PAGE * db + r[i] * 4
                    self.buf[page[i], o:o + 4] = scb[i]
            else:
                data = rows.to(BF16).contiguous().view(torch.uint8).view(-1, db)
                for i in range(slots.numel()):
                    self.buf[page[i], r[i] * db:(r[i] + 1) * db] = data[i]

    def read_rows_cpu(self, slots: torch.Tensor) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """-> (rows [n, dim] fp32 dequantised (indexer fp8: raw fp8 values), scales [n] for indexer fp8)."""
        n = slots.numel()
        out = torch.zeros(n, self.dim, dtype=F32)
        scales = torch.ones(n, dtype=F32) if (self.kind == "indexer" and self.fp8 and not self.fp4) else None
        db = self.data_bytes
        for i in range(n):
            s = int(slots[i])
            if s < 0:
                continue
            page, r = s // PAGE, s % PAGE
            raw = self.buf[page, r * db:(r + 1) * db]
            if self.kind == "latent":
                if self.fp8:
                    nope = self.dim - self.rope_dim
                    o = PAGE * db + r * KV_SCALE_BYTES
                    sc = self.buf[page, o:o + KV_SCALE_BYTES]
                    out[i] = R.kv_row_dequant(raw[:nope].view(FP8)[None], raw[nope:].view(BF16)[None], sc[None])[0]
                else:
                    out[i] = raw.view(BF16).to(F32)
            else:
                if self.fp4:
                    nsb = self.dim // 32
                    o = PAGE * db + r * nsb
                    out[i] = R.dequant_mxfp4(raw[None], self.buf[page, o:o + nsb][None])[0]
                elif self.fp8:
                    out[i] = raw.view(FP8).to(F32)
                    o = PAGE * db + r * 4
                    scales[i] = self.buf[page, o:o + 4].view(F32)[0]
                else:
                    out[i] = raw.view(BF16).to(F32)
        return out, scales


def kv_rope_quant_insert(kv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, inv: torch.Tensor,
                         cache: PagedCache) -> None:
    """kv [T, D] bf16 (normed): RoPE on the last R dims, quantise, write at `slots` (int64, -1 = skip)."""
    t, d = kv.shape
    rd = cache.rope_dim
    if not kv.is_cuda:
        ang = positions.to(F32)[:, None] * inv[None, :]
        kf = kv.to(F32)
        roped = R.apply_rope_interleaved(kf[:, d - rd:], torch.cos(ang), torch.sin(ang)).to(BF16).to(F32)
        cache.write_rows_cpu(slots, torch.cat([kf[:, :d - rd], roped], 1))
        return
    _lib.call("stk_kv_rope_quant_insert", kv, kv.stride(0), positions, slots, inv, cache.buf, cache.page_stride,
              cache.data_bytes, 1 if cache.fp8 else 0, cache.num_slots, t, d, rd, _lib.status_buffer(), _lib.stream())


def q_rope_kv_insert(q: Optional[torch.Tensor], kv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                     inv: torch.Tensor, cache: PagedCache, eps: float, kv_norm_w: Optional[torch.Tensor] = None
                     ) -> Optional[torch.Tensor]:
    """One launch: per-head weightless RMSNorm + RoPE of q [T, nh, D] (in place) and RoPE + quantise +
    insert of the latent rows kv [T, D].

    kv_norm_w: kv arrives un-normalised and its RMSNorm (this weight, same eps) happens inside the insert.
    q None: only the latent rows are written (the decode attention kernel norms and rotates q itself)."""
    if not kv.is_cuda:
        from .functional import cpu_act_dtype, q_norm_rope
        if kv_norm_w is not None:
            kv = R.rms_norm(kv, kv_norm_w, eps).to(cpu_act_dtype())
        kv_rope_quant_insert(kv, positions, slots, inv, cache)
        return q_norm_rope(q, positions, inv, cache.rope_dim, eps) if q is not None else None
    t, d = kv.shape
    nh = q.shape[1] if q is not None else 0
    _lib.call("stk_q_rope_kv_insert", q, q.stride(0) if q is not None else 0, nh, eps, kv, kv.stride(0), positions, slots,
              inv, cache.buf, cache.page_stride, cache.data_bytes, 1 if cache.fp8 else 0, cache.num_slots, t, d,
              cache.rope_dim, kv_norm_w, _lib.status_buffer(), _lib.stream())
    return q


def kv_gather_dequant(cache: PagedCache, slots: torch.Tensor) -> torch.Tensor:
    """slots [n] int64 -> rows [n, D] bf16 (zeros for slot < 0)."""
    n = slots.numel()
    if not cache.buf.is_cuda:
        return cache.read_rows_cpu(slots)[0].to(Fn_act())
    out = torch.empty(n, cache.dim, dtype=BF16, device=cache.buf.device)
    _lib.call("stk_kv_gather_dequant", cache.buf, cache.page_stride, cache.data_bytes, 1 if cache.fp8 else 0, slots, out,
              n, cache.dim, cache.rope_dim, _lib.stream())
    return out


def compress_windows(kvs: torch.Tensor, ape: torch.Tensor, norm_w: torch.Tensor, inv: torch.Tensor,
                     positions: torch.Tensor, tok_req: torch.Tensor, tok_first_pos: torch.Tensor,
                     tok_last_pos: torch.Tensor, state: torch.Tensor, block_table: torch.Tensor, cache: PagedCache,
                     ratio: int, slots_c: int, eps: float) -> None:
    """Pool every window that closes in this step and insert it into `cache`; then keep the raw
    rows that later windows need.

    kvs [T, 2*c*D] fp32 (value slots then gate slots); state [req_rows, ring, 2*c*D] fp32;
    block_table [req_rows, max_pages] int32 pages of `cache`."""
    t = kvs.shape[0]
    d = cache.dim
    c = slots_c
    ring = state.shape[1]
    if not kvs.is_cuda:
        w = 2 * c * d
        apev = ape.to(F32).view(ratio, c, d)
        for i in range(t):
            pos = int(positions[i])
            if pos < 0 or (pos + 1) % ratio:
                continue
            j = (pos + 1) // ratio - 1
            p0 = j * ratio
            req = int(tok_req[i])
            first = int(tok_first_pos[i])

            def src(p):
                row = kvs[i - (pos - p)] if p >= first else state[req, p % ring]
                return row.to(F32)

            own = torch.stack([src(p0 + k) for k in range(ratio)])
            vals = [own[:, :d]]
            logits = [own[:, c * d:c * d + d] + apev[:, 0]]
            if c == 2 and j >= 1:
                prev = torch.stack([src(p0 - ratio + k) for k in range(ratio)])
                vals.append(prev[:, d:2 * d])
                logits.append(prev[:, c * d + d:c * d + 2 * d] + apev[:, 1])
            v, l = torch.cat(vals), torch.cat(logits)
            pooled = (torch.softmax(l, 0) * v).sum(0, keepdim=True)
            pooled = R.rms_norm(pooled, norm_w, eps)
            rd = cache.rope_dim
            ang = torch.tensor([float(p0)])[:, None] * inv[None, :]
            pooled[:, d - rd:] = R.apply_rope_interleaved(pooled[:, d - rd:], torch.cos(ang), torch.sin(ang))
            if cache.kind == "latent" and cache.fp8:
                pooled[:, d - rd:] = pooled[:, d - rd:].to(BF16).to(F32)
            page = int(block_table[req, j // PAGE])
            cache.write_rows_cpu(torch.tensor([page * PAGE + j % PAGE]), pooled)
        for i in range(t):
            pos = int(positions[i])
            if pos < 0 or pos + ring <= int(tok_last_pos[i]):
                continue
            state[int(tok_req[i]), pos % ring] = kvs[i]
        return
    _lib.call("stk_compress_windows", kvs, kvs.stride(0), ape, norm_w, inv, positions, tok_req, tok_first_pos, tok_last_pos, state,
              block_table, block_table.stride(0), cache.buf, cache.page_stride, cache.data_bytes,
              1 if cache.fp8 else 0, 1 if cache.kind == "indexer" else 0, cache.num_slots, t, d, cache.rope_dim, ratio, c,
              ring, eps, _lib.status_buffer(), _lib.stream())


@dataclass
class Mxfp4Rows:
    """An MXFP4 operand: packed e2m1 pairs [T, ..., d/2] and ue8m0 scale bytes [T, ..., d/32]; sliced by rows."""
    packed: torch.Tensor
    scales: torch.Tensor

    def __getitem__(self, idx) -> "Mxfp4Rows":
        return Mxfp4Rows(self.packed[idx], self.scales[idx])

    @property
    def shape(self):
        return (*self.packed.shape[:-1], self.packed.shape[-1] * 2)

    @property
    def is_cuda(self) -> bool:
        return self.packed.is_cuda

    @property
    def device(self):
        return self.packed.device

    def dequant(self) -> torch.Tensor:
        return R.dequant_mxfp4(self.packed, self.scales)


def indexer_q_prep(q: torch.Tensor, w: torch.Tensor, positions: torch.Tensor, inv: torch.Tensor, rope_dim: int,
                   quantize: bool, fmt: str = "fp8"):
    """q [T, ih, d] bf16, w [T, ih] fp32 -> (q operand: fp8 bytes or bf16 [T, ih, d], folded weights fp32).
    fmt "mxfp4": the operand is an `Mxfp4Rows` and the weights carry no q scale (reference path only)."""
    t, ih, d = q.shape
    if fmt == "mxfp4":
        if q.is_cuda:
            raise NotImplementedError("MXFP4 indexer operands are served by the reference (CPU) path only")
        ang = positions.to(F32)[:, None] * inv[None, :]
        packed, sb, wf = R.indexer_q_prepare_mxfp4(q, w, torch.cos(ang), torch.sin(ang), rope_dim)
        return Mxfp4Rows(packed, sb), wf
    if not q.is_cuda:
        ang = positions.to(F32)[:, None] * inv[None, :]
        qq, wf = R.indexer_q_prepare(q, w, torch.cos(ang), torch.sin(ang), rope_dim, quantize)
        return (qq.to(FP8) if quantize else qq.to(BF16)), wf
    qo = torch.empty(t, ih, d, dtype=torch.uint8 if quantize else BF16, device=q.device)
    wo = torch.empty(t, ih, dtype=F32, device=q.device)
    _lib.call("stk_indexer_q_prep", q, q.stride(0), w, w.stride(0), positions, inv, qo, wo, t, ih, d, rope_dim, 1 if quantize else 0,
              _lib.stream())
    return (qo.view(FP8) if quantize else qo), wo
