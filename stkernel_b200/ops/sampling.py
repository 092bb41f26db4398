"""Sampling ops: seeded-Gumbel argmax, coupled verify/accept, Markov top-k bias."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from . import reference as R
from .scratch import scratch

BF16 = torch.bfloat16
F32 = torch.float32


def gumbel_argmax(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor, pos: torch.Tensor,
                  rows_per_request: int = 1, want_processed: bool = False, top_k: Optional[torch.Tensor] = None,
                  top_p: Optional[torch.Tensor] = None, vocab_start: int = 0, ll=None,
                  agreed_status: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """logits [B*n, V]; row r belongs to request r // n and samples position pos[req] + r % n.

    token = argmax(logits/T + g(seed, position, v)); T <= 0 is greedy.  Returns int64 tokens [B*n]
    and (optionally) the processed logits logits/T as fp32 (-inf outside the truncated set).

    top_k (int32 per request, <= 0 off) / top_p (float per request, >= 1 off): the arg-max runs over the k largest
    logits and/or the smallest set whose probability at temperature T reaches p (ties at the threshold stay in);
    the noise stays a function of (seed, position, vocab id), so truncated drafts and verifications stay coupled.

    vocab_start / ll: `logits` is one tensor-parallel rank's vocabulary shard starting at that id; the ranks of the
    exchange `ll` agree on the winner without gathering logits (GPU only, no truncation); `agreed_status` (int32 [1])
    receives the largest kernel status code of any rank."""
    rows, v = logits.shape
    n = rows_per_request
    if not logits.is_cuda:
        req = torch.arange(rows) // n
        p = pos[req] + torch.arange(rows) % n
        tok, proc = R.gumbel_sample(logits, temperature[req], seed[req], p,
                                    top_k[req] if top_k is not None else None, top_p[req] if top_p is not None else None)
        return tok, (proc if want_processed else None)
    dev = logits.device
    chunks = 32 if v >= 32768 else 4
    pv = scratch("samp.pv", (rows * chunks,), F32, dev)
    pi = scratch("samp.pi", (rows * chunks,), torch.int32, dev)
    out = torch.empty(rows, dtype=torch.int64, device=dev)
    proc = torch.empty(rows, v, dtype=F32, device=dev) if want_processed else None
    group = None
    if n > 1:
        group = scratch("samp.group", (rows,), torch.int32, dev)
        group.copy_(torch.arange(rows, device=dev, dtype=torch.int32) // n)
    trunc = top_k is not None or top_p is not None
    thr = scratch("samp.thr", (rows,), torch.int32, dev) if trunc else None
    _lib.call("stk_gumbel_argmax", logits, logits.stride(0), 1 if logits.dtype == BF16 else 0, temperature, seed, pos,
              group, n if n > 1 else 0, pv, pi, chunks, out, proc, v, rows, v, top_k, top_p, thr, int(vocab_start),
              ll.ctx if ll is not None else None, _lib.status_buffer() if ll is not None else None, agreed_status,
              _lib.status_buffer(), _lib.stream())
    return out, proc


def coupled_accept(verifier: torch.Tensor, draft: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """verifier [B, N+1], draft [B, N] int64 -> (n_accepted [B], emitted [B, N+1] with -1 after the first reject)."""
    b, n1 = verifier.shape
    n = n1 - 1
    if not verifier.is_cuda:
        ok = torch.ones(b, dtype=torch.bool)
        acc = torch.zeros(b, dtype=torch.int64)
        em = torch.full((b, n1), -1, dtype=torch.int64)
        for i in range(n1):
            em[:, i] = torch.where(ok, verifier[:, i], em[:, i])
            if i < n:
                ok = ok & (verifier[:, i] == draft[:, i])
                acc += ok.long()
        return acc, em
    acc = torch.empty(b, dtype=torch.int64, device=verifier.device)
    em = torch.empty(b, n1, dtype=torch.int64, device=verifier.device)
    _lib.call("stk_coupled_accept", verifier.contiguous(), draft.contiguous(), acc, em, b, n, _lib.stream())
    return acc, em


def markov_topk_bias(base: torch.Tensor, w2: torch.Tensor, embed: torch.Tensor, topk: int) -> torch.Tensor:
    """base logits [B, V], w2 [V, R] bf16, embed [B, R] bf16 -> fp32 logits with the Markov bias on the
    base top-k and -inf elsewhere (topk == 0: dense bias)."""
    b, v = base.shape
    if not base.is_cuda:
        return R.markov_bias_topk(base, w2, embed, topk)
    out = torch.empty(b, v, dtype=F32, device=base.device)
    _lib.call("stk_markov_topk_bias", base, base.stride(0), 1 if base.dtype == BF16 else 0, w2, embed, embed.stride(0),
              out, v, b, v, w2.shape[1], topk, _lib.stream())
    return out


def topk_candidates(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """logits [rows, V] -> (vocab ids int32 [rows, k], values fp32 [rows, k]) of the k largest entries per row, in no
    particular order.  Two levels of the register-resident row top-k: the vocabulary is cut into segments of at most
    16384 entries, each segment keeps its own top-k, and a second pass picks k among those candidates."""
    from . import attention as A
    rows, v = logits.shape
    lf = logits.float()
    if not logits.is_cuda:
        val, idx = torch.topk(lf, k, dim=-1)
        return idx.to(torch.int32), val
    segs = max(1, -(-v // 16384))
    seg = -(-v // segs)
    seg = (seg + 3) // 4 * 4
    if seg * segs != v:
        lf = torch.nn.functional.pad(lf, (0, seg * segs - v), value=float("-inf"))
    flat = lf.view(rows * segs, seg)
    n_valid = torch.full((rows * segs,), seg, dtype=torch.int32, device=lf.device)
    if seg * segs != v:
        n_valid.view(rows, segs)[:, -1] = v - seg * (segs - 1)
    kk = min(k, seg)
    local = A.topk_rows(flat, n_valid, kk)                                   # [rows*segs, kk], -1 padded
    ok = local >= 0
    vals = torch.where(ok, flat.gather(1, local.clamp(min=0).long()), torch.full_like(local, float("-inf"), dtype=F32))
    gidx = torch.where(ok, local + (torch.arange(rows * segs, device=lf.device, dtype=torch.int32) % segs)[:, None] * seg,
                       torch.full_like(local, -1))
    if segs == 1:
        return gidx.contiguous(), vals.contiguous()
    cand_v = vals.view(rows, segs * kk).contiguous()
    cand_i = gidx.view(rows, segs * kk)
    n2 = torch.full((rows,), segs * kk, dtype=torch.int32, device=lf.device)
    sel = A.topk_rows(cand_v, n2, k).clamp(min=0).long()
    return cand_i.gather(1, sel).contiguous(), cand_v.gather(1, sel).contiguous()


def markov_chain(cand_idx: torch.Tensor, cand_val: torch.Tensor, anchors: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
                 temperature: torch.Tensor, seed: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """Sequential Markov sampling over fixed candidate sets.  cand_idx int32 / cand_val fp32 [B, N, K]; anchors [B] the
    token before the block; position i is drawn with the noise key (seed, pos + i).  Returns tokens int64 [B, N]."""
    b, n, k = cand_idx.shape
    if not cand_idx.is_cuda:
        out = torch.empty(b, n, dtype=torch.int64)
        prev = anchors.clone()
        v = w1.shape[0]
        for i in range(n):
            e = w1[prev].float()
            idx = cand_idx[:, i].long()
            ok = idx >= 0
            bias = torch.einsum("bkr,br->bk", w2.float()[idx.clamp(min=0)], e)
            full = torch.full((b, v), float("-inf"))
            full.scatter_(1, idx.clamp(min=0), torch.where(ok, cand_val[:, i] + bias, torch.full_like(bias, float("-inf"))))
            tok, _ = R.gumbel_sample(full, temperature, seed, pos + i)
            out[:, i] = tok
            prev = tok
        return out
    out = torch.empty(b, n, dtype=torch.int64, device=cand_idx.device)
    _lib.call("stk_markov_chain", cand_idx.contiguous(), cand_val.contiguous(), anchors.contiguous(), w1, w2, temperature,
              seed, pos.contiguous(), out, b, n, k, w1.shape[1], w1.shape[0], _lib.stream())
    return out
