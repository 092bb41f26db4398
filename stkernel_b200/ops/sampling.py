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
                  rows_per_request: int = 1, want_processed: bool = False
                  ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """logits [B*n, V]; row r belongs to request r // n and samples position pos[req] + r % n.

    token = argmax(logits/T + g(seed, position, v)); T <= 0 is greedy.  Returns int64 tokens [B*n]
    and (optionally) the processed logits logits/T as fp32."""
    rows, v = logits.shape
    n = rows_per_request
    if not logits.is_cuda:
        req = torch.arange(rows) // n
        p = pos[req] + torch.arange(rows) % n
        tok, proc = R.gumbel_sample(logits, temperature[req], seed[req], p)
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
    _lib.call("stk_gumbel_argmax", logits, logits.stride(0), 1 if logits.dtype == BF16 else 0, temperature, seed, pos,
              group, n if n > 1 else 0, pv, pi, chunks, out, proc, v, rows, v, _lib.stream())
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
