"""Refit the drafter's Markov head from a token corpus.

    python -m stkernel_b200.tools.markov_refit --corpus FILES... --tokenizer DIR [--base CKPT] \
        --rank 256 --blend 0.5 --out markov.pt

The Markov head scores the next token by ``W2[next] . W1[prev]``, a rank-R model of a [V, V] bias.
This tool estimates that bias from data as the smoothed, clipped pointwise mutual information of
adjacent token pairs, blends it with the shipped head's ``W1 W2^T`` (never materialising V x V: both
are applied as operators), and re-factorises the blend to rank R with a randomised range finder +
SVD.  The payload ``{"markov_w1", "markov_w2", "meta"}`` is what the serving loader's sideload
accepts; only the proposal distribution changes, the verified output distribution does not.
(Method: tools/markov_refit.py:174-203 PMI, :206-224 randomised SVD, :227-343 driver in the reference.)
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import sys
from collections import Counter
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch


def count_bigrams(docs: Iterable[Sequence[int]]) -> Tuple[Counter, Counter, int]:
    pairs: Counter = Counter()
    uni: Counter = Counter()
    total = 0
    for ids in docs:
        uni.update(ids)
        total += len(ids)
        pairs.update(zip(ids, ids[1:]))
    return pairs, uni, total


def pmi_operator(pairs: Counter, uni: Counter, total: int, vocab: int, smooth_k: float = 5.0, clip: float = 4.0,
                 min_count: int = 2) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """clip(log P(next | prev) - log P(next)) with add-k smoothing toward the unigram, as a sparse
    [V, V] matrix (rows = prev) and its transpose."""
    rows, cols, vals = [], [], []
    for (prev, nxt), c in pairs.items():
        if c < min_count or not (0 <= prev < vocab and 0 <= nxt < vocab):
            continue
        p_next = uni[nxt] / total
        v = math.log((c + smooth_k * p_next) / (uni[prev] + smooth_k)) - math.log(p_next)
        rows.append(prev)
        cols.append(nxt)
        vals.append(max(-clip, min(clip, v)))
    if not rows:
        raise ValueError("no bigram survived min_count; corpus too small or too diverse")
    idx = torch.tensor([rows, cols], dtype=torch.int64)
    val = torch.tensor(vals, dtype=torch.float32)
    m = torch.sparse_coo_tensor(idx, val, (vocab, vocab), check_invariants=True).coalesce()
    mt = torch.sparse_coo_tensor(idx.flip(0), val, (vocab, vocab), check_invariants=True).coalesce()
    return m, mt, len(rows)


def randomized_factor(matvec: Callable[[torch.Tensor], torch.Tensor], rmatvec: Callable[[torch.Tensor], torch.Tensor],
                      vocab: int, rank: int, oversample: int = 16, power_iters: int = 2, seed: int = 0
                      ) -> Tuple[torch.Tensor, torch.Tensor, float]:
    """M ~= W1 @ W2^T for an operator given by M x and M^T x.  Returns (W1 [V,R], W2 [V,R], share of the
    sketched spectrum kept)."""
    g = torch.Generator().manual_seed(seed)
    sketch = min(vocab, rank + oversample)
    y = matvec(torch.randn(vocab, sketch, generator=g))
    for _ in range(power_iters):
        y, _ = torch.linalg.qr(y)                          # re-orthonormalise: keeps small directions alive
        y = matvec(rmatvec(y))
    q, _ = torch.linalg.qr(y)
    b = rmatvec(q).T                                       # [sketch, V] = Q^T M
    u, s, vh = torch.linalg.svd(b, full_matrices=False)
    root = torch.sqrt(s[:rank])
    w1 = (q @ u)[:, :rank] * root
    w2 = vh[:rank].T * root
    kept = float(s[:rank].sum() / s.sum()) if float(s.sum()) > 0 else 0.0
    return w1.contiguous(), w2.contiguous(), kept


def refit(pairs: Counter, uni: Counter, total: int, vocab: int, rank: int, blend: float = 0.5,
          base: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, scale: float = 1.0, **kw) -> Dict[str, object]:
    if not 0.0 <= blend <= 1.0:
        raise ValueError(f"blend must be in [0, 1], got {blend}")
    if base is None and blend < 1.0:
        blend = 1.0                                        # nothing to blend with: pure PMI
    m, mt, kept_pairs = pmi_operator(pairs, uni, total, vocab, kw.get("smooth_k", 5.0), kw.get("clip", 4.0), kw.get("min_count", 2))
    if base is not None:
        b1, b2 = base[0].float(), base[1].float()
        mv = lambda x: blend * scale * torch.sparse.mm(m, x) + (1 - blend) * (b1 @ (b2.T @ x))
        rmv = lambda x: blend * scale * torch.sparse.mm(mt, x) + (1 - blend) * (b2 @ (b1.T @ x))
    else:
        mv = lambda x: scale * torch.sparse.mm(m, x)
        rmv = lambda x: scale * torch.sparse.mm(mt, x)
    w1, w2, energy = randomized_factor(mv, rmv, vocab, rank, kw.get("oversample", 16), kw.get("power_iters", 2), kw.get("seed", 0))
    return {"markov_w1": w1, "markov_w2": w2,
            "meta": {"vocab_size": vocab, "rank": rank, "blend": blend, "pairs": kept_pairs, "tokens": total, "energy": energy}}


def load_base(path: str) -> Tuple[torch.Tensor, torch.Tensor]:
    from ..models.loader import SafetensorsIndex
    idx = SafetensorsIndex(path)
    return idx.get("mtp.markov_w1.weight").float().clone(), idx.get("mtp.markov_w2.weight").float().clone()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--corpus", nargs="+", required=True)
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--base", default="", help="checkpoint directory with the shipped mtp.markov_w{1,2}")
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--blend", type=float, default=0.5)
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--smooth-k", type=float, default=5.0)
    ap.add_argument("--clip", type=float, default=4.0)
    ap.add_argument("--min-count", type=int, default=2)
    ap.add_argument("--vocab-size", type=int, default=0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    from ..bench.ngram_ceiling import iter_docs
    if a.tokenizer:
        from ..serve.tokenizer import HFTokenizer
        tk = HFTokenizer(a.tokenizer)
        enc, vocab = tk.encode, tk.vocab_size
    else:
        from ..serve.tokenizer import ByteTokenizer
        tk = ByteTokenizer(512)
        enc, vocab = tk.encode, 512
    vocab = max(vocab, a.vocab_size)
    base = load_base(a.base) if a.base else None
    if base is not None:
        vocab = max(vocab, base[0].shape[0])
        if base[0].shape != base[1].shape or base[0].shape[0] != vocab:
            print(f"shipped markov shapes disagree: {tuple(base[0].shape)} vs {tuple(base[1].shape)} (vocab {vocab})")
            return 1
    rank = a.rank or (base[0].shape[1] if base is not None else 0)
    if not rank:
        print("--rank is required without --base")
        return 1
    pairs, uni, total = count_bigrams(enc(p + c) for p, c in iter_docs(a.corpus))
    payload = refit(pairs, uni, total, vocab, rank, a.blend, base, a.scale, smooth_k=a.smooth_k, clip=a.clip,
                    min_count=a.min_count, seed=a.seed)
    payload["markov_w1"] = payload["markov_w1"].to(torch.bfloat16)
    payload["markov_w2"] = payload["markov_w2"].to(torch.bfloat16)
    torch.save(payload, a.out)
    sha = hashlib.sha256(open(a.out, "rb").read()).hexdigest()
    print(json.dumps({**payload["meta"], "out": a.out, "sha256": sha}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
