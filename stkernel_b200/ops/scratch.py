"""Per-device scratch arena with cached, address-stable views.

Each named buffer is allocated once per device and only grows, so a kernel
launched with the same name and size sees the same address every step (needed
for CUDA-graph replay).  Buffers used on different streams must use different
names: two names never alias; inside `side_branch(stream)` every name gets the
branch's suffix, so the same op may run on the main and on a side stream at once.
This is the engine's equivalent of the reference's eager scratch pool
(overlay/eager_scratch.py:27-168).
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Dict, Sequence, Tuple

import torch

_pool: Dict[Tuple[str, str], torch.Tensor] = {}
_frozen = False
_branch = ""


@contextmanager
def side_branch(stream, label: str = "side"):
    """Run the enclosed ops on `stream` (a fork of the step's dependency graph, also under CUDA-graph capture) with
    their own copies of every named scratch buffer.  The caller orders the streams with events."""
    global _branch
    prev = _branch
    _branch = "@" + label
    try:
        with torch.cuda.stream(stream):
            yield
    finally:
        _branch = prev


def freeze(flag: bool = True) -> None:
    """After freezing (graphs captured) a request that would grow a buffer raises instead."""
    global _frozen
    _frozen = flag


def scratch(name: str, shape: Sequence[int], dtype: torch.dtype, device, zero: bool = False) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = max(n * torch.empty((), dtype=dtype).element_size(), 16)
    key = (name + _branch, str(device))
    buf = _pool.get(key)
    if buf is None or buf.numel() < nbytes:
        if _frozen and buf is not None:
            raise RuntimeError(f"scratch buffer {name!r} would grow after graphs were captured")
        cap = max(nbytes, 2 * buf.numel() if buf is not None else 0)
        cap = (cap + 255) // 256 * 256
        buf = torch.zeros(cap, dtype=torch.uint8, device=device) if zero else torch.empty(cap, dtype=torch.uint8, device=device)
        _pool[key] = buf
    return buf[:n * torch.empty((), dtype=dtype).element_size()].view(dtype).view(*shape)


def reset() -> None:
    _pool.clear()


def total_bytes() -> int:
    return sum(b.numel() for b in _pool.values())
