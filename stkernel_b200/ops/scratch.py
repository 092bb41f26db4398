"""Per-device scratch arena with cached, address-stable views.

Each named buffer is allocated once per device and only grows, so a kernel
launched with the same name and size sees the same address every step (needed
for CUDA-graph replay).  Buffers used on different streams must use different
names: two names never alias.  This is the engine's equivalent of the
reference's eager scratch pool (overlay/eager_scratch.py:27-168).
"""
from __future__ import annotations

from typing import Dict, Sequence, Tuple

import torch

_pool: Dict[Tuple[str, str], torch.Tensor] = {}
_frozen = False


def freeze(flag: bool = True) -> None:
    """After freezing (graphs captured) a request that would grow a buffer raises instead."""
    global _frozen
    _frozen = flag


def scratch(name: str, shape: Sequence[int], dtype: torch.dtype, device, zero: bool = False) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = max(n * torch.empty((), dtype=dtype).element_size(), 16)
    key = (name, str(device))
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
