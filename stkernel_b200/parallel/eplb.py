"""Expert-parallel load balancing: logical -> physical expert placement with redundant replicas, load recording.

Routing picks *logical* experts.  Under expert parallelism each rank holds `n_physical / ep` *physical* expert slots;
with `n_redundant` spare slots the most loaded logical experts get extra replicas, and the slots are packed onto the
ranks so that the expected tokens per rank are even.  A token's pair is sent to one replica of its logical expert,
chosen round-robin by the token's index, so replicas split the load evenly and the choice needs no communication.

Pieces (the counterpart of the reference's EPLB hooks: logical->physical replica map, load recording, redundant
experts -- overlay/nvidia_model.py:258,452-500,852-892,2039-2073):
  * `Placement`            the maps, as python lists and as device tables;
  * `initial_placement`    identity + round-robin replicas (nothing known about the load yet);
  * `rebalance`            greedy replication (highest load per replica first) + longest-processing-time packing;
  * `LoadRecorder`         per-layer token counts per logical expert, accumulated on the device inside the step;
  * `to_physical`          router ids -> physical slot ids for this step.
The engine applies a new placement between steps by rebuilding the experts of each layer from the weight source
(`Engine.rebalance_experts`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch


@dataclass
class Placement:
    n_logical: int
    ep_size: int
    phys_to_logical: List[int]                  # [n_physical]; slot p lives on rank p // slots_per_rank

    @property
    def n_physical(self) -> int:
        return len(self.phys_to_logical)

    @property
    def slots_per_rank(self) -> int:
        return self.n_physical // self.ep_size

    @property
    def is_identity(self) -> bool:
        return self.phys_to_logical == list(range(self.n_logical))

    def replicas(self) -> List[List[int]]:
        out: List[List[int]] = [[] for _ in range(self.n_logical)]
        for p, l in enumerate(self.phys_to_logical):
            out[l].append(p)
        return out

    def validate(self) -> None:
        if self.n_physical % self.ep_size:
            raise ValueError("physical slots must divide evenly over the ranks")
        if any(not r for r in self.replicas()):
            raise ValueError("every logical expert needs at least one physical slot")

    def tables(self, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """(l2p int32 [n_logical, max_replicas] padded with the first replica, replica_count int32 [n_logical])."""
        reps = self.replicas()
        m = max(len(r) for r in reps)
        l2p = torch.tensor([r + [r[0]] * (m - len(r)) for r in reps], dtype=torch.int32, device=device)
        cnt = torch.tensor([len(r) for r in reps], dtype=torch.int32, device=device)
        return l2p, cnt

    def local_logical(self, rank: int) -> List[int]:
        """Logical expert held by each of this rank's slots, in slot order."""
        s = self.slots_per_rank
        return self.phys_to_logical[rank * s:(rank + 1) * s]


def initial_placement(n_logical: int, n_redundant: int, ep_size: int) -> Placement:
    if (n_logical + n_redundant) % ep_size:
        raise ValueError("n_logical + n_redundant must be a multiple of the expert-parallel size")
    return rebalance([1.0] * n_logical, n_redundant, ep_size)


def _pack(load: Sequence[float], reps: Sequence[int], ep_size: int) -> List[int]:
    """Physical slots (one per replica, load split evenly) onto ranks of equal slot count: heaviest first, each onto the
    rank with the smallest total that still has a free slot and, where possible, no replica of the same expert yet."""
    n = len(load)
    items = [(load[e] / reps[e], e) for e in range(n) for _ in range(reps[e])]
    items.sort(key=lambda x: (-x[0], x[1]))
    per = len(items) // ep_size
    rank_load = [0.0] * ep_size
    rank_slots: List[List[int]] = [[] for _ in range(ep_size)]
    for share, e in items:
        free = [r for r in range(ep_size) if len(rank_slots[r]) < per]
        fresh = [r for r in free if e not in rank_slots[r]] or free
        r = min(fresh, key=lambda q: (rank_load[q], q))
        rank_slots[r].append(e)
        rank_load[r] += share
    return [e for r in range(ep_size) for e in sorted(rank_slots[r])]


def _replicate(load: Sequence[float], n_redundant: int, ep_size: int) -> List[int]:
    """Replica counts: each spare slot goes to the expert whose load per replica is currently highest, up to one replica
    per rank (a second replica on a rank takes nothing off that rank); what is left over goes to the least loaded experts."""
    n = len(load)
    reps = [1] * n
    for _ in range(n_redundant):
        open_ = [i for i in range(n) if reps[i] < ep_size]
        if open_:
            e = max(open_, key=lambda i: (load[i] / reps[i], -i))
        else:
            # every expert is on every rank already: a further copy cannot help, so it goes where it disturbs least
            e = min(range(n), key=lambda i: (load[i], reps[i], i))
        reps[e] += 1
    return reps


def rebalance(load: Sequence[float], n_redundant: int, ep_size: int) -> Placement:
    """Placement for the observed per-logical-expert load (tokens routed to it).

    Replication and packing are greedy (`_replicate`, `_pack`); the result is compared with the placement that ignores
    the load (uniform replication, same packing) and the one with the smaller busiest rank is returned, so a rebalance
    never makes the busiest rank busier.  With no spares and uniform load this is the identity."""
    n = len(load)
    n_phys = n + n_redundant
    if n_phys % ep_size:
        raise ValueError("n_logical + n_redundant must be a multiple of the expert-parallel size")
    load = [max(float(x), 0.0) for x in load]
    if n_redundant == 0 and len(set(load)) <= 1:
        return Placement(n, ep_size, list(range(n)))
    flat = [1.0] * n
    candidates = [Placement(n, ep_size, _pack(load, _replicate(load, n_redundant, ep_size), ep_size)),
                  Placement(n, ep_size, _pack(flat, _replicate(flat, n_redundant, ep_size), ep_size))]
    out = min(candidates, key=lambda p: max(rank_loads(p, load)))
    out.validate()
    return out


def rank_loads(p: Placement, load: Sequence[float]) -> List[float]:
    """Expected tokens per rank under placement `p` (a logical expert's load splits evenly over its replicas)."""
    reps = p.replicas()
    out = [0.0] * p.ep_size
    for e, slots in enumerate(reps):
        for s in slots:
            out[s // p.slots_per_rank] += float(load[e]) / len(slots)
    return out


def to_physical(ids: torch.Tensor, l2p: torch.Tensor, rep_count: torch.Tensor) -> torch.Tensor:
    """Logical router ids [T, k] -> physical slot ids [T, k]: replica (token index mod replica count)."""
    t = ids.shape[0]
    tok = torch.arange(t, device=ids.device, dtype=torch.int64)[:, None]
    lid = ids.long()
    which = tok % rep_count[lid].long()
    return l2p[lid, which].to(torch.int32)


class LoadRecorder:
    """Tokens routed to every logical expert of every layer since the last `take()`; lives on the device and is
    updated inside the (possibly captured) step with one scatter-add per layer."""

    def __init__(self, n_layers: int, n_logical: int, device):
        self.counts = torch.zeros(n_layers, n_logical, dtype=torch.int32, device=device)
        self._ones: Optional[torch.Tensor] = None

    def record(self, layer: int, ids: torch.Tensor) -> None:
        flat = ids.reshape(-1).long()
        if self._ones is None or self._ones.numel() < flat.numel():
            self._ones = torch.ones(max(flat.numel(), 64), dtype=torch.int32, device=ids.device)
        self.counts[layer].scatter_add_(0, flat, self._ones[:flat.numel()])

    def take(self) -> torch.Tensor:
        """Counts since the last call as a CPU tensor [layers, experts]; the device counters restart at zero."""
        out = self.counts.to("cpu", copy=True)
        self.counts.zero_()
        return out
