"""Pipeline parallelism: the decoder cut into contiguous stages of layers, one stage per group of ranks.

A stage receives the residual streams of a step from its predecessor, runs its layers over its own KV caches, and
sends them on; the first stage embeds, the last one runs the head and samples, and the sampled tokens are broadcast
back so that every stage's scheduler advances identically (lock-step scheduling, as under tensor parallelism).
With tensor parallelism inside the stages, rank (pp_rank, tp_rank) talks to (pp_rank +- 1, tp_rank): global rank =
pp_rank * tp_size + tp_rank.

What crosses a stage boundary per step: the streams [T, hc, H] bf16 (the rank's 1/tp of the rows when the residual is
sequence-parallel) and, when the next stage begins inside an IndexCache group, the shared top-k row list
[T, index_topk] int32 of the group's computing layer.

Counterpart of the reference's pipeline hooks (overlay/nvidia_model.py:1623-1648 make_empty_intermediate_tensors /
PPMissingLayer, 1693-1711 stage-local layer ranges, 1823-1824 intermediate tensors in forward); the stage arithmetic is
`runtime/planning.pp_layer_range`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..runtime.planning import index_cache_pattern, pp_layer_range


@dataclass
class PipeStage:
    pp_rank: int
    pp_size: int
    tp_rank: int = 0
    tp_size: int = 1
    group: Optional[dist.ProcessGroup] = None        # a group that contains every rank of the pipeline (default: world)

    @property
    def first(self) -> bool:
        return self.pp_rank == 0

    @property
    def last(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    def _global(self, pp_rank: int) -> int:
        return pp_rank * self.tp_size + self.tp_rank

    def layer_range(self, num_layers: int) -> Tuple[int, int]:
        return pp_layer_range(num_layers, self.pp_size, self.pp_rank)

    # ---- point to point ------------------------------------------------------------------------------------------
    def send_next(self, t: torch.Tensor) -> None:
        dist.send(t.contiguous(), dst=self._global(self.pp_rank + 1), group=self.group)

    def recv_prev(self, shape, dtype, device) -> torch.Tensor:
        t = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(t, src=self._global(self.pp_rank - 1), group=self.group)
        return t

    def broadcast_from_last(self, t: torch.Tensor) -> torch.Tensor:
        """Every stage ends the step with the last stage's tensor (the sampled tokens)."""
        # one broadcast per tensor-parallel column: the ranks with this tp_rank form the pipeline
        src = self._global(self.pp_size - 1)
        if self.tp_size == 1:
            dist.broadcast(t, src=src, group=self.group)
            return t
        # with tensor parallelism the pipeline's ranks are a strided subset of the world: relay backwards stage by stage
        if not self.last:
            dist.recv(t, src=self._global(self.pp_rank + 1), group=self.group)
        if not self.first:
            dist.send(t, dst=self._global(self.pp_rank - 1), group=self.group)
        return t


def stage_starts_inside_index_group(cfg, lo: int, hi: int) -> bool:
    """Whether the first ratio-4 layer of stage [lo, hi) reuses the top-k rows of a layer in an earlier stage."""
    pat = index_cache_pattern(cfg.compress_ratios, cfg.num_hidden_layers, cfg.index_topk_freq if cfg.use_index_cache else 1)
    for li in range(lo, hi):
        if pat[li] is not None:
            return pat[li] is False
    return False


class MicroBatchPipeline:
    """Several engines of one stage taking turns, so that every stage has work while another engine's step is in flight.

    The requests are dealt over `len(engines)` engines that share the stage's weights (each has its own scheduler and
    its own share of the KV pools).  Tick t begins the step of engine t mod G (schedule, forward, send to the next
    stage) and then finishes the step that engine (t + 1) mod G began G - 1 ticks ago (receive its tokens from the last
    stage, update its requests): with G = number of stages, those tokens were produced one stage-time earlier, so in the
    steady state no stage waits.  Every stage runs the same ticks in the same order, which keeps the sends, receives
    and broadcasts of all stages matched.
    """

    def __init__(self, engines):
        assert engines and all(e.model.pipe is not None for e in engines)
        self.engines = list(engines)
        for e in self.engines:
            e.model.pipe_defer = True
        self.tick = 0
        self.overlapped_ticks = 0                          # ticks that finished one step while another was in flight
        self.pending = [None] * len(self.engines)          # a begun, unfinished step per engine
        self._next = 0
        self._where = {}                                    # global request id -> (engine index, its request id)

    def add_request(self, prompt, params=None) -> int:
        gi = self._next
        self._next += 1
        ei = gi % len(self.engines)                         # the same on every stage
        self._where[gi] = (ei, self.engines[ei].add_request(prompt, params))
        return gi

    def has_work(self) -> bool:
        return any(p is not None for p in self.pending) or any(e.has_work() for e in self.engines)

    def step(self):
        """One tick.  Returns [(global request id, token)] of the step that finished in it."""
        g = len(self.engines)
        ei = self.tick % g
        out = []
        if self.pending[ei] is None and self.engines[ei].has_work():
            self.pending[ei] = self.engines[ei].step_begin()
        fi = (self.tick + 1) % g                            # begun G - 1 ticks ago (this tick's own step when G is 1)
        if self.pending[fi] is not None:
            ticket, self.pending[fi] = self.pending[fi], None
            self.overlapped_ticks += any(p is not None for p in self.pending)
            back = {rid: gid for gid, (e, rid) in self._where.items() if e == fi}
            out = [(back[rid], tok) for rid, tok in self.engines[fi].step_finish(ticket)]
        self.tick += 1
        return out

    def output(self, gid: int):
        ei, rid = self._where[gid]
        return self.engines[ei].requests[rid].output

    # ---- the rest of the engine surface that the serving layer uses --------------------------------------------------
    @property
    def cfg(self):
        return self.engines[0].cfg

    @property
    def device(self):
        return self.engines[0].device

    @property
    def metrics(self):
        """Counters summed over the engines (a fresh object: read it, do not write to it)."""
        import dataclasses
        from ..runtime.metrics import Metrics
        total = Metrics()
        for e in self.engines:
            for f in dataclasses.fields(Metrics):
                a, b = getattr(total, f.name), getattr(e.metrics, f.name)
                if isinstance(b, list):
                    setattr(total, f.name, [x + y for x, y in zip(a + [0] * (len(b) - len(a)), b + [0] * (len(a) - len(b)))])
                elif f.name == "kv_cache_usage":
                    setattr(total, f.name, max(a, b))
                else:
                    setattr(total, f.name, a + b)
        return total

    @property
    def requests(self):
        """global request id -> Request, for the requests that have not been released."""
        out = {}
        for gid, (ei, rid) in self._where.items():
            r = self.engines[ei].requests.get(rid)
            if r is not None:
                out[gid] = r
        return out

    def abort(self, gid: int) -> bool:
        if gid not in self._where:
            return False
        ei, rid = self._where[gid]
        return self.engines[ei].abort(rid)

    def release(self, gid: int) -> None:
        if gid in self._where:
            ei, rid = self._where[gid]
            r = self.engines[ei].requests.get(rid)
            if r is not None and r.finished:
                self.engines[ei].release(rid)
                del self._where[gid]

    def reset_prefix_cache(self) -> int:
        self.engines[0].metrics.prefix_cache_resets += 1
        return sum(e.reset_prefix_cache() for e in self.engines)

    def generate(self, prompts, params=None):
        ids = [self.add_request(p, params) for p in prompts]
        while self.has_work():
            self.step()
        return [self.output(i) for i in ids]
