"""CUDA-event stage probes: device time of named spans on whatever stream they run.

Enabled with ``STK_PROF=1`` (off: `span()` is a no-op context manager costing one attribute read).
Events are recorded around a stage, kept in a batch, and resolved with a single `synchronize()` every
`FLUSH_EVERY` spans, so the probes add no per-stage host stall.  Nothing is recorded while the
current stream is being captured into a CUDA graph (an event record inside a capture would invalidate
it); captured steps are profiled with the torch-profiler tools instead.  Steps are classified as decode
or prefill by their row count (`decode_rows` = max sequences x (1 + speculative tokens)).
Equivalent of the reference's stage probes (probes/attn_prof.py:88-183, probes/moe_prof.py:59-101,
probes/oproj_prof.py:13-50).
"""
from __future__ import annotations

import contextlib
import os
from collections import defaultdict
from typing import Dict, Iterator, List, Optional, Tuple

import torch

ENABLED = os.environ.get("STK_PROF", "0") == "1"
FLUSH_EVERY = 400


class SpanRecorder:
    def __init__(self, decode_rows: int = 256):
        self.decode_rows = decode_rows
        self.pending: List[Tuple[str, str, "torch.cuda.Event", "torch.cuda.Event"]] = []
        self.totals: Dict[Tuple[str, str], List[float]] = defaultdict(lambda: [0.0, 0])
        self.skipped_in_capture = 0

    def phase(self, rows: int) -> str:
        return "decode" if rows <= self.decode_rows else "prefill"

    @contextlib.contextmanager
    def span(self, name: str, rows: int = 1) -> Iterator[None]:
        if not torch.cuda.is_available():
            yield
            return
        if torch.cuda.is_current_stream_capturing():
            self.skipped_in_capture += 1
            yield
            return
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        try:
            yield
        finally:
            e1.record()
            self.pending.append((self.phase(rows), name, e0, e1))
            if len(self.pending) >= FLUSH_EVERY:
                self.flush()

    def add_ms(self, phase: str, name: str, ms: float) -> None:
        t = self.totals[(phase, name)]
        t[0] += ms
        t[1] += 1

    def flush(self) -> None:
        if not self.pending:
            return
        self.pending[-1][3].synchronize()
        for phase, name, e0, e1 in self.pending:
            self.add_ms(phase, name, e0.elapsed_time(e1))
        self.pending.clear()

    def report(self) -> str:
        self.flush()
        lines = []
        for phase in ("decode", "prefill"):
            rows = [(n, v) for (p, n), v in self.totals.items() if p == phase]
            if not rows:
                continue
            total = sum(v[0] for _, v in rows)
            lines.append(f"[{phase}] {total:.2f} ms in {sum(v[1] for _, v in rows)} spans")
            for n, (ms, cnt) in sorted(rows, key=lambda r: -r[1][0]):
                lines.append(f"  {n:24s} {ms:10.3f} ms  {cnt:7d}x  {1e3 * ms / max(cnt, 1):9.1f} us/call  {100 * ms / max(total, 1e-9):5.1f} %")
        if self.skipped_in_capture:
            lines.append(f"({self.skipped_in_capture} spans skipped inside CUDA-graph capture)")
        return "\n".join(lines)


_RECORDER: Optional[SpanRecorder] = None
_NULL = contextlib.nullcontext()


def recorder() -> SpanRecorder:
    global _RECORDER
    if _RECORDER is None:
        _RECORDER = SpanRecorder()
    return _RECORDER


def span(name: str, rows: int = 1):
    """`with span("attn", rows=T): ...` -- a no-op unless STK_PROF=1."""
    return recorder().span(name, rows) if ENABLED else _NULL
