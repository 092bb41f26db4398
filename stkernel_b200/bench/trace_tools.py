"""Chrome-trace post-processing: bucketed busy time, inter-kernel gaps, cross-stream attribution, and
a profile-over-HTTP driver.

    python -m stkernel_b200.bench.trace_tools profile --workload decode:200 [--base URL]
    python -m stkernel_b200.bench.trace_tools gaps TRACE.json
    python -m stkernel_b200.bench.trace_tools concurrent TRACE.json
    python -m stkernel_b200.bench.trace_tools fingerprint NCCL_DEBUG_LOG

* profile: POST /start_profile, run one workload (`prefill:N` = a fresh N-token prompt with max_tokens 1,
  `decode:N` = N decode tokens), POST /stop_profile, wait until the trace file stops growing, then the
  bucket table with busy time as the union of kernel intervals (so overlapping streams are not counted
  twice) and the top kernels (bench/profile-step.py:49-57,166-281 in the reference);
* gaps: idle gaps between consecutive kernels on the busiest stream (histogram, largest gaps with the
  kernels on both sides) and min/median/p99/max per kernel name (probes/trace_precise.py);
* concurrent: for every main-stream gap, which kernels other streams ran meanwhile (probes/gap_concurrent.py);
* fingerprint: a hash of the NCCL topology lines of an NCCL_DEBUG=INFO log, to tell boots apart whose
  rings/trees differ (probes/nccl_fingerprint.py).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import re
import sys
import time
from typing import Dict, List, Optional, Sequence, Tuple

from .kernel_table import BUCKETS, bucket_of, interval_union

GPU_CATS = ("kernel", "gpu_memcpy", "gpu_memset")


def gpu_events(trace: Dict) -> List[Dict]:
    return sorted((e for e in trace.get("traceEvents", []) if e.get("cat") in GPU_CATS and "dur" in e), key=lambda e: e["ts"])


def stream_of(e: Dict) -> int:
    a = e.get("args") or {}
    return int(a.get("stream", e.get("tid", 0)))


def bucket_table(events: Sequence[Dict]) -> Dict:
    per: Dict[str, List[float]] = {}
    for e in events:
        per.setdefault(e["name"], []).append(float(e["dur"]))
    busy = interval_union([(e["ts"], e["ts"] + e["dur"]) for e in events])
    span = (max(e["ts"] + e["dur"] for e in events) - min(e["ts"] for e in events)) if events else 0.0
    buckets: Dict[str, float] = {}
    for n, d in per.items():
        buckets[bucket_of(n)] = buckets.get(bucket_of(n), 0.0) + sum(d)
    return {"kernels": per, "busy_us": busy, "span_us": span, "idle_us": span - busy, "buckets": buckets}


def busiest_stream(events: Sequence[Dict]) -> int:
    tot: Dict[int, float] = {}
    for e in events:
        tot[stream_of(e)] = tot.get(stream_of(e), 0.0) + e["dur"]
    return max(tot, key=tot.get) if tot else 0


def percentile(xs: Sequence[float], q: float) -> float:
    if not xs:
        return 0.0
    s = sorted(xs)
    i = min(len(s) - 1, max(0, int(round(q * (len(s) - 1)))))
    return s[i]


def gap_report(events: Sequence[Dict], top: int = 10, edges: Sequence[float] = (1, 2, 5, 10, 20, 50, 100, 1000)) -> Dict:
    main = busiest_stream(events)
    evs = [e for e in events if stream_of(e) == main]
    gaps: List[Tuple[float, str, str, float]] = []
    for a, b in zip(evs, evs[1:]):
        g = b["ts"] - (a["ts"] + a["dur"])
        if g > 0:
            gaps.append((g, a["name"], b["name"], a["ts"] + a["dur"]))
    hist = [0] * (len(edges) + 1)
    for g, *_ in gaps:
        i = 0
        while i < len(edges) and g >= edges[i]:
            i += 1
        hist[i] += 1
    per: Dict[str, List[float]] = {}
    for e in evs:
        per.setdefault(e["name"], []).append(float(e["dur"]))
    stats = {n: {"n": len(d), "min": min(d), "med": percentile(d, 0.5), "p99": percentile(d, 0.99), "max": max(d)} for n, d in per.items()}
    return {"stream": main, "n_kernels": len(evs), "gap_total_us": sum(g for g, *_ in gaps), "hist_edges_us": list(edges),
            "hist": hist, "largest": sorted(gaps, reverse=True)[:top], "kernel_stats": stats}


def concurrent_report(events: Sequence[Dict], min_gap_us: float = 5.0) -> List[Dict]:
    main = busiest_stream(events)
    evs = [e for e in events if stream_of(e) == main]
    others = [e for e in events if stream_of(e) != main]
    out = []
    for a, b in zip(evs, evs[1:]):
        g0, g1 = a["ts"] + a["dur"], b["ts"]
        if g1 - g0 < min_gap_us:
            continue
        during = [(o["name"], min(g1, o["ts"] + o["dur"]) - max(g0, o["ts"])) for o in others
                  if o["ts"] < g1 and o["ts"] + o["dur"] > g0]
        covered = interval_union([(max(g0, o["ts"]), min(g1, o["ts"] + o["dur"])) for o in others
                                  if o["ts"] < g1 and o["ts"] + o["dur"] > g0])
        out.append({"gap_us": g1 - g0, "after": a["name"], "before": b["name"], "covered_us": covered,
                    "other": sorted(during, key=lambda x: -x[1])[:4]})
    return sorted(out, key=lambda r: -r["gap_us"])


_NCCL_TOPO = re.compile(r"(Channel \d+/\d+ ?:|Ring \d+ ?:|Trees? \[|NVLS|Connected all (rings|trees)|nChannels|P2P/|via NVL|comm 0x\w+ rank \d+ nranks)")


def nccl_fingerprint(log_text: str) -> Tuple[str, int]:
    """Hash of the topology-bearing lines with volatile parts (pids, pointers, host names, times) removed."""
    keep = []
    for line in log_text.splitlines():
        if "NCCL INFO" not in line or not _NCCL_TOPO.search(line):
            continue
        body = line.split("NCCL INFO", 1)[1]
        body = re.sub(r"0x[0-9a-fA-F]+", "PTR", body)
        body = re.sub(r"\b\d+\.\d+\.\d+\.\d+(<\d+>)?", "IP", body)
        body = re.sub(r"pid \d+", "pid N", body)
        keep.append(body.strip())
    keep.sort()
    return hashlib.sha256("\n".join(keep).encode()).hexdigest()[:16], len(keep)


def wait_stable(path: str, settle: float = 2.0, timeout: float = 300.0) -> bool:
    t0, last, since = time.time(), -1, time.time()
    while time.time() - t0 < timeout:
        size = os.path.getsize(path) if os.path.exists(path) else -1
        if size != last:
            last, since = size, time.time()
        elif size > 0 and time.time() - since >= settle:
            return True
        time.sleep(0.5)
    return False


def format_table(tab: Dict, steps: int = 1, top: int = 40) -> str:
    steps = max(steps, 1)
    lines = [f"busy {tab['busy_us'] / steps:.1f} us/step, span {tab['span_us'] / steps:.1f} us/step, "
             f"idle {100 * tab['idle_us'] / max(tab['span_us'], 1e-9):.1f} %"]
    for b, v in sorted(tab["buckets"].items(), key=lambda x: -x[1]):
        lines.append(f"  bucket {b:16s} {v / steps:9.1f} us/step  {100 * v / max(tab['busy_us'], 1e-9):5.1f} %")
    for n, d in sorted(tab["kernels"].items(), key=lambda x: -sum(x[1]))[:top]:
        lines.append(f"  {sum(d) / steps:9.1f} us/step {len(d) / steps:6.1f}x/step avg {sum(d) / len(d):7.1f} us  {n[:70]}")
    return "\n".join(lines)


def run_profile(base: str, model: str, workload: str) -> int:
    from .http_client import Client, spec_counters, unique_prompt
    cl = Client(base, model)
    kind, _, n = workload.partition(":")
    n = int(n or 200)
    m0 = cl.metrics()
    cl.post("/start_profile", {})
    if kind == "prefill":
        cl.chat(unique_prompt(int(time.time()), int(n * 0.55)), 1, 0.0)
    else:
        cl.chat("Write a long story about a lighthouse keeper.", n, 0.8, ignore_eos=True)
    trace = cl.post("/stop_profile", {}).get("trace")
    m1 = cl.metrics()
    if not trace or not wait_stable(trace):
        print("no stable trace file reported by the server", file=sys.stderr)
        return 1
    steps = int(sum(v for k, v in m1.items() if k.startswith("stk:engine_steps_total")) -
                sum(v for k, v in m0.items() if k.startswith("stk:engine_steps_total"))) or 1
    with open(trace) as f:
        tab = bucket_table(gpu_events(json.load(f)))
    print(f"workload {workload}: {steps} engine steps, trace {trace}")
    print(format_table(tab, steps))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("profile")
    p.add_argument("--base", default="http://127.0.0.1:8000")
    p.add_argument("--model", default="deepseek-v4-flash")
    p.add_argument("--workload", default="decode:200")
    for name in ("gaps", "concurrent", "table"):
        q = sub.add_parser(name)
        q.add_argument("trace")
    q = sub.add_parser("fingerprint")
    q.add_argument("log")
    a = ap.parse_args(argv)
    if a.cmd == "profile":
        return run_profile(a.base, a.model, a.workload)
    if a.cmd == "fingerprint":
        fp, n = nccl_fingerprint(open(a.log, errors="replace").read())
        print(f"{fp}  ({n} topology lines)")
        return 0
    with open(a.trace) as f:
        evs = gpu_events(json.load(f))
    if a.cmd == "table":
        print(format_table(bucket_table(evs)))
    elif a.cmd == "gaps":
        r = gap_report(evs)
        print(f"stream {r['stream']}: {r['n_kernels']} kernels, idle between kernels {r['gap_total_us']:.1f} us")
        edges = r["hist_edges_us"]
        labels = [f"<{edges[0]}"] + [f"{a_}-{b_}" for a_, b_ in zip(edges, edges[1:])] + [f">={edges[-1]}"]
        print("gap histogram (us): " + "  ".join(f"{l}:{c}" for l, c in zip(labels, r["hist"])))
        for g, a_, b_, ts in r["largest"]:
            print(f"  {g:9.1f} us  after {a_[:40]}  before {b_[:40]}")
        for n, s in sorted(r["kernel_stats"].items(), key=lambda x: -x[1]["med"] * x[1]["n"])[:25]:
            print(f"  {s['n']:5d}x min {s['min']:7.1f} med {s['med']:7.1f} p99 {s['p99']:7.1f} max {s['max']:7.1f}  {n[:60]}")
    else:
        for r in concurrent_report(evs)[:20]:
            other = ", ".join(f"{n[:30]} {d:.0f}us" for n, d in r["other"]) or "nothing"
            print(f"  gap {r['gap_us']:8.1f} us (covered {r['covered_us']:.1f}) after {r['after'][:30]} -> {other}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
