"""Read-only audit of the serving host: memory policy, GPU state, NVLink fabric, leftovers.

    python -m stkernel_b200.fleet.host_audit [--json]

Changes nothing.  Items (reference: launchers/fleet-audit.sh:13-59, restated for one NVSwitch node in
place of four RoCE nodes): THP and compaction policy (the paged pools are allocated once at boot,
fragmentation shows up as slow boots), buddy high-order pages, per-GPU SM clock vs its maximum with the
active throttle reasons, persistence mode, ECC mode, NVLink link state and speed per GPU, P2P access
between every GPU pair, NCCL-relevant env, stray processes that still hold GPU memory.  Every probe is
a function of injectable `run`/`read` callables so the parsers are tested against canned output.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
from typing import Callable, Dict, List, Optional

Run = Callable[[List[str]], Optional[str]]
Read = Callable[[str], Optional[str]]

EXPECTED_LINKS = 18                # NVLink 5 links per B200
EXPECTED_LINK_GBS = 50.0           # GB/s per link per direction


def _run(cmd: List[str]) -> Optional[str]:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=30).stdout
    except (OSError, subprocess.TimeoutExpired):
        return None


def _read(path: str) -> Optional[str]:
    try:
        with open(path) as f:
            return f.read()
    except OSError:
        return None


def bracketed(text: Optional[str]) -> str:
    m = re.search(r"\[(\w+)\]", text or "")
    return m.group(1) if m else "n/a"


def memory_policy(read: Read = _read) -> Dict[str, str]:
    out = {"thp_enabled": bracketed(read("/sys/kernel/mm/transparent_hugepage/enabled")),
           "thp_defrag": bracketed(read("/sys/kernel/mm/transparent_hugepage/defrag")),
           "compaction_proactiveness": (read("/proc/sys/vm/compaction_proactiveness") or "n/a").strip()}
    buddy = read("/proc/buddyinfo") or ""
    hi = 0
    for line in buddy.splitlines():
        if "Normal" in line:
            cols = line.split()
            hi += int(cols[-1]) if cols[-1].isdigit() else 0
    out["buddy_order10_free"] = str(hi)
    return out


def gpu_state(run: Run = _run) -> List[Dict[str, str]]:
    q = "index,name,clocks.sm,clocks.max.sm,temperature.gpu,power.draw,power.limit,persistence_mode,ecc.mode.current,clocks_event_reasons.active,memory.used"
    txt = run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits"]) or ""
    keys = q.split(",")
    rows = []
    for line in txt.strip().splitlines():
        vals = [v.strip() for v in line.split(",")]
        if len(vals) == len(keys):
            rows.append(dict(zip(keys, vals)))
    return rows


def nvlink_state(run: Run = _run) -> Dict[int, Dict[str, float]]:
    """GPU index -> {links_up, min_gbs} parsed from `nvidia-smi nvlink --status`."""
    txt = run(["nvidia-smi", "nvlink", "--status"]) or ""
    out: Dict[int, Dict[str, float]] = {}
    gpu = None
    for line in txt.splitlines():
        m = re.match(r"GPU (\d+):", line)
        if m:
            gpu = int(m.group(1))
            out[gpu] = {"links_up": 0, "min_gbs": float("inf")}
            continue
        m = re.search(r"Link \d+:\s*([\d.]+)\s*GB/s", line)
        if m and gpu is not None:
            out[gpu]["links_up"] += 1
            out[gpu]["min_gbs"] = min(out[gpu]["min_gbs"], float(m.group(1)))
    for g in out.values():
        if g["min_gbs"] == float("inf"):
            g["min_gbs"] = 0.0
    return out


def p2p_matrix(n: int) -> Optional[List[List[bool]]]:
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        n = min(n, torch.cuda.device_count())
        return [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]
    except Exception:
        return None


def findings(mem: Dict[str, str], gpus: List[Dict[str, str]], links: Dict[int, Dict[str, float]],
             p2p: Optional[List[List[bool]]]) -> List[str]:
    """Human-readable deviations from the accepted state (empty = clean)."""
    out = []
    if mem.get("thp_defrag") in ("always",):
        out.append("THP defrag=always: allocation stalls during boot; use madvise or defer")
    for g in gpus:
        idx = g.get("index", "?")
        try:
            sm, mx = float(g["clocks.sm"]), float(g["clocks.max.sm"])
        except (KeyError, ValueError):
            continue
        reasons = g.get("clocks_event_reasons.active", "")
        if "0x0000000000000000" not in reasons and reasons not in ("", "N/A", "[N/A]"):
            out.append(f"GPU {idx}: clock event reasons active: {reasons}")
        if g.get("ecc.mode.current", "Enabled") not in ("Enabled", "N/A", "[N/A]"):
            out.append(f"GPU {idx}: ECC is {g['ecc.mode.current']}")
        try:
            if float(g.get("memory.used", "0")) > 1024:
                out.append(f"GPU {idx}: {g['memory.used']} MiB already in use (stray process?)")
        except ValueError:
            pass
        _ = sm, mx
    for gi, st in sorted(links.items()):
        if st["links_up"] < EXPECTED_LINKS:
            out.append(f"GPU {gi}: {int(st['links_up'])}/{EXPECTED_LINKS} NVLink links up")
        elif st["min_gbs"] < EXPECTED_LINK_GBS * 0.99:
            out.append(f"GPU {gi}: slowest NVLink link {st['min_gbs']} GB/s < {EXPECTED_LINK_GBS}")
    if p2p is not None:
        for i, row in enumerate(p2p):
            for j, ok in enumerate(row):
                if not ok:
                    out.append(f"GPU {i} cannot access GPU {j} peer memory (symmetric-memory path unavailable)")
    return out


def audit(run: Run = _run, read: Read = _read, with_p2p: bool = True) -> Dict[str, object]:
    mem = memory_policy(read)
    gpus = gpu_state(run)
    links = nvlink_state(run)
    p2p = p2p_matrix(len(gpus)) if with_p2p else None
    env = {k: os.environ[k] for k in sorted(os.environ) if k.startswith(("NCCL_", "STK_", "CUDA_VISIBLE"))}
    return {"memory": mem, "gpus": gpus, "nvlink": {str(k): v for k, v in links.items()}, "p2p": p2p, "env": env,
            "findings": findings(mem, gpus, links, p2p)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    rep = audit()
    if a.json:
        print(json.dumps(rep, indent=1))
    else:
        print("-- memory policy --")
        for k, v in rep["memory"].items():
            print(f"  {k}={v}")
        print("-- GPUs --")
        for g in rep["gpus"]:
            print("  " + " ".join(f"{k.split('.')[-1]}={v}" for k, v in g.items()))
        print("-- NVLink --")
        for k, v in rep["nvlink"].items():
            print(f"  GPU {k}: links_up={int(v['links_up'])} min={v['min_gbs']} GB/s")
        print("-- findings --")
        for f in rep["findings"] or ["  none"]:
            print(f"  {f}" if not f.startswith("  ") else f)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
