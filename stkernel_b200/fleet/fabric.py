"""NVLink fabric gate: refuse to start a TP job on a degraded fabric.

    python -m stkernel_b200.fleet.fabric [--gpus N] [--apply]

The reference's fabric script forces its Ethernet switch ports to 200G because links that
auto-negotiate to 100G halve the collective bandwidth (launchers/fabric-200g.sh:1-28).  On an NVSwitch
node there is nothing to force: link speed is fixed by the hardware.  What can go wrong instead is a
link that trained down or a GPU that lost peer access, so the equivalent here is a read-only gate run
before launch: all 18 links up at full rate on every GPU of the job, and peer access for every pair.
`--apply` exists for symmetry with the reference tool and is a no-op that says so: this tool never
writes a GPU or switch setting.
"""
from __future__ import annotations

import argparse
from typing import Dict, List, Optional

from .host_audit import EXPECTED_LINK_GBS, EXPECTED_LINKS, Run, _run, nvlink_state, p2p_matrix


def check(n_gpus: int, run: Run = _run, p2p: Optional[List[List[bool]]] = None) -> List[str]:
    links = nvlink_state(run)
    problems = []
    for g in range(n_gpus):
        st = links.get(g)
        if st is None:
            problems.append(f"GPU {g}: no NVLink status reported")
        elif st["links_up"] < EXPECTED_LINKS:
            problems.append(f"GPU {g}: {int(st['links_up'])}/{EXPECTED_LINKS} links up")
        elif st["min_gbs"] < EXPECTED_LINK_GBS * 0.99:
            problems.append(f"GPU {g}: link at {st['min_gbs']} GB/s, expected {EXPECTED_LINK_GBS}")
    for i, row in enumerate(p2p or []):
        for j, ok in enumerate(row[:n_gpus]):
            if i < n_gpus and not ok:
                problems.append(f"GPU {i} -> GPU {j}: no peer access")
    return problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--apply", action="store_true")
    a = ap.parse_args(argv)
    if a.apply:
        print("fabric: nothing to apply on an NVSwitch node (link rate is not a software setting); checking only")
    problems = check(a.gpus, p2p=p2p_matrix(a.gpus))
    for p in problems:
        print(f"fabric: {p}")
    print("fabric: OK" if not problems else f"fabric: {len(problems)} problem(s)")
    return 0 if not problems else 1


if __name__ == "__main__":
    raise SystemExit(main())
