"""Audit the kernel sources for lower AND upper bounds on every externally supplied id.

    python -m stkernel_b200.fleet.audit_guards [--root DIR] [--json] [--self-test]

A token id indexes the embedding and the hash-routing table, a sampled id indexes the vocabulary, an
expert id indexes the expert weights, a slot id indexes a cache page: each must be checked on both
sides in the kernel that consumes it, because one corrupt id in a batch otherwise reads or writes
foreign memory.  The audit greps the sources that are actually deployed; a missing source is UNKNOWN,
never PASS.  Exit codes: 0 = all PASS, 1 = at least one FAIL, 2 = UNKNOWN or probe error (the
contract of launchers/audit-runtime-guards.py:1-8,145-153,255-281 in the reference, applied to this
package's own CUDA sources instead of a third-party image).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
from dataclasses import asdict, dataclass
from typing import Callable, Dict, List, Optional, Tuple

SAMPLER = "stkernel_b200/csrc/sampler.cu"
MOE = "stkernel_b200/csrc/moe.cu"
ROUTER = "stkernel_b200/csrc/router.cuh"      # the selection code shared by the router kernel and the gate epilogue
ELEMENTWISE = "stkernel_b200/csrc/elementwise.cu"
KVCACHE = "stkernel_b200/csrc/kvcache.cu"
ATTENTION = "stkernel_b200/csrc/attention_tc.cu"
INDEXER = "stkernel_b200/csrc/indexer.cu"


@dataclass(frozen=True)
class Result:
    name: str
    status: str                 # PASS | FAIL | UNKNOWN
    path: Optional[str]
    detail: str


Checker = Callable[[str], Tuple[bool, str]]


def _count(text: str, pattern: str) -> int:
    return len(re.findall(pattern, text, flags=re.MULTILINE | re.DOTALL))


def _sampler(text: str) -> Tuple[bool, str]:
    upper = _count(text, r"v1\s*=\s*min\s*\(\s*V\s*,\s*v0\s*\+\s*chunk\s*\)")
    loop = _count(text, r"for\s*\(\s*int\s+v\s*=\s*v0\s*\+\s*threadIdx\.x\s*;\s*v\s*<\s*v1\s*;")
    sentinel = _count(text, r"best_i\s*==\s*0x7fffffff\s*\?\s*0\s*:\s*best_i")
    ok = upper >= 1 and loop >= 1 and sentinel >= 1
    return ok, f"argmax scan clamped to V: {upper}/1, bounded loop: {loop}/1, empty-row fallback: {sentinel}/1"


def _embed(text: str) -> Tuple[bool, str]:
    both = _count(text, r"id\s*>=\s*0\s*&&\s*id\s*<\s*vocab\b")
    flagged = _count(text, r"set_status\s*\(\s*status\s*,\s*kBadIndex")
    return both >= 1 and flagged >= 1, f"token id lower+upper guard: {both}/1, status flag on violation: {flagged}/1"


def _hash_moe(text: str) -> Tuple[bool, str]:
    tok = _count(text, r"tok\s*>=\s*0\s*&&\s*tok\s*<\s*(r\.)?vocab\b")
    eid = _count(text, r"e\s*<\s*0\s*\|\|\s*e\s*>=\s*(r\.)?E\b")
    return tok >= 1 and eid >= 1, f"hash-table token guard: {tok}/1, table-entry expert guard: {eid}/1"


def _expert_map(text: str) -> Tuple[bool, str]:
    n = _count(text, r"e\s*<\s*0\s*\|\|\s*e\s*>=\s*e_local\b")
    return n >= 4, f"lower+upper expert guards (align, sort, fc1, fc2): {n}/4"


def _kv_slots(text: str) -> Tuple[bool, str]:
    lo = _count(text, r"slot\s*<\s*0")
    hi = _count(text, r"slot\s*>=\s*(a\.)?num_slots")
    return lo >= 1 and hi >= 1, f"cache slot lower guards: {lo}, upper guards: {hi}"


def _attn_slots(text: str) -> Tuple[bool, str]:
    lo = _count(text, r"slot\s*(>=|<)\s*0")
    return lo >= 2, f"gathered-row validity checks: {lo}/2"


RULES: Tuple[Tuple[str, str, Checker], ...] = (
    ("sampler.gumbel_argmax", SAMPLER, _sampler),
    ("embed.token_id", ELEMENTWISE, _embed),
    ("hash_moe.token_table", ROUTER, _hash_moe),
    ("expert_map.kernels", MOE, _expert_map),
    ("kv_cache.slot", KVCACHE, _kv_slots),
    ("sparse_mla.gather", ATTENTION, _attn_slots),
)


def read_sources(root: str) -> Dict[str, Dict[str, str]]:
    out: Dict[str, Dict[str, str]] = {}
    for _, rel, _ in RULES:
        full = os.path.join(root, rel)
        if rel not in out and os.path.isfile(full):
            with open(full, encoding="utf-8", errors="replace") as f:
                out[rel] = {"path": full, "text": f.read()}
    return out


def evaluate(sources: Dict[str, Dict[str, str]]) -> List[Result]:
    results = []
    for name, rel, checker in RULES:
        src = sources.get(rel)
        if src is None:
            results.append(Result(name, "UNKNOWN", None, f"{rel} is absent; a built library cannot prove the guard"))
            continue
        ok, detail = checker(src["text"])
        results.append(Result(name, "PASS" if ok else "FAIL", src["path"], detail))
    return results


def exit_code(results: List[Result]) -> int:
    if any(r.status == "FAIL" for r in results):
        return 1
    if any(r.status == "UNKNOWN" for r in results):
        return 2
    return 0


def summary(results: List[Result]) -> Dict[str, int]:
    return {s: sum(r.status == s for r in results) for s in ("PASS", "FAIL", "UNKNOWN")}


def self_test() -> int:
    """Synthetic sources: a guarded set must PASS, the same set with one bound removed must FAIL on
    exactly that rule, an empty set must be UNKNOWN."""
    good = {
        SAMPLER: "const int v0 = blockIdx.y * chunk, v1 = min(V, v0 + chunk);\nfor (int v = v0 + threadIdx.x; v < v1; v += 1) {}\n"
                 "out[row] = best_i == 0x7fffffff ? 0 : best_i;",
        ELEMENTWISE: "const bool in_vocab = id >= 0 && id < vocab; if (!in_vocab) set_status(status, kBadIndex, t);",
        ROUTER: "const bool ok = tok >= 0 && tok < r.vocab; if (e < 0 || e >= r.E) {}\n",
        MOE: "if (e < 0 || e >= e_local) return;\n" * 4,
        KVCACHE: "if (slot < 0) return; if (slot >= num_slots) {}",
        ATTENTION: "valid = slot >= 0; if (slot < 0) {}",
    }
    src = {k: {"path": k, "text": v} for k, v in good.items()}
    r = evaluate(src)
    if exit_code(r) != 0:
        print("self-test: guarded sources did not PASS", [x for x in r if x.status != "PASS"])
        return 1
    broken = dict(src)
    broken[ROUTER] = {"path": ROUTER, "text": good[ROUTER].replace("tok >= 0 && ", "")}
    r = evaluate(broken)
    bad = [x.name for x in r if x.status == "FAIL"]
    if exit_code(r) != 1 or bad != ["hash_moe.token_table"]:
        print("self-test: missing lower bound not caught", bad)
        return 1
    if exit_code(evaluate({})) != 2:
        print("self-test: absent sources must be UNKNOWN")
        return 1
    print("self-test: ok")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--root", default=os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--self-test", action="store_true")
    a = ap.parse_args(argv)
    if a.self_test:
        return self_test()
    try:
        results = evaluate(read_sources(a.root))
    except OSError as e:
        print(f"probe error: {e}")
        return 2
    if a.json:
        print(json.dumps({"results": [asdict(r) for r in results], "summary": summary(results)}, indent=1))
    else:
        print(f"runtime ID bounds audit ({a.root})")
        for r in results:
            print(f"{r.status:7} {r.name}" + (f" [{r.path}]" if r.path else ""))
            print(f"        {r.detail}")
        print("summary: " + " ".join(f"{k}={v}" for k, v in summary(results).items()))
    return exit_code(results)


if __name__ == "__main__":
    raise SystemExit(main())
