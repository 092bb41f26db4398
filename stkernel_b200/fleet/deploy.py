"""Gate, then install: nothing is copied unless the tree compiles, audits clean and passes its tests.

    python -m stkernel_b200.fleet.deploy --dest /opt/stk [--write-manifest] [--skip-tests]

Gates, in order (reference: launchers/deploy-overlays.sh:58-77): byte-compile every Python source;
runtime-guard audit self-test and audit of the tree; the CPU test suite.  Then the manifest is
(re)generated, every listed file is copied to the destination and re-hashed there; one mismatch
aborts (:79-97).  With several destinations (one per host mount) every copy must produce the same
inventory fingerprint.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from typing import List, Optional, Sequence, Tuple

from . import audit_guards
from . import manifest as M
from .launcher import repo_root


def gate_compile(root: str) -> List[str]:
    bad = []
    for e in M.collect(root):
        if e.kind == "py":
            try:
                with open(os.path.join(root, e.path), "rb") as f:
                    compile(f.read(), e.path, "exec")          # syntax check only; writes no .pyc
            except SyntaxError as ex:
                bad.append(f"{e.path}:{ex.lineno}: {ex.msg}")
    return bad


def gate_audit(root: str) -> Optional[str]:
    if audit_guards.self_test() != 0:
        return "guard audit self-test failed"
    rc = audit_guards.exit_code(audit_guards.evaluate(audit_guards.read_sources(root)))
    return None if rc == 0 else f"guard audit exit code {rc}"


def gate_tests(root: str) -> Optional[str]:
    rc = subprocess.call([sys.executable, "-m", "pytest", os.path.join(root, "tests"), "-x", "-q", "-m", "not gpu"], cwd=root)
    return None if rc == 0 else f"CPU tests failed (exit {rc})"


def write_manifest(root: str) -> Tuple[str, List[M.Entry]]:
    entries = M.collect(root)
    path = os.path.join(root, "stkernel_b200", "fleet", M.MANIFEST_NAME)
    with open(path, "w") as f:
        f.write(M.dumps(entries))
    return path, entries


def install(root: str, entries: Sequence[M.Entry], dest: str) -> str:
    """Copy + verify; returns the inventory fingerprint of the destination."""
    for e in entries:
        dst = os.path.join(dest, e.path)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(root, e.path), dst)
    man_dst = os.path.join(dest, "stkernel_b200", "fleet", M.MANIFEST_NAME)
    os.makedirs(os.path.dirname(man_dst), exist_ok=True)
    with open(man_dst, "w") as f:
        f.write(M.dumps(entries))
    _, problems = M.verify(dest, entries, require_lib=False)
    if problems:
        raise M.ManifestError("ABORT: verify failed on " + dest + ":\n  " + "\n  ".join(problems))
    return M.fingerprint(entries)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dest", action="append", default=[])
    ap.add_argument("--write-manifest", action="store_true")
    ap.add_argument("--skip-tests", action="store_true")
    a = ap.parse_args(argv)
    root = repo_root()
    bad = gate_compile(root)
    if bad:
        print("ABORT: sources do not compile:\n  " + "\n  ".join(bad))
        return 1
    err = gate_audit(root)
    if err:
        print(f"ABORT: {err}")
        return 1
    if not a.skip_tests:
        err = gate_tests(root)
        if err:
            print(f"ABORT: {err}")
            return 1
    path, entries = write_manifest(root)
    print(f"manifest: {len(entries)} files -> {path} (inventory {M.fingerprint(entries)[:19]})")
    fps = set()
    for d in a.dest:
        try:
            fps.add(install(root, entries, d))
        except M.ManifestError as e:
            print(str(e))
            return 1
        print(f"=== {d}: verified")
    if len(fps) > 1:
        print("ABORT: destinations disagree on the inventory fingerprint")
        return 1
    if a.dest:
        print(f"{len(entries)} files + manifest deployed and SHA-256 verified on {len(a.dest)} destination(s); "
              "restart to apply: systemctl --user restart stk-b200")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
