"""Source/binary manifest: the one inventory of what a deployment runs, with SHA-256 per file.

A TSV of three fields per row -- `path<TAB>kind<TAB>sha256` -- generated from the tree and verified
before launch and after every copy, so list skew, a missing file and byte skew all fail closed.  Same
invariants as the reference's overlay manifest (launchers/start-hy4-tp4.sh:217-259: exactly three fields,
safe characters, targets confined to one root, valid hashes, no duplicates, not empty) and its
hash-everything check (:317-320); here the targets are this package's own sources and its built
library instead of files bind-mounted over an image.
"""
from __future__ import annotations

import hashlib
import os
import re
from dataclasses import dataclass
from typing import Dict, Iterable, List, Sequence, Tuple

MANIFEST_NAME = "manifest.tsv"
KINDS = ("py", "cuda", "lib", "data")
_SAFE = re.compile(r"^[A-Za-z0-9_./-]+$")
_SHA = re.compile(r"^[0-9a-f]{64}$")
# files whose absence must never pass silently: the speculative-decoding path changes what is sampled from
PINNED = ("stkernel_b200/spec/dspark.py", "stkernel_b200/ops/sampling.py", "stkernel_b200/csrc/sampler.cu",
          "stkernel_b200/serve/encoding.py", "stkernel_b200/runtime/engine.py")


class ManifestError(RuntimeError):
    pass


@dataclass(frozen=True)
class Entry:
    path: str
    kind: str
    sha256: str


def sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def _kind_of(path: str) -> str:
    if path.endswith(".py"):
        return "py"
    if path.endswith((".cu", ".cuh", ".h")):
        return "cuda"
    if path.endswith(".so"):
        return "lib"
    return "data"


def collect(root: str, package: str = "stkernel_b200") -> List[Entry]:
    """Every source of the package and its built library, sorted by path."""
    out: List[Entry] = []
    base = os.path.join(root, package)
    for d, dirs, files in os.walk(base):
        dirs[:] = sorted(x for x in dirs if x != "__pycache__")
        for f in sorted(files):
            if f.endswith((".py", ".cu", ".cuh", ".h", ".so", ".tsv", ".service", ".timer")) and f != MANIFEST_NAME:
                rel = os.path.relpath(os.path.join(d, f), root)
                out.append(Entry(rel, _kind_of(rel), sha256_file(os.path.join(root, rel))))
    return sorted(out, key=lambda e: e.path)


def dumps(entries: Iterable[Entry]) -> str:
    lines = ["# path\tkind\tsha256"]
    lines += [f"{e.path}\t{e.kind}\t{e.sha256}" for e in entries]
    return "\n".join(lines) + "\n"


def parse(text: str, root_prefix: str = "stkernel_b200/") -> List[Entry]:
    """Parse and check the structural invariants (no file access)."""
    out: List[Entry] = []
    seen = set()
    for n, line in enumerate(text.splitlines(), 1):
        if not line.strip() or line.startswith("#"):
            continue
        parts = line.split("\t")
        if len(parts) != 3 or not all(parts):
            raise ManifestError(f"ABORT: malformed manifest row {n}: {line!r}")
        path, kind, sha = parts
        if not _SAFE.match(path) or path.startswith(("/", ".")) or ".." in path:
            raise ManifestError(f"ABORT: unsafe path in manifest: {path}")
        if not path.startswith(root_prefix):
            raise ManifestError(f"ABORT: manifest path outside {root_prefix}: {path}")
        if kind not in KINDS:
            raise ManifestError(f"ABORT: unknown kind in manifest row {n}: {kind}")
        if not _SHA.match(sha):
            raise ManifestError(f"ABORT: invalid sha256 for {path}: {sha}")
        if path in seen:
            raise ManifestError(f"ABORT: duplicate path in manifest: {path}")
        seen.add(path)
        out.append(Entry(path, kind, sha))
    if not out:
        raise ManifestError("ABORT: manifest is empty")
    missing = [p for p in PINNED if p not in seen]
    if missing:
        raise ManifestError(f"ABORT: pinned files missing from manifest: {missing}")
    return out


def verify(root: str, entries: Sequence[Entry], require_lib: bool = True) -> Tuple[int, List[str]]:
    """Hash every listed file under `root`; returns (files checked, problems)."""
    problems: List[str] = []
    for e in entries:
        full = os.path.join(root, e.path)
        if not os.path.isfile(full) or os.path.islink(full):
            problems.append(f"missing or not a regular file: {e.path}")
            continue
        got = sha256_file(full)
        if got != e.sha256:
            problems.append(f"byte skew: {e.path} expected {e.sha256[:12]} got {got[:12]}")
    if require_lib and not any(e.kind == "lib" for e in entries):
        problems.append("no built library (kind=lib) in manifest")
    return len(entries), problems


def fingerprint(entries: Sequence[Entry]) -> str:
    """One hash over the whole inventory: equal on two hosts iff they run the same bytes."""
    h = hashlib.sha256()
    for e in sorted(entries, key=lambda x: x.path):
        h.update(f"{e.path}\t{e.sha256}\n".encode())
    return h.hexdigest()


def unlisted(root: str, entries: Sequence[Entry], package: str = "stkernel_b200") -> List[str]:
    """Files that exist in the tree but not in the manifest (list skew in the other direction)."""
    listed = {e.path for e in entries}
    return [e.path for e in collect(root, package) if e.path not in listed]
