"""Launch the serving stack on one node: validate knobs, attest the tree, start one rank per GPU.

    python -m stkernel_b200.fleet.launcher [--dry-run] [--manifest PATH] [--no-attest]

Order of work, each stage failing closed before the next (reference: launchers/start-hy4-tp4.sh:16-118
knobs, :217-259 manifest, :274-337 preflight, :354-392 serve flags, :395-421 launch):

1. knobs from the environment -> exit 2 with an `ABORT:` line on the first bad value;
2. manifest parse + SHA-256 of every listed file + no unlisted files -> exit 1 on skew;
3. preflight: model directory, sideload payload, visible GPU count;
4. the command: `torch.distributed.run --nproc-per-node TP` over the loopback rendezvous running
   `stkernel_b200.serve.tp_worker` (rank 0 also hosts the HTTP server), env from the knobs.

Nothing here touches a GPU setting: clocks, power limits and persistence mode stay as found.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

from . import manifest as M
from .knobs import EXIT_BAD_KNOB, KnobError, Knobs, parse_knobs


def repo_root() -> str:
    return os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def attest(root: str, manifest_path: str) -> str:
    """Returns the inventory fingerprint; raises ManifestError on any skew."""
    if not os.path.isfile(manifest_path):
        raise M.ManifestError(f"ABORT: manifest missing ({manifest_path})")
    with open(manifest_path) as f:
        entries = M.parse(f.read())
    n, problems = M.verify(root, entries)
    extra = M.unlisted(root, entries)
    problems += [f"unlisted file in tree: {p}" for p in extra]
    if problems:
        raise M.ManifestError("ABORT: tree does not match manifest:\n  " + "\n  ".join(problems))
    return M.fingerprint(entries)


def preflight(k: Knobs, gpu_count: Optional[int] = None) -> List[str]:
    problems = []
    if not k.model_path:
        problems.append("MODEL_PATH is not set")
    elif not os.path.isfile(os.path.join(k.model_path, "config.json")):
        problems.append(f"model config missing ({k.model_path}/config.json)")
    if k.markov_sideload and not os.path.isfile(k.markov_sideload):
        problems.append(f"MARKOV_SIDELOAD missing ({k.markov_sideload})")
    if gpu_count is not None and gpu_count < k.tp_size * k.pp_size:
        problems.append(f"TP_SIZE={k.tp_size} x PP_SIZE={k.pp_size} but only {gpu_count} GPU(s) visible")
    return problems


def serve_command(k: Knobs, python: str = sys.executable) -> List[str]:
    cmd = [python, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={k.tp_size * k.pp_size}",
           "--master-addr", "127.0.0.1", "--master-port", "29400",
           "-m", "stkernel_b200.serve.tp_worker",
           "--model", k.model_path, "--served-model-name", k.served_name, "--port", str(k.port),
           "--tensor-parallel-size", str(k.tp_size), "--gpu-memory-utilization", str(k.gpu_mem),
           "--max-model-len", str(k.max_model_len), "--max-num-seqs", str(k.max_num_seqs),
           "--max-num-batched-tokens", str(k.max_num_batched), "--graph-cap", str(k.graph_cap),
           "--kv-cache-dtype", "fp8_ds_mla", "--temperature", str(k.temperature)]
    if k.pp_size > 1:
        cmd += ["--pipeline-parallel-size", str(k.pp_size), "--pipeline-micro-batches"]
    if k.async_sched:
        cmd += ["--async-scheduling"]
    if k.dcp:
        cmd += ["--decode-context-parallel-size", str(k.tp_size)]
    if k.spec_tokens:
        cmd += ["--speculative-config", json.dumps({"method": "dspark", "num_speculative_tokens": k.spec_tokens,
                                                   "draft_sample_method": "probabilistic", "markov_topk": k.markov_topk})]
    if k.effort:
        cmd += ["--default-chat-template-kwargs", json.dumps({"reasoning_effort": k.effort})]
    if k.dev_mode:
        cmd += ["--profiler-dir", "/tmp/stk_profiles"]
    return cmd


def main(argv: Optional[Sequence[str]] = None, env: Optional[Mapping[str, str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dry-run", action="store_true", help="validate and print the command; start nothing")
    ap.add_argument("--manifest", default=None)
    ap.add_argument("--no-attest", action="store_true", help="skip the SHA-256 attestation (development trees)")
    a = ap.parse_args(argv)
    env = dict(os.environ if env is None else env)
    try:
        k = parse_knobs(env)
    except KnobError as e:
        print(str(e))
        return EXIT_BAD_KNOB
    for w in k.warnings:
        print(f"WARN: {w}")
    root = repo_root()
    fp = "unattested"
    if not a.no_attest:
        try:
            fp = attest(root, a.manifest or os.path.join(root, "stkernel_b200", "fleet", M.MANIFEST_NAME))
        except M.ManifestError as e:
            print(str(e))
            return 1
    gpus = None
    if not a.dry_run:
        import torch
        gpus = torch.cuda.device_count()
    problems = preflight(k, gpus)
    if problems and not a.dry_run:
        print("ABORT: preflight failed:\n  " + "\n  ".join(problems))
        return 1
    cmd = serve_command(k)
    print(f"preflight OK (inventory {fp[:19]}, TP={k.tp_size})")
    if a.dry_run:
        print(json.dumps({"cmd": cmd, "env": k.to_env(), "preflight": problems}, indent=1))
        return 0
    child_env = dict(os.environ)
    child_env.update(k.to_env())
    return subprocess.call(cmd, env=child_env)


if __name__ == "__main__":
    raise SystemExit(main())
