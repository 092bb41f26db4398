"""Multi-GPU checks run as child processes under torchrun (skipped with fewer than 2 GPUs)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(script, nproc, port, timeout=300, extra_env=None):
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), script]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_symmetric_allreduce_and_fused_gemm():
    r = _torchrun(os.path.join(ROOT, "tests", "multigpu", "symm_check.py"), 2, 29531)
    assert "SYMM_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
