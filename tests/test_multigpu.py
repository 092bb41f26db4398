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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_moe_over_peer_memory():
    """Route/dispatch/grouped GEMM/return/combine against the fp32 reference (32 experts so that every rank
    can hold all dequantised weights), two calls in a row with different routing."""
    env = dict(os.environ)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29532", os.path.join(ROOT, "tests", "multigpu", "ep_check.py"), "--experts", "32",
           "--tokens", "1,16", "--check-tokens", "48"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert "EP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_folded_allreduce_sharded_argmax_and_engine_across_ranks():
    """Producer/consumer all-reduce, vocabulary-sharded arg-max and a tensor-parallel engine with every decode fusion
    on, against library collectives.  NVLS off: a rank that fails must not leave multicast bindings behind."""
    r = _torchrun(os.path.join(ROOT, "tests", "multigpu", "ll_check.py"), 2, 29533, timeout=420,
                  extra_env={"NCCL_NVLS_ENABLE": "0"})
    assert "LL_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_decode_context_parallel_engine_across_ranks():
    """The ratio-4 caches dealt page by page over two ranks against the same engine with replicated caches."""
    r = _torchrun(os.path.join(ROOT, "tests", "multigpu", "dcp_check.py"), 2, 29534, timeout=420,
                  extra_env={"NCCL_NVLS_ENABLE": "0"})
    assert "DCP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pipeline_stages_across_two_gpus():
    """Two pipeline stages on two GPUs against the whole model on one."""
    r = _torchrun(os.path.join(ROOT, "tests", "multigpu", "pp_check.py"), 2, 29535, timeout=420,
                  extra_env={"NCCL_NVLS_ENABLE": "0"})
    assert "PP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
