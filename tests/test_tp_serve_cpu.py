"""Multi-rank serving on CPU (gloo): lockstep leader/followers behind the HTTP server, and the follower's
exit when the leader disappears between steps (host-side failure, no device involved)."""
import json
import os
import signal
import socket
import subprocess
import sys
import time
import urllib.error
import urllib.request

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _post(port, path, body, timeout=120):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def _wait_up(port, proc, timeout=180):
    t0 = time.time()
    while time.time() - t0 < timeout:
        if proc.poll() is not None:
            raise RuntimeError(f"server exited early with {proc.returncode}")
        try:
            urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2).read()
            return
        except OSError:
            time.sleep(0.5)
    raise TimeoutError("server did not come up")


def _launch(world, port, extra=(), tp=None):
    # tiny thresholds so that the prompt's prefill step takes the sequence-parallel indexer path and the
    # token-parallel attention path (q / output all-to-all) at world 2, and (for a prompt of even length) the
    # sequence-parallel residual (all-gather / reduce-scatter around each sub-block)
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2", STK_CPU_ACT_FP32="1",
               STK_INDEXER_SP_MIN_ROWS="4", STK_MLA_TP_MIN_ROWS="4",
               STK_SEQ_PARALLEL_MIN_ROWS="4")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), "-m", "stkernel_b200.serve.tp_worker", "--tiny", "--port", str(port),
           "--tensor-parallel-size", str(tp if tp is not None else world), "--max-model-len", "512", "--max-num-seqs", "4",
           "--max-num-batched-tokens", "128", "--graph-cap", "0", "--heartbeat-timeout", "20", *extra]
    return subprocess.Popen(cmd, env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, start_new_session=True)


def _stop(proc):
    if proc.poll() is None:
        os.killpg(proc.pid, signal.SIGTERM)          # exactly the process group this test started
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)


@pytest.mark.timeout(600)
def test_tp2_lockstep_serving_matches_tp1():
    body = {"prompt": "lockstep serving over two ranks, with a prompt long enough to fill compressed rows", "max_tokens": 8,
            "temperature": 0, "ignore_eos": True}
    outs = {}
    # the third server also deals the ratio-4 KV pages over its two ranks (decode context parallelism); the fourth
    # runs its two ranks as two pipeline stages of one layer each; the fifth launches every step before the previous
    # one's tokens are read (leader and follower must still take the same steps); the sixth runs two engines per stage
    # with their steps interleaved (micro-batches in flight).  All six run side by side.
    configs = ((1, 1, (), None), (2, 2, (), None), ("dcp", 2, ("--decode-context-parallel-size", "2"), None),
               ("pp", 2, ("--pipeline-parallel-size", "2"), 1), ("async", 2, ("--async-scheduling",), None),
               ("ppmb", 2, ("--pipeline-parallel-size", "2", "--pipeline-micro-batches"), 1))
    servers = []
    lps = {}
    try:
        for key, world, extra, tp in configs:
            port = _free_port()
            servers.append((key, port, _launch(world, port, extra, tp)))
        for key, port, proc in servers:
            _wait_up(port, proc)
            r1 = _post(port, "/v1/completions", body)
            r2 = _post(port, "/v1/completions", body)
            assert r1["usage"]["completion_tokens"] == 8
            assert r1["choices"][0]["text"] == r2["choices"][0]["text"]           # followers stayed in step
            chat = _post(port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                                                        "temperature": 0.7, "seed": 3, "ignore_eos": True})
            assert chat["usage"]["completion_tokens"] == 4
            # one character more: of the two prompt lengths one is even, which the sequence-parallel residual needs
            r3 = _post(port, "/v1/completions", dict(body, prompt="!" + body["prompt"][::-1]))
            outs[key] = (r1["choices"][0]["text"], r3["choices"][0]["text"])
            lp_body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "temperature": 0, "ignore_eos": True,
                       "logprobs": True, "top_logprobs": 2}
            if key in (1, 2, "dcp"):
                lp = _post(port, "/v1/chat/completions", lp_body)["choices"][0]["logprobs"]["content"]
                lps[key] = [(e["token"], e["logprob"]) for e in lp]
            else:
                # stages and the asynchronous scheduler do not report log-probabilities: a clear refusal
                try:
                    _post(port, "/v1/chat/completions", lp_body)
                    refused = False
                except urllib.error.HTTPError as e:
                    refused = e.code == 400
                assert refused
    finally:
        for _, _, proc in servers:
            _stop(proc)
    # the same weights split over two ranks give the same greedy text (fp32 activations on CPU)
    assert outs[1] == outs[2] == outs["dcp"] == outs["pp"] == outs["async"] == outs["ppmb"]
    # log-probabilities over two ranks (logits gathered) are those of one rank
    for key in (2, "dcp"):
        assert [t for t, _ in lps[key]] == [t for t, _ in lps[1]]
        assert all(abs(a - b) < 1e-3 for (_, a), (_, b) in zip(lps[key], lps[1]))


@pytest.mark.timeout(300)
def test_single_process_entry_point_serves():
    """`python -m stkernel_b200.serve.api_server`: the one-device command of the quick start."""
    port = _free_port()
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2", STK_CPU_ACT_FP32="1")
    cmd = [sys.executable, "-m", "stkernel_b200.serve.api_server", "--tiny", "--port", str(port), "--max-model-len", "512",
           "--max-num-seqs", "2", "--max-num-batched-tokens", "128", "--graph-cap", "0", "--default-thinking"]
    proc = subprocess.Popen(cmd, env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, start_new_session=True)
    try:
        _wait_up(port, proc)
        r = _post(port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                                                 "temperature": 0, "ignore_eos": True})
        assert r["usage"]["completion_tokens"] == 4 and r["choices"][0]["finish_reason"] == "length"
    finally:
        _stop(proc)


def _follower_main(rank, port, result_path):
    import datetime
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="2")
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=10))
    if rank == 0:
        # a leader that sends one heartbeat and then dies between steps, without the STOP event
        dist.broadcast_object_list([[]], src=0)
        os._exit(0)
    from stkernel_b200.serve.tp_worker import follower_loop

    class Idle:
        def has_work(self): return False
    t0 = time.time()
    rc = follower_loop(Idle(), dist.group.WORLD, 10.0)
    open(result_path, "w").write(json.dumps({"rc": rc, "dt": time.time() - t0}))
    os._exit(0)


@pytest.mark.timeout(120)
def test_follower_exits_when_leader_dies(tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    res = str(tmp_path / "res.json")
    ctx = mp.get_context("spawn")
    ps = [ctx.Process(target=_follower_main, args=(r, port, res)) for r in range(2)]
    for p in ps:
        p.start()
    for p in ps:
        p.join(90)
        assert not p.is_alive()
    out = json.load(open(res))
    assert out["rc"] == 3 and out["dt"] < 60


def _leader_main(rank, port):
    import datetime
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="2")
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=10))
    if rank == 1:
        # a follower that takes one heartbeat and then dies
        box = [None]
        dist.broadcast_object_list(box, src=0)
        os._exit(0)
    import types
    from stkernel_b200.runtime.metrics import Metrics
    from stkernel_b200.serve.tp_worker import LockstepLeader
    idle = types.SimpleNamespace(has_work=lambda: False, requests={}, metrics=Metrics())
    LockstepLeader(idle, dist.group.WORLD)            # its thread sends heartbeats; the second one finds nobody
    time.sleep(60)
    os._exit(0)                                       # not reached: the leader ends the process with code 3


@pytest.mark.timeout(120)
def test_leader_exits_when_a_follower_dies():
    import torch.multiprocessing as mp
    port = _free_port()
    ctx = mp.get_context("spawn")
    ps = [ctx.Process(target=_leader_main, args=(r, port)) for r in range(2)]
    t0 = time.time()
    for p in ps:
        p.start()
    for p in ps:
        p.join(90)
        assert not p.is_alive()
    assert ps[0].exitcode == 3 and ps[1].exitcode == 0 and time.time() - t0 < 50
