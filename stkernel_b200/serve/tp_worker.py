"""One serving process per GPU: rank 0 hosts the HTTP server, every rank runs the same engine.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m stkernel_b200.serve.tp_worker --model DIR --tensor-parallel-size N ...

The engines advance in lockstep: before each step rank 0 broadcasts the control events it drained
(new requests with their sampling parameters, aborts) over the CPU (gloo) group; every rank applies
them in the same order and calls `step()`, so schedulers, page tables and seeded samplers stay
identical and the only device collectives are the model's own.  A follower that hears nothing for
`--heartbeat-timeout` seconds exits instead of waiting forever in a collective.  With `--model`
absent, random weights of the flagship architecture are served (benchmarks, tests).

Flag names follow the reference's serve script (launchers/start-hy4-tp4.sh:354-392).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..config import CacheConfig, EngineConfig, ParallelConfig, SchedulerConfig, SpecConfig, flash_config, tiny_config
from ..runtime.engine import Engine, SamplingParams
from .api_server import AsyncEngine, create_app
from .tokenizer import ByteTokenizer, ChatTokenizer, HFTokenizer

EV_ADD, EV_ABORT, EV_STOP = 0, 1, 2


class LockstepLeader(AsyncEngine):
    """AsyncEngine whose control events are mirrored to the follower ranks before every step."""

    def __init__(self, engine: Engine, cpu_group):
        self.cpu_group = cpu_group
        self._mirror: List[Tuple[int, Any]] = []
        super().__init__(engine)

    def _broadcast(self, events: List[Tuple[int, Any]]) -> None:
        try:
            dist.broadcast_object_list([events], src=0, group=self.cpu_group)
        except RuntimeError as e:
            # a follower is gone (or the group timed out): the ranks cannot be in step any more.  Every open stream gets
            # an error and the process ends, so that the supervisor restarts the stack instead of probing a server that
            # still answers /health with nothing behind it.
            from .api_server import TokenEvent
            for rid in list(self._streams):
                self._post(rid, TokenEvent([], True, "error", error=f"control channel lost: {e}"))
            self._streams.clear()
            self.failed = f"control channel lost: {e}"
            print(f"leader: {self.failed}; stopping", file=sys.stderr)
            os._exit(3)

    def _on_add(self, rid: int, prompt: List[int], params: SamplingParams) -> None:
        self._mirror.append((EV_ADD, (list(prompt), dict(vars(params)))))

    def _on_abort(self, rid: int) -> None:
        self._mirror.append((EV_ABORT, rid))

    def _run(self) -> None:
        eng = self.engine
        idle_since = time.time()
        while not self._stop:
            self._drain_inbox()
            if not eng.has_work() and not self._mirror:
                if time.time() - idle_since > 1.0:          # heartbeat: followers know the leader is alive
                    self._broadcast([])
                    idle_since = time.time()
                self._wake.wait(timeout=0.05)
                self._wake.clear()
                continue
            self._broadcast(self._mirror)
            self._mirror = []
            idle_since = time.time()
            if not eng.has_work():
                continue
            try:
                self._publish(eng.step())
            except Exception as e:                           # a failed step ends every open stream and the job:
                from .api_server import TokenEvent          # the ranks can no longer be assumed to be in step
                for rid in list(self._streams):
                    self._post(rid, TokenEvent([], True, "error", error=f"{type(e).__name__}: {e}"))
                self._streams.clear()
                self.failed = f"{type(e).__name__}: {e}"
                print(f"leader: step failed ({self.failed}); stopping", file=sys.stderr)
                os._exit(4)
        self._broadcast([(EV_STOP, None)])


def follower_loop(engine: Engine, cpu_group, heartbeat_timeout: float = 120.0) -> int:
    """Ranks > 0: apply the leader's events, step when there is work.  Returns the exit code."""
    while True:
        box: List[Any] = [None]
        try:
            dist.broadcast_object_list(box, src=0, group=cpu_group)
        except RuntimeError as e:                           # leader gone or group timed out
            print(f"follower: control channel lost ({e}); exiting", file=sys.stderr)
            return 3
        for kind, payload in box[0] or []:
            if kind == EV_ADD:
                prompt, params = payload
                engine.add_request(prompt, SamplingParams(**params))
            elif kind == EV_ABORT:
                engine.abort(payload)
                engine.release(payload)
            elif kind == EV_STOP:
                return 0
        # The leader sends one message per step while it has work and empty heartbeats only while idle;
        # lockstep engines agree on `has_work`, so a message that finds work pending is a step.
        if engine.has_work():
            for rid in {rid for rid, _ in engine.step()}:
                engine.release(rid)                      # forgets the request once it has finished (a no-op before)


def build_engine(a, rank: int, world: int, device) -> Tuple[Engine, Any]:
    from ..models.dsv4 import RandomSource, build_model_weights
    spec_cfg = SpecConfig()
    if a.speculative_config:
        sc = json.loads(a.speculative_config)
        spec_cfg = SpecConfig(method=sc.get("method", "dspark"), num_speculative_tokens=int(sc.get("num_speculative_tokens", 5)),
                              markov_topk=int(sc.get("markov_topk", 512)), markov_sideload=os.environ.get("STK_MARKOV_SIDELOAD", ""))
    if a.model:
        from ..models.loader import CheckpointSource, load_model_config
        mcfg = load_model_config(a.model)
        src = CheckpointSource(a.model)
    else:
        n_mtp = 3 if spec_cfg.method == "dspark" else 0
        if a.tiny:
            mcfg = tiny_config(n_mtp_layers=min(n_mtp, 2), dspark_target_layer_ids=(0, 1) if n_mtp else (), dspark_markov_rank=16)
        else:
            mcfg = flash_config(a.layers, n_mtp_layers=n_mtp,
                                dspark_target_layer_ids=(a.layers // 4, a.layers // 2, a.layers - 1) if n_mtp else ())
        src = RandomSource(0)
    # ranks are laid out stage-major: global rank = pp_rank * tp + tp_rank
    pp = getattr(a, "pipeline_parallel_size", 1)
    tp = world // pp
    pp_rank, tp_rank = divmod(rank, tp)
    ecfg = EngineConfig(model=mcfg, parallel=ParallelConfig(tp_size=tp, ep_size=tp, pp_size=pp,
                                                            dcp_size=getattr(a, "decode_context_parallel_size", 1),
                                                            fused_collectives=os.environ.get("STK_FUSED_COLLECTIVES", "1") == "1"),
                        sched=SchedulerConfig(max_model_len=a.max_model_len, max_num_seqs=a.max_num_seqs,
                                              max_num_batched_tokens=a.max_num_batched_tokens, graph_cap=a.graph_cap,
                                              async_scheduling=getattr(a, "async_scheduling", False)),
                        cache=CacheConfig(gpu_memory_utilization=a.gpu_memory_utilization, size_by_memory=True),
                        spec=spec_cfg).validate()
    comm = None
    pipe = None
    layer_range = None
    if pp > 1:
        from ..parallel.pipeline import PipeStage
        pipe = PipeStage(pp_rank=pp_rank, pp_size=pp, tp_rank=tp_rank, tp_size=tp)
        layer_range = pipe.layer_range(mcfg.num_hidden_layers)
    if tp > 1:
        from ..parallel.communicator import Communicator
        group = None
        if pp > 1:
            # one tensor-parallel group per stage; every rank creates every group.  The stages' groups use the library
            # collectives (the symmetric-memory kernels are set up for one group spanning all ranks).
            groups = [dist.new_group(list(range(s * tp, (s + 1) * tp))) for s in range(pp)]
            group = groups[pp_rank]
        comm = Communicator(group=group, device=device,
                            use_symm=pp == 1 and os.environ.get("STK_ONESHOT_AR", "1") == "1" and device.type == "cuda")
    weights = build_model_weights(mcfg, src, device, tp_rank, tp, head_fp8=mcfg.dense_dtype == "fp8" and device.type == "cuda",
                                  layer_range=layer_range)
    draft = None
    if spec_cfg.method == "dspark":
        from ..spec.dspark import build_draft_weights
        draft = build_draft_weights(mcfg, src, weights, device, tp_rank, tp)
    micro = getattr(a, "pipeline_micro_batches", False)
    if pipe is not None and micro:
        # as many engines per stage as there are stages, taking turns: every stage has work while another micro-batch is
        # in flight.  They share the weights; each gets its share of the sequence slots and of the KV pools.
        from ..parallel.pipeline import MicroBatchPipeline
        share = dataclasses.replace(ecfg, sched=dataclasses.replace(ecfg.sched, max_num_seqs=max(1, ecfg.sched.max_num_seqs // pp)))
        return MicroBatchPipeline([Engine(share, weights, device, comm, tp_rank, pipe=pipe) for _ in range(pp)]), mcfg
    eng = Engine(ecfg, weights, device, comm, tp_rank, draft_weights=draft, pipe=pipe)
    return eng, mcfg


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="")
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--served-model-name", default="deepseek-v4-flash")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.6)
    ap.add_argument("--max-model-len", type=int, default=32768)
    ap.add_argument("--max-num-seqs", type=int, default=32)
    ap.add_argument("--max-num-batched-tokens", type=int, default=4096)
    ap.add_argument("--graph-cap", type=int, default=64)
    ap.add_argument("--async-scheduling", action="store_true",
                    help="launch step k+1 before the tokens of step k are read (not with speculative decoding)")
    ap.add_argument("--pipeline-parallel-size", type=int, default=1,
                    help="contiguous stages of layers; WORLD_SIZE = pipeline x tensor parallel size (stage-major ranks)")
    ap.add_argument("--pipeline-micro-batches", action="store_true",
                    help="with pipeline stages: one engine per stage and micro-batch, their steps interleaved")
    ap.add_argument("--decode-context-parallel-size", type=int, default=1,
                    help="1, or the tensor-parallel size: the ratio-4 KV caches are dealt page by page over the ranks")
    ap.add_argument("--kv-cache-dtype", default="fp8_ds_mla")
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--speculative-config", default="")
    ap.add_argument("--default-chat-template-kwargs", default="")
    ap.add_argument("--default-thinking", action="store_true", help="requests think unless they say otherwise")
    ap.add_argument("--profiler-dir", default="/tmp/stk_profiles")
    ap.add_argument("--layers", type=int, default=2, help="random-weight mode: decoder layers")
    ap.add_argument("--tiny", action="store_true", help="random-weight mode: CPU-sized architecture")
    ap.add_argument("--heartbeat-timeout", type=float, default=120.0)
    a = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if a.tensor_parallel_size * a.pipeline_parallel_size != world:
        print(f"ABORT: --tensor-parallel-size {a.tensor_parallel_size} x --pipeline-parallel-size "
              f"{a.pipeline_parallel_size} but WORLD_SIZE={world}", file=sys.stderr)
        return 2
    use_cuda = torch.cuda.is_available()
    device = torch.device(f"cuda:{local}" if use_cuda else "cpu")
    cpu_group = None
    if world > 1:
        import datetime
        if use_cuda:
            torch.cuda.set_device(device)
        dist.init_process_group("nccl" if use_cuda else "gloo", timeout=datetime.timedelta(seconds=max(600, a.heartbeat_timeout)))
        cpu_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=a.heartbeat_timeout))
    eng, mcfg = build_engine(a, rank, world, device)
    if rank != 0:
        return follower_loop(eng, cpu_group, a.heartbeat_timeout)
    import uvicorn
    tok = ChatTokenizer(HFTokenizer(a.tokenizer or a.model) if (a.tokenizer or a.model) else ByteTokenizer(mcfg.vocab_size))
    kwargs = json.loads(a.default_chat_template_kwargs) if a.default_chat_template_kwargs else None
    app = create_app(eng, tok, a.served_model_name, default_thinking=a.default_thinking, profile_dir=a.profiler_dir,
                     default_chat_template_kwargs=kwargs,
                     async_engine=LockstepLeader(eng, cpu_group) if world > 1 else None,
                     default_temperature=a.temperature)
    uvicorn.run(app, host=a.host, port=a.port, log_level="info")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
