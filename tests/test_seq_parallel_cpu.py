"""Large-step paths under tensor parallelism on CPU (two gloo ranks): sequence-parallel residual (all-gather /
reduce-scatter around each sub-block), token-parallel attention (q / output all-to-all) and the sequence-parallel
indexer give the same greedy tokens as one rank, and they are the paths that actually ran."""
import json
import os
import socket

import pytest
import torch


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(rank, world, port, path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      STK_CPU_ACT_FP32="1", STK_INDEXER_SP_MIN_ROWS="4", STK_MLA_TP_MIN_ROWS="4",
                      STK_SEQ_PARALLEL_MIN_ROWS="4", CUDA_VISIBLE_DEVICES="")
    import torch.distributed as dist
    torch.set_num_threads(2)                      # several ranks share the host: tiny tensors gain nothing from more
    from stkernel_b200.config import EngineConfig, ParallelConfig, SchedulerConfig, tiny_config
    from stkernel_b200.models.dsv4 import DictSource, build_model_weights
    from stkernel_b200.models.weights import init_random_weights
    from stkernel_b200.runtime.engine import Engine, SamplingParams
    comm = None
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from stkernel_b200.parallel.communicator import Communicator
        comm = Communicator(device="cpu", use_symm=False)
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="bf16", expert_dtype="bf16")
    w = init_random_weights(cfg, seed=1)
    ec = EngineConfig(model=cfg, parallel=ParallelConfig(tp_size=world, ep_size=world),
                      sched=SchedulerConfig(max_model_len=256, max_num_seqs=2, max_num_batched_tokens=64,
                                            graph_cap=0)).validate()
    eng = Engine(ec, build_model_weights(cfg, DictSource(w), "cpu", rank, world), "cpu", comm, rank, max_context=256)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (40, 33)]
    out = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
    if rank == 0:
        json.dump({"out": out, "stats": eng.model.stats}, open(path, "w"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_sequence_parallel_paths_match_single_rank(tmp_path):
    import torch.multiprocessing as mp
    one, two = str(tmp_path / "one.json"), str(tmp_path / "two.json")
    ctx = mp.get_context("spawn")
    p = ctx.Process(target=_run, args=(0, 1, _free_port(), one))
    p.start()
    p.join(240)
    assert p.exitcode == 0
    port = _free_port()
    ps = [ctx.Process(target=_run, args=(r, 2, port, two)) for r in range(2)]
    for q in ps:
        q.start()
    for q in ps:
        q.join(240)
        assert q.exitcode == 0
    a, b = json.load(open(one)), json.load(open(two))
    assert a["out"] == b["out"]
    assert a["stats"]["sp_steps"] == 0
    assert b["stats"]["sp_steps"] >= 1 and b["stats"]["mla_token_parallel_calls"] >= 1
