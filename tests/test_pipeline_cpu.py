"""Pipeline parallelism on CPU (gloo ranks): the decoder cut into 2 and 3 stages gives the same greedy tokens as one
process, each stage holds only its own layers and KV caches, and a stage that begins inside an IndexCache group gets the
shared top-k rows from its predecessor."""
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
                      STK_CPU_ACT_FP32="1", CUDA_VISIBLE_DEVICES="")
    import torch.distributed as dist
    torch.set_num_threads(2)                      # several ranks share the host: tiny tensors gain nothing from more
    from stkernel_b200.config import EngineConfig, ParallelConfig, SchedulerConfig, tiny_config
    from stkernel_b200.models.dsv4 import DictSource, build_model_weights
    from stkernel_b200.models.weights import init_random_weights
    from stkernel_b200.parallel.pipeline import PipeStage, stage_starts_inside_index_group
    from stkernel_b200.runtime.engine import Engine, SamplingParams
    # five layers, ratio-4 layers at 0, 1, 3, 4 with IndexCache frequency 2: layers 1 and 4 reuse the rows of 0 and 3
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="bf16", expert_dtype="bf16", num_hidden_layers=5,
                      compress_ratios=(4, 4, 0, 4, 4), index_topk_freq=2)
    w = init_random_weights(cfg, seed=2)
    pipe = None
    rng = None
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        pipe = PipeStage(pp_rank=rank, pp_size=world)
        rng = pipe.layer_range(cfg.num_hidden_layers)
    ec = EngineConfig(model=cfg, parallel=ParallelConfig(pp_size=world),
                      sched=SchedulerConfig(max_model_len=256, max_num_seqs=2, max_num_batched_tokens=64,
                                            graph_cap=0)).validate()
    weights = build_model_weights(cfg, DictSource(w), "cpu", layer_range=rng)
    eng = Engine(ec, weights, "cpu", max_context=256, pipe=pipe)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (70, 33)]
    out = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
    info = {"out": out, "layers": [weights.layer_offset, weights.layer_offset + len(weights.layers)],
            "kv_layers": sorted(eng.kv.swa_cache.keys()),
            "starts_inside_group": stage_starts_inside_index_group(cfg, *rng) if rng else False}
    json.dump(info, open(f"{path}.{rank}", "w"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _run_pp_tp(rank, port, path, dcp=1):
    """Four ranks: two pipeline stages of two tensor-parallel ranks each (global rank = pp_rank * 2 + tp_rank), with
    the sequence-parallel residual on, so a stage boundary carries each rank's share of the token rows."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="4",
                      STK_CPU_ACT_FP32="1", STK_SEQ_PARALLEL_MIN_ROWS="4", CUDA_VISIBLE_DEVICES="")
    import torch.distributed as dist
    torch.set_num_threads(2)                      # several ranks share the host: tiny tensors gain nothing from more
    from stkernel_b200.config import EngineConfig, ParallelConfig, SchedulerConfig, tiny_config
    from stkernel_b200.models.dsv4 import DictSource, build_model_weights
    from stkernel_b200.models.weights import init_random_weights
    from stkernel_b200.parallel.communicator import Communicator
    from stkernel_b200.parallel.pipeline import PipeStage
    from stkernel_b200.runtime.engine import Engine, SamplingParams
    dist.init_process_group("gloo", rank=rank, world_size=4)
    groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]          # every rank creates every group
    pp_rank, tp_rank = divmod(rank, 2)
    comm = Communicator(group=groups[pp_rank], device="cpu", use_symm=False)
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="bf16", expert_dtype="bf16", num_hidden_layers=5,
                      compress_ratios=(4, 4, 0, 4, 4), index_topk_freq=2)
    w = init_random_weights(cfg, seed=2)
    pipe = PipeStage(pp_rank=pp_rank, pp_size=2, tp_rank=tp_rank, tp_size=2)
    ec = EngineConfig(model=cfg, parallel=ParallelConfig(tp_size=2, ep_size=2, pp_size=2, dcp_size=dcp),
                      sched=SchedulerConfig(max_model_len=256, max_num_seqs=2, max_num_batched_tokens=64,
                                            graph_cap=0)).validate()
    weights = build_model_weights(cfg, DictSource(w), "cpu", tp_rank, 2, layer_range=pipe.layer_range(cfg.num_hidden_layers))
    eng = Engine(ec, weights, "cpu", comm, tp_rank, max_context=256, pipe=pipe)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (70, 33)]
    out = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
    json.dump({"out": out, "sp_steps": eng.model.stats["sp_steps"]}, open(f"{path}.{rank}", "w"))
    dist.barrier()
    dist.destroy_process_group()


def _run_micro(rank, world, port, path):
    """Two stages, each with two engines taking turns (micro-batches in flight)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      STK_CPU_ACT_FP32="1", CUDA_VISIBLE_DEVICES="")
    import torch.distributed as dist
    torch.set_num_threads(2)                      # several ranks share the host: tiny tensors gain nothing from more
    from stkernel_b200.config import EngineConfig, ParallelConfig, SchedulerConfig, tiny_config
    from stkernel_b200.models.dsv4 import DictSource, build_model_weights
    from stkernel_b200.models.weights import init_random_weights
    from stkernel_b200.parallel.pipeline import MicroBatchPipeline, PipeStage
    from stkernel_b200.runtime.engine import Engine, SamplingParams
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="bf16", expert_dtype="bf16", num_hidden_layers=5,
                      compress_ratios=(4, 4, 0, 4, 4), index_topk_freq=2)
    w = init_random_weights(cfg, seed=2)
    pipe = PipeStage(pp_rank=rank, pp_size=world)
    ec = EngineConfig(model=cfg, parallel=ParallelConfig(pp_size=world),
                      sched=SchedulerConfig(max_model_len=256, max_num_seqs=2, max_num_batched_tokens=64,
                                            graph_cap=0)).validate()
    weights = build_model_weights(cfg, DictSource(w), "cpu", layer_range=pipe.layer_range(cfg.num_hidden_layers))
    mb = MicroBatchPipeline([Engine(ec, weights, "cpu", max_context=256, pipe=pipe) for _ in range(world)])
    g = torch.Generator().manual_seed(0)
    lens = (70, 33, 21, 90, 5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    # uneven lengths and token budgets: engines run out of work at different ticks
    ids = [mb.add_request(p, SamplingParams(temperature=0.0, max_tokens=3 + 2 * i)) for i, p in enumerate(prompts)]
    while mb.has_work():
        mb.step()
    outs = [list(mb.output(i)) for i in ids]
    # the engine surface the serving layer uses: summed counters, request lookup, release
    assert mb.metrics.generation_tokens_total == sum(len(o) for o in outs) and mb.metrics.requests_finished == len(ids)
    assert sorted(mb.requests) == ids and all(mb.requests[i].finished for i in ids)
    assert mb.abort(ids[0]) is False                    # finished already
    for i in ids:
        mb.release(i)
    assert mb.requests == {} and not mb.has_work()
    json.dump({"out": outs, "ticks": mb.tick, "overlapped": mb.overlapped_ticks},
              open(f"{path}.{rank}", "w"))
    dist.barrier()
    dist.destroy_process_group()


def _run_prefix(rank, world, port, path):
    """Stages with different layer kinds (stage 0: ratio-4 + ratio-128 layers, stage 1: a sliding-window layer only) and
    a request that starts from a cached prefix: every stage must keep and find the same entry."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      STK_CPU_ACT_FP32="1", CUDA_VISIBLE_DEVICES="")
    import torch.distributed as dist
    torch.set_num_threads(2)                      # several ranks share the host: tiny tensors gain nothing from more
    from stkernel_b200.config import EngineConfig, ParallelConfig, SchedulerConfig, tiny_config
    from stkernel_b200.models.dsv4 import DictSource, build_model_weights
    from stkernel_b200.models.weights import init_random_weights
    from stkernel_b200.parallel.pipeline import PipeStage
    from stkernel_b200.runtime.engine import Engine, SamplingParams
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="bf16", expert_dtype="bf16", num_hidden_layers=3,
                      compress_ratios=(4, 128, 0))
    w = init_random_weights(cfg, seed=2)
    pipe = rng = None
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        pipe = PipeStage(pp_rank=rank, pp_size=world)
        rng = pipe.layer_range(cfg.num_hidden_layers)
    ec = EngineConfig(model=cfg, parallel=ParallelConfig(pp_size=world),
                      sched=SchedulerConfig(max_model_len=1024, max_num_seqs=2, max_num_batched_tokens=128,
                                            graph_cap=0)).validate()
    eng = Engine(ec, build_model_weights(cfg, DictSource(w), "cpu", layer_range=rng), "cpu", max_context=1024, pipe=pipe)
    g = torch.Generator().manual_seed(0)
    base = torch.randint(0, cfg.vocab_size, (600,), generator=g).tolist()
    tail = torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=4)
    out = [eng.generate([base], sp), eng.generate([base[:520] + tail], sp)]
    json.dump({"out": out, "hits": eng.prefix_cache.hit_tokens, "c4_pages": eng.kv.c4.pages_in_use}, open(f"{path}.{rank}", "w"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _spawn(world, path):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    port = _free_port()
    ps = [ctx.Process(target=_run, args=(r, world, port, path)) for r in range(world)]
    for q in ps:
        q.start()
    for q in ps:
        q.join(240)
        assert q.exitcode == 0
    return [json.load(open(f"{path}.{r}")) for r in range(world)]


@pytest.mark.timeout(600)
def test_pipeline_stages_match_single_process(tmp_path):
    one = _spawn(1, str(tmp_path / "one"))[0]
    assert one["layers"] == [0, 5]
    for world in (2, 3):
        stages = _spawn(world, str(tmp_path / f"pp{world}"))
        # every stage ends each step with the last stage's tokens, and they are the single-process tokens
        for st in stages:
            assert st["out"] == one["out"], (world, st["layers"])
        # contiguous cover, own KV only
        assert stages[0]["layers"][0] == 0 and stages[-1]["layers"][1] == 5
        for a, b in zip(stages, stages[1:]):
            assert a["layers"][1] == b["layers"][0]
        for st in stages:
            assert st["kv_layers"] == list(range(*st["layers"]))
        # the 3-stage cut is [0,2) [2,4) [4,5): the last stage starts at layer 4, which reuses layer 3's top-k rows
        if world == 3:
            assert stages[2]["starts_inside_group"] is True


def test_pipeline_stage_arithmetic_and_guards():
    from stkernel_b200.config import EngineConfig, ParallelConfig, SchedulerConfig, tiny_config
    from stkernel_b200.models.dsv4 import DictSource, build_model_weights
    from stkernel_b200.models.weights import init_random_weights
    from stkernel_b200.parallel.pipeline import PipeStage
    from stkernel_b200.runtime.engine import Engine
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="bf16", expert_dtype="bf16")
    st = PipeStage(pp_rank=1, pp_size=2, tp_rank=1, tp_size=4)
    assert st._global(0) == 1 and st._global(1) == 5 and st.last and not st.first
    w = build_model_weights(cfg, DictSource(init_random_weights(cfg, seed=0)), "cpu")
    ec = EngineConfig(model=cfg, parallel=ParallelConfig(pp_size=2),
                      sched=SchedulerConfig(max_model_len=128, max_num_seqs=2, max_num_batched_tokens=64, graph_cap=0)).validate()
    with pytest.raises(ValueError):
        Engine(ec, w, "cpu", max_context=128)                                   # pp_size 2 without a stage
    with pytest.raises(ValueError):
        Engine(ec, w, "cpu", max_context=128, pipe=PipeStage(pp_rank=0, pp_size=2))   # the weights hold every layer


@pytest.mark.timeout(600)
@pytest.mark.parametrize("dcp", [1, 2])
def test_pipeline_stages_of_tensor_parallel_ranks(tmp_path, dcp):
    """dcp 2: each stage's two ranks also deal the ratio-4 KV pages of the stage's layers between them."""
    import torch.multiprocessing as mp
    one = _spawn(1, str(tmp_path / "one"))[0]
    ctx = mp.get_context("spawn")
    port = _free_port()
    path = str(tmp_path / "pptp")
    ps = [ctx.Process(target=_run_pp_tp, args=(r, port, path, dcp)) for r in range(4)]
    for q in ps:
        q.start()
    for q in ps:
        q.join(300)
        assert q.exitcode == 0
    got = [json.load(open(f"{path}.{r}")) for r in range(4)]
    for g_ in got:
        assert g_["out"] == one["out"]
        assert g_["sp_steps"] >= 1


@pytest.mark.timeout(600)
def test_micro_batches_in_flight_match_single_process(tmp_path):
    """Five requests of uneven length over two stages with two engines each: the texts are those of one process that
    runs each request alone, and most ticks have a step in flight while another begins."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    port = _free_port()
    path = str(tmp_path / "mb")
    ps = [ctx.Process(target=_run_micro, args=(r, 2, port, path)) for r in range(2)]
    for q in ps:
        q.start()
    for q in ps:
        q.join(400)
        assert q.exitcode == 0
    a, b = (json.load(open(f"{path}.{r}")) for r in range(2))
    assert a == b
    # reference: the whole model in this process, one request at a time
    from stkernel_b200.config import EngineConfig, SchedulerConfig, tiny_config
    from stkernel_b200.models.dsv4 import DictSource, build_model_weights
    from stkernel_b200.models.weights import init_random_weights
    from stkernel_b200.ops import functional as Fn
    from stkernel_b200.runtime.engine import Engine, SamplingParams
    Fn.set_cpu_act_dtype(torch.float32)
    try:
        cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="bf16", expert_dtype="bf16", num_hidden_layers=5,
                          compress_ratios=(4, 4, 0, 4, 4), index_topk_freq=2)
        w = init_random_weights(cfg, seed=2)
        ec = EngineConfig(model=cfg, sched=SchedulerConfig(max_model_len=256, max_num_seqs=2, max_num_batched_tokens=64,
                                                           graph_cap=0)).validate()
        eng = Engine(ec, build_model_weights(cfg, DictSource(w), "cpu"), "cpu", max_context=256)
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (70, 33, 21, 90, 5)]
        want = [eng.generate([p], SamplingParams(temperature=0.0, max_tokens=3 + 2 * i))[0] for i, p in enumerate(prompts)]
    finally:
        Fn.set_cpu_act_dtype(torch.bfloat16)
    assert a["out"] == want
    assert a["overlapped"] >= a["ticks"] // 2


@pytest.mark.timeout(600)
def test_cached_prefix_across_stages_with_different_layer_kinds(tmp_path):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    res = {}
    for world in (1, 2):
        port = _free_port()
        path = str(tmp_path / f"pfx{world}")
        ps = [ctx.Process(target=_run_prefix, args=(r, world, port, path)) for r in range(world)]
        for q in ps:
            q.start()
        for q in ps:
            q.join(300)
            assert q.exitcode == 0
        res[world] = [json.load(open(f"{path}.{r}")) for r in range(world)]
    assert res[1][0]["hits"] == 512
    assert res[2][0] == res[2][1] == res[1][0]          # texts, hit tokens and page accounting alike on every stage
