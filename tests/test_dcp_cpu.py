"""Decode context parallelism on CPU (two gloo ranks): the ratio-4 caches dealt page by page over the ranks, every rank
scoring its own indexer keys, the candidates merged across ranks and the selected latent rows staged on every rank give
the same greedy tokens as one rank that holds everything; each rank allocates only its own pages."""
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


def _run(rank, world, port, path, kv_dtype, stage_mb, shared_prefix=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      STK_CPU_ACT_FP32="1", STK_DCP_STAGE_MB=stage_mb, CUDA_VISIBLE_DEVICES="")
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
    # three layers: the ratio-4 layers 0 and 2 share one top-k list (IndexCache), so a reusing layer stages rows too
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype=kv_dtype, expert_dtype="bf16", num_hidden_layers=3,
                      compress_ratios=(4, 0, 4), index_topk_freq=2)
    w = init_random_weights(cfg, seed=1)
    ec = EngineConfig(model=cfg, parallel=ParallelConfig(tp_size=world, ep_size=world, dcp_size=world),
                      sched=SchedulerConfig(max_model_len=1024, max_num_seqs=2, max_num_batched_tokens=128,
                                            graph_cap=0)).validate()
    eng = Engine(ec, build_model_weights(cfg, DictSource(w), "cpu", rank, world), "cpu", comm, rank, max_context=1024)
    g = torch.Generator().manual_seed(0)
    # 4 tokens per compressed row, 64 rows per page: 530 tokens reach the third page of the ratio-4 caches
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (530, 270)]
    hits = None
    if shared_prefix:
        # a finished request leaves its first 512 tokens (two pages of compressed rows: one per rank) in the prefix
        # cache; the next request starts from them
        first = eng.generate([prompts[0][:600]], SamplingParams(temperature=0.0, max_tokens=3))
        prompts = [prompts[0][:520] + prompts[1][:90]]
    rows = [eng.add_request(p, SamplingParams(temperature=0.0, max_tokens=5)) for p in prompts]
    peak = 0
    while eng.has_work():
        eng.step()
        peak = max(peak, eng.kv.c4.pages_in_use)
    out = [list(eng.requests[r].output) for r in rows]
    if shared_prefix:
        out = first + out
    json.dump({"out": out, "prefix_hit_tokens": eng.prefix_cache.hit_tokens if eng.prefix_cache is not None else -1, "stats": eng.model.stats, "c4_peak": peak, "c4_pool": eng.kv.c4.num_pages},
              open(f"{path}.{rank}", "w"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _spawn_all(runs):
    """runs: [(world, path, kv_dtype, stage_mb, shared_prefix)], started together; -> the ranks' results of each run."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    procs = []
    for world, path, kv_dtype, stage_mb, shared_prefix in runs:
        port = _free_port()
        procs.append([ctx.Process(target=_run, args=(r, world, port, path, kv_dtype, stage_mb, shared_prefix)) for r in range(world)])
    for ps in procs:
        for q in ps:
            q.start()
    for ps in procs:
        for q in ps:
            q.join(500)
            assert q.exitcode == 0
    return [[json.load(open(f"{run[1]}.{r}")) for r in range(run[0])] for run in runs]


@pytest.mark.timeout(900)
@pytest.mark.parametrize("kv_dtype", ["bf16", "fp8_ds_mla"])
def test_context_parallel_decode_matches_one_rank(tmp_path, kv_dtype):
    # the bf16 run has a staging budget of zero megabytes, which forces one token per staging call (the block loop of
    # large steps); the fp8 run stages a whole step at once
    (one,), two = _spawn_all([(1, str(tmp_path / "one"), kv_dtype, "64", False),
                              (2, str(tmp_path / "two"), kv_dtype, "0" if kv_dtype == "bf16" else "64", False)])
    assert one["stats"]["dcp_topk_merges"] == 0
    for r in two:
        assert r["out"] == one["out"]
        assert r["stats"]["dcp_topk_merges"] >= 1
    # 530 + 270 tokens fill 3 + 2 pages of compressed rows: the single rank holds all 5, rank 0 pages 0 and 2 of the
    # first request and page 0 of the second, rank 1 the two pages numbered 1
    assert one["c4_peak"] == 5
    assert [r["c4_peak"] for r in two] == [3, 2]
    assert all(r["c4_pool"] < one["c4_pool"] for r in two)


@pytest.mark.timeout(900)
def test_context_parallel_with_a_cached_prefix(tmp_path):
    (one,), two = _spawn_all([(1, str(tmp_path / "one"), "bf16", "64", True), (2, str(tmp_path / "two"), "bf16", "64", True)])
    assert one["prefix_hit_tokens"] == 512
    for r in two:
        assert r["prefix_hit_tokens"] == 512
        assert r["out"] == one["out"]


def _run_spec(rank, world, port, path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      STK_CPU_ACT_FP32="1", CUDA_VISIBLE_DEVICES="")
    import torch.distributed as dist
    torch.set_num_threads(2)                      # several ranks share the host: tiny tensors gain nothing from more
    from stkernel_b200.config import EngineConfig, ParallelConfig, SchedulerConfig, SpecConfig, tiny_config
    from stkernel_b200.models.dsv4 import DictSource, build_model_weights
    from stkernel_b200.models.weights import init_random_weights
    from stkernel_b200.runtime.engine import Engine, SamplingParams
    from stkernel_b200.spec import dspark as DS
    comm = None
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from stkernel_b200.parallel.communicator import Communicator
        comm = Communicator(device="cpu", use_symm=False)
    cfg = tiny_config(n_mtp_layers=2, dspark_target_layer_ids=(0, 1), dspark_markov_rank=16, dense_dtype="bf16",
                      kv_cache_dtype="bf16", expert_dtype="bf16")
    w = init_random_weights(cfg, seed=0)
    tw = build_model_weights(cfg, DictSource(w), "cpu", rank, world)
    # one rank: plain decoding; two ranks: speculative decoding over context-parallel caches
    spec = SpecConfig(method="dspark", num_speculative_tokens=3, markov_topk=8) if world > 1 else SpecConfig()
    dw = DS.build_draft_weights(cfg, DictSource(w), tw, "cpu", rank, world) if world > 1 else None
    ec = EngineConfig(model=cfg, parallel=ParallelConfig(tp_size=world, ep_size=world, dcp_size=world), spec=spec,
                      sched=SchedulerConfig(max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=96,
                                            graph_cap=0)).validate()
    eng = Engine(ec, tw, "cpu", comm, rank, max_context=1024, draft_weights=dw)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (300, 150, 7)]
    out = eng.generate(prompts, SamplingParams(temperature=0.8, seed=11, max_tokens=10))
    json.dump({"out": out, "drafts": eng.metrics.spec_num_drafts}, open(f"{path}.{rank}", "w"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(900)
def test_speculative_decoding_over_context_parallel_caches(tmp_path):
    """Verify rows, rollbacks of rejected rows and the draft layers with the ratio-4 pages dealt over two ranks: the
    sampled text (fixed seeds) equals plain decoding on one rank."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    res, procs = {}, {}
    for world in (1, 2):
        port = _free_port()
        procs[world] = [ctx.Process(target=_run_spec, args=(r, world, port, str(tmp_path / f"w{world}"))) for r in range(world)]
        for q in procs[world]:
            q.start()
    for world in (1, 2):
        for q in procs[world]:
            q.join(500)
            assert q.exitcode == 0
        res[world] = [json.load(open(str(tmp_path / f"w{world}") + f".{r}")) for r in range(world)]
    assert res[2][0]["out"] == res[2][1]["out"] == res[1][0]["out"]
    assert res[2][0]["drafts"] > 0 and res[1][0]["drafts"] == 0


def test_group_table_deals_pages_over_ranks():
    from stkernel_b200.runtime.kv import GroupTable
    tabs = [GroupTable("c4", 4, 2, 10, torch.device("cpu"), 0.25, r, 3) for r in range(3)]
    for t in tabs:
        t.ensure(0, 0, 6)
    for lp in range(7):
        owners = [r for r, t in enumerate(tabs) if int(t.table_np[0, lp]) != t.trash]
        assert owners == [lp % 3]
    assert [t.pages_in_use for t in tabs] == [3, 2, 2]
    # shared and adopted page lists keep the scratch entries out of the reference counts
    pages = tabs[1].share(0, 0, 6)
    tabs[1].adopt(1, 0, pages)
    tabs[1].release_all(0)
    assert tabs[1].pages_in_use == 2
    for pg in pages:
        tabs[1].unref(pg)
    tabs[1].release_all(1)
    assert tabs[1].pages_in_use == 0
    tabs[1].sync()
    assert tabs[1].local_table().shape == (2, 3)
