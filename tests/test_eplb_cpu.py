"""Expert-parallel load balancing: placement properties, and a re-placed model that computes the same function."""
import pytest
import torch

from stkernel_b200.config import EngineConfig, ParallelConfig, SchedulerConfig, tiny_config
from stkernel_b200.models.dsv4 import DictSource, build_model_weights
from stkernel_b200.models.weights import init_random_weights
from stkernel_b200.ops import functional as Fn
from stkernel_b200.parallel.eplb import Placement, initial_placement, rank_loads, rebalance, to_physical
from stkernel_b200.runtime.engine import Engine, SamplingParams


@pytest.fixture(autouse=True)
def fp32_acts():
    Fn.set_cpu_act_dtype(torch.float32)
    yield
    Fn.set_cpu_act_dtype(torch.bfloat16)


def test_placement_covers_every_expert_and_fills_every_rank():
    p = initial_placement(256, 32, 8)
    assert p.n_physical == 288 and p.slots_per_rank == 36
    assert all(len(r) >= 1 for r in p.replicas())
    assert rebalance([1.0] * 16, 0, 4).is_identity
    with pytest.raises(ValueError):
        rebalance([1.0] * 10, 1, 4)


def test_rebalance_replicates_hot_experts_and_evens_out_the_ranks():
    g = torch.Generator().manual_seed(0)
    load = (torch.rand(64, generator=g) ** 4 * 1000).tolist()          # a few hot experts
    load[5] = 5000.0
    base = Placement(64, 8, list(range(64)))
    new = rebalance(load, 16, 8)
    new.validate()
    reps = new.replicas()
    assert len(reps[5]) >= 3                                            # the hottest expert is replicated
    assert len({s // new.slots_per_rank for s in reps[5]}) == min(len(reps[5]), 8)   # spread over the ranks first
    before, after = max(rank_loads(base, load)), max(rank_loads(new, load))
    mean = sum(load) / 8
    assert after < 0.7 * before and after < 1.25 * mean
    # without spares the packing alone still helps
    packed = rebalance(load, 0, 8)
    assert sorted(packed.phys_to_logical) == list(range(64))
    assert max(rank_loads(packed, load)) <= before


def test_router_ids_map_to_replicas_round_robin():
    p = Placement(4, 2, [0, 1, 2, 0, 3, 0])                             # expert 0 has three replicas: slots 0, 3, 5
    l2p, cnt = p.tables("cpu")
    ids = torch.tensor([[0, 1], [0, 2], [0, 3], [0, 1]], dtype=torch.int32)
    phys = to_physical(ids, l2p, cnt)
    assert phys[:, 0].tolist() == [0, 3, 5, 0]                          # token index mod 3
    assert phys[:, 1].tolist() == [1, 2, 4, 1]
    assert all(p.phys_to_logical[int(s)] == int(l) for s, l in zip(phys.reshape(-1), ids.reshape(-1)))


def test_engine_records_load_and_a_rebalanced_engine_emits_the_same_text():
    torch.manual_seed(2)
    cfg = tiny_config()
    w = init_random_weights(cfg, seed=0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (48, 20)]
    sp = SamplingParams(temperature=0.0, max_tokens=8)

    def engine(redundant):
        ec = EngineConfig(model=cfg, parallel=ParallelConfig(eplb_redundant=redundant, eplb_record=True),
                          sched=SchedulerConfig(max_model_len=512, max_num_seqs=4, max_num_batched_tokens=4096,
                                                graph_cap=0)).validate()
        e = Engine(ec, build_model_weights(cfg, DictSource(w), "cpu"), "cpu", max_context=512)
        e.weight_source = DictSource(w)
        return e

    plain = engine(0)
    ref = plain.generate(prompts, sp)
    load = plain.expert_load()
    assert load.shape == (cfg.num_hidden_layers, cfg.n_routed_experts)
    n_tokens = sum(len(p) for p in prompts) + 2 * (sp.max_tokens - 1)
    assert int(load[0].sum()) == n_tokens * cfg.num_experts_per_tok
    eng = engine(2)                                                     # 8 logical experts in 10 slots
    gains = eng.rebalance_experts(load)
    assert len(gains) == cfg.num_hidden_layers and all(g <= 1.0 + 1e-9 for g in gains)
    assert eng.model.w.layers[0].experts.num_local == 10 and eng.model.w.layers[0].eplb is not None
    assert eng.generate(prompts, sp) == ref


def test_random_loads_keep_the_placement_valid_and_never_make_the_busiest_rank_busier():
    import random
    from stkernel_b200.parallel.eplb import initial_placement, rank_loads, rebalance, to_physical
    rng = random.Random(0)
    for _ in range(300):
        ep = rng.choice([1, 2, 4, 8])
        n_log = ep * rng.randint(1, 8)
        red = ep * rng.randint(0, 3)
        kind = rng.choice(["uniform", "zero", "skew", "one"])
        load = {"uniform": [1.0] * n_log, "zero": [0.0] * n_log,
                "skew": [rng.random() ** 4 * 100 for _ in range(n_log)],
                "one": [100.0 if i == n_log // 2 else 0.0 for i in range(n_log)]}[kind]
        p = rebalance(load, red, ep)
        p.validate()
        reps = p.replicas()
        assert len(reps) == n_log and all(len(r) >= 1 for r in reps)
        assert p.n_physical == n_log + red and sorted(x for r in reps for x in r) == list(range(p.n_physical))
        if sum(load) > 0:
            assert max(rank_loads(p, load)) <= max(rank_loads(initial_placement(n_log, red, ep), load)) * (1 + 1e-9)
        if kind == "one" and red >= ep and ep > 1:
            # the one busy expert has a replica on every rank and no more: the load is even
            assert len(reps[n_log // 2]) >= ep and max(rank_loads(p, load)) == pytest.approx(100.0 / ep)
        l2p, cnt = p.tables("cpu")
        ids = torch.randint(0, n_log, (40, 3), dtype=torch.int32)
        ph = to_physical(ids, l2p, cnt)
        owner = {s: e for e, r in enumerate(reps) for s in r}
        assert [owner[x] for x in ph.flatten().tolist()] == ids.flatten().tolist()
