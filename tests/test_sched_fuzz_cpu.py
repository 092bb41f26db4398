"""Randomised scheduling against one-request-at-a-time generation: requests of assorted lengths (some sharing a prefix)
arrive a few at a time into engines with small step budgets, with and without asynchronous scheduling and a capped KV
pool; every request must get exactly the text it gets alone on an engine without a prefix cache."""
import random

import pytest
import torch

from stkernel_b200.config import CacheConfig, EngineConfig, SchedulerConfig, tiny_config
from stkernel_b200.models.dsv4 import DictSource, build_model_weights
from stkernel_b200.models.weights import init_random_weights
from stkernel_b200.ops import functional as Fn
from stkernel_b200.runtime.engine import Engine, SamplingParams


@pytest.fixture(autouse=True)
def fp32_acts():
    Fn.set_cpu_act_dtype(torch.float32)
    yield
    Fn.set_cpu_act_dtype(torch.bfloat16)


@pytest.fixture(scope="module")
def model():
    cfg = tiny_config(num_hidden_layers=3, compress_ratios=(4, 128, 4), index_topk_freq=2)
    return cfg, build_model_weights(cfg, DictSource(init_random_weights(cfg, seed=0)), "cpu")


def _engine(model, seqs, chunk, async_on=False, pool=None, prefix=True):
    cfg, tw = model
    ec = EngineConfig(model=cfg, cache=CacheConfig(kv_pool_tokens=pool, enable_prefix_caching=prefix),
                      sched=SchedulerConfig(max_model_len=768, max_num_seqs=seqs, max_num_batched_tokens=chunk, graph_cap=0,
                                            async_scheduling=async_on)).validate()
    return Engine(ec, tw, "cpu", max_context=768)


@pytest.mark.parametrize("trial", [100, 105, 106])
def test_random_arrivals_match_requests_run_alone(model, trial):
    cfg, _ = model
    rng = random.Random(trial)
    g = torch.Generator().manual_seed(trial)
    shared = torch.randint(0, cfg.vocab_size, (300,), generator=g).tolist()
    prompts, params = [], []
    for _ in range(rng.randint(4, 9)):
        n = rng.choice([1, 3, 17, 63, 64, 65, 130, 257, 300])
        p = torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
        if rng.random() < 0.7:
            p = shared[:rng.choice([256, 290])] + p[:40]
        prompts.append(p)
        params.append(SamplingParams(temperature=rng.choice([0.0, 0.8]), seed=rng.randint(0, 99), max_tokens=rng.randint(1, 9)))
    alone = _engine(model, 1, 4096, prefix=False)
    want = [alone.generate([p], sp)[0] for p, sp in zip(prompts, params)]
    eng = _engine(model, rng.choice([2, 3, 5]), rng.choice([24, 64, 128, 256]), async_on=rng.random() < 0.5,
                  pool=rng.choice([None, 900]))
    ids, k = [], 0
    while k < len(prompts) or eng.has_work():
        for _ in range(rng.randint(0, 2)):                       # a few arrivals between steps
            if k < len(prompts):
                ids.append(eng.add_request(prompts[k], params[k]))
                k += 1
        if eng.has_work():
            eng.step()
    assert [eng.requests[i].output for i in ids] == want
    assert eng.prefix_cache.hits >= 1                           # the chosen seeds do reuse a cached prefix
    assert eng.kv.promised() == 0 and not eng.kv.reserved


@pytest.mark.parametrize("trial", [202, 207])
def test_speculative_engine_with_partly_right_drafts_matches_requests_run_alone(trial):
    """The same arrivals into a speculative engine whose drafts are right about 70 % of the time (accepts and rollbacks at
    every position), over a capped pool: the texts are those of plain decoding, one request at a time."""
    from stkernel_b200.config import SpecConfig
    from stkernel_b200.spec import dspark as DS
    cfg = tiny_config(n_mtp_layers=2, dspark_target_layer_ids=(0, 1), dspark_markov_rank=16, num_hidden_layers=3,
                      compress_ratios=(4, 128, 4), index_topk_freq=2)
    w = init_random_weights(cfg, seed=0)
    tw = build_model_weights(cfg, DictSource(w), "cpu")
    dw = DS.build_draft_weights(cfg, DictSource(w), tw, "cpu")

    def engine(seqs, chunk, spec, pool=None, prefix=True):
        ec = EngineConfig(model=cfg, cache=CacheConfig(kv_pool_tokens=pool, enable_prefix_caching=prefix),
                          spec=SpecConfig(method="dspark", num_speculative_tokens=3, markov_topk=8) if spec else SpecConfig(),
                          sched=SchedulerConfig(max_model_len=768, max_num_seqs=seqs, max_num_batched_tokens=chunk,
                                                graph_cap=0)).validate()
        return Engine(ec, tw, "cpu", max_context=768, draft_weights=dw if spec else None)

    rng = random.Random(trial)
    g = torch.Generator().manual_seed(trial)
    shared = torch.randint(0, cfg.vocab_size, (300,), generator=g).tolist()
    prompts, params = [], []
    for _ in range(rng.randint(3, 7)):
        n = rng.choice([1, 3, 17, 63, 64, 65, 130, 257])
        p = torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
        if rng.random() < 0.6:
            p = shared[:rng.choice([256, 290])] + p[:40]
        prompts.append(p)
        params.append(SamplingParams(temperature=rng.choice([0.0, 0.8]), seed=rng.randint(0, 99), max_tokens=rng.randint(1, 12)))
    alone = engine(1, 4096, False, prefix=False)
    want = [alone.generate([p], sp)[0] for p, sp in zip(prompts, params)]
    eng = engine(rng.choice([2, 3, 5]), rng.choice([32, 64, 128, 256]), True, pool=rng.choice([None, 900]))
    truth = {}

    def mostly_right(req, drafted):
        text, k, out = truth[req.req_id], len(req.output), list(drafted)
        for j in range(len(out)):
            if k + j < len(text) and rng.random() < 0.7:
                out[j] = text[k + j]
        return out
    eng.draft_override = mostly_right
    ids, k = [], 0
    while k < len(prompts) or eng.has_work():
        for _ in range(rng.randint(0, 2)):
            if k < len(prompts):
                rid = eng.add_request(prompts[k], params[k])
                truth[rid] = want[k]
                ids.append(rid)
                k += 1
        if eng.has_work():
            eng.step()
    assert [eng.requests[i].output for i in ids] == want
    m = eng.metrics
    assert 0 < m.spec_num_accepted_tokens < m.spec_num_draft_tokens


@pytest.mark.parametrize("trial", [302, 308])
def test_random_aborts_leave_the_other_requests_and_the_pools_intact(model, trial):
    """Requests aborted at random moments (waiting, mid-prefill, decoding, with a step in flight): the others get the
    text they get alone, and once everything has ended no page, row or promise is left behind."""
    cfg, _ = model
    rng = random.Random(trial)
    g = torch.Generator().manual_seed(trial)
    prompts = [torch.randint(0, cfg.vocab_size, (rng.choice([3, 40, 130, 257, 300]),), generator=g).tolist()
               for _ in range(rng.randint(4, 8))]
    params = [SamplingParams(temperature=0.0, max_tokens=rng.randint(2, 10)) for _ in prompts]
    alone = _engine(model, 1, 4096, prefix=False)
    want = [alone.generate([p], sp)[0] for p, sp in zip(prompts, params)]
    eng = _engine(model, rng.choice([2, 3]), rng.choice([24, 64, 128]), async_on=rng.random() < 0.5,
                  pool=rng.choice([None, 900]), prefix=rng.random() < 0.5)
    ids, k, aborted = [], 0, set()
    while k < len(prompts) or eng.has_work():
        for _ in range(rng.randint(0, 2)):
            if k < len(prompts):
                ids.append(eng.add_request(prompts[k], params[k]))
                k += 1
        if ids and rng.random() < 0.25:
            victim = rng.choice(ids)
            if eng.abort(victim):
                aborted.add(victim)
                eng.release(victim)
        if eng.has_work():
            eng.step()
    assert len(aborted) >= 2
    for j, i in enumerate(ids):
        if i not in aborted:
            assert eng.requests[i].output == want[j]
    if eng.prefix_cache is not None:
        eng.prefix_cache.reset()
    kv = eng.kv
    assert (kv.c4.pages_in_use, kv.swa.pages_in_use, kv.c128.pages_in_use) == (0, 0, 0)
    assert len(kv.free_rows) == eng.cfg.sched.max_num_seqs and kv.promised() == 0 and not kv.reserved
