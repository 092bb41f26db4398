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
