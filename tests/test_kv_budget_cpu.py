"""A compressed-KV pool smaller than max_num_seqs x max_model_len: requests wait for room instead of running out of
pages, finish with the same text, and a request that could never fit is refused when it is added."""
import pytest
import torch

from stkernel_b200.config import CacheConfig, EngineConfig, SchedulerConfig, tiny_config
from stkernel_b200.models.dsv4 import DictSource, build_model_weights
from stkernel_b200.models.weights import init_random_weights
from stkernel_b200.ops import functional as Fn
from stkernel_b200.ops.cache import PAGE
from stkernel_b200.runtime.engine import Engine, SamplingParams
from stkernel_b200.runtime.kv import kv_bytes_per_context_token, memory_pool_tokens, size_pools


@pytest.fixture(autouse=True)
def fp32_acts():
    Fn.set_cpu_act_dtype(torch.float32)
    yield
    Fn.set_cpu_act_dtype(torch.bfloat16)


def _engine(cfg, w, pool_tokens, prefix=False):
    ec = EngineConfig(model=cfg, cache=CacheConfig(kv_pool_tokens=pool_tokens, enable_prefix_caching=prefix),
                      sched=SchedulerConfig(max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=128,
                                            graph_cap=0)).validate()
    return Engine(ec, build_model_weights(cfg, DictSource(w), "cpu"), "cpu", max_context=1024)


def test_requests_wait_for_pages_and_finish_with_the_same_text():
    torch.manual_seed(0)
    cfg = tiny_config(num_hidden_layers=3, compress_ratios=(4, 128, 4), index_topk_freq=2)
    w = init_random_weights(cfg, seed=0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (300, 280, 270, 20, 290)]
    sp = SamplingParams(temperature=0.0, max_tokens=6)
    roomy = _engine(cfg, w, None)
    want = roomy.generate(prompts, sp)
    assert roomy.kv.c4.num_pages == 4 * (1024 // 4 // PAGE + 1)
    # 700 tokens of context in all: two of the 300-token requests fit together (2 pages each), a third must wait
    tight = _engine(cfg, w, 700)
    assert tight.kv.c4.num_pages == -(-(700 // 4) // PAGE) + 4 and tight.kv.c4.num_pages < roomy.kv.c4.num_pages
    ids = [tight.add_request(p, sp) for p in prompts]
    most_running, waited = 0, False
    while tight.has_work():
        tight.step()
        most_running = max(most_running, tight.sched.num_running)
        assert 0.0 <= tight.metrics.kv_cache_usage <= 1.0
        waited = waited or (tight.sched.num_waiting > 0 and tight.sched.num_running < 4)
        assert len(tight.kv.c4.free) - tight.kv.promised() >= 0          # never promised more than the pool has
    assert [tight.requests[i].output for i in ids] == want
    assert waited and most_running < 5
    m = tight.metrics
    assert m.kv_cache_usage == 0.0 and m.ttft_count == 5 and m.ttft_sum > 0
    assert tight.kv.c4.pages_in_use == 0 and tight.kv.promised() == 0 and not tight.kv.reserved


def test_request_larger_than_the_pool_is_refused():
    cfg = tiny_config()
    w = init_random_weights(cfg, seed=0)
    eng = _engine(cfg, w, 300)                       # 2 pages + 4: six pages, 1536 tokens at most per request
    eng.add_request([1] * 200, SamplingParams(max_tokens=8))
    small = Engine(EngineConfig(model=cfg, cache=CacheConfig(kv_pool_tokens=256),
                                sched=SchedulerConfig(max_model_len=4096, max_num_seqs=1, max_num_batched_tokens=128,
                                                      graph_cap=0)).validate(),
                   build_model_weights(cfg, DictSource(w), "cpu"), "cpu", max_context=4096)
    assert small.kv.c4.num_pages == 2
    with pytest.raises(ValueError, match="more compressed-KV pages"):
        small.add_request([1] * 600, SamplingParams(max_tokens=8))      # 608 tokens = 152 rows: three pages


def test_bytes_per_context_token_and_pool_sizes():
    from stkernel_b200.config import flash_config
    cfg = flash_config(num_layers=48)
    n4 = sum(cfg.layer_kind(i) == "c4a" for i in range(48))
    n128 = sum(cfg.layer_kind(i) == "c128a" for i in range(48))
    per = kv_bytes_per_context_token(cfg)
    # 584-byte latent rows and 132-byte indexer-K rows (page-rounded), one per 4 tokens; latent rows per 128 tokens
    assert abs(per - (n4 * (592.0 + 135.0) / 4 + n128 * 592.0 / 128)) / per < 0.02
    assert abs(kv_bytes_per_context_token(cfg, dcp_size=8) - (n4 * (592.0 + 135.0) / 32 + n128 * 592.0 / 128)) / per < 0.02
    assert kv_bytes_per_context_token(cfg, layers=[0]) < per / 20
    full = size_pools(cfg, 32, 430000, 4096)
    capped = size_pools(cfg, 32, 430000, 4096, pool_tokens=2_800_000)
    assert capped["c4_pages"] == -(-(2_800_000 // 4) // PAGE) + 32 < full["c4_pages"]
    assert capped["swa_pages"] == full["swa_pages"]
    assert size_pools(cfg, 32, 430000, 4096, dcp_size=8, pool_tokens=2_800_000)["c4_pages"] == -(-(2_800_000 // 4) // (PAGE * 8)) + 32


def test_pool_tokens_from_a_memory_share():
    from stkernel_b200.config import flash_config
    cfg = flash_config(num_layers=48)
    gb = 1 << 30
    per = kv_bytes_per_context_token(cfg)
    # 60 % of 180 GB with 25 GB taken by the weights: 83 GB of compressed KV
    got = memory_pool_tokens(cfg, 0.60, free_bytes=155 * gb, total_bytes=180 * gb, min_tokens=32768)
    assert abs(got - 83 * gb / per) / got < 1e-6 and got > 15_000_000
    # the same share of a GPU that other tenants have filled: one request's worth, never less
    assert memory_pool_tokens(cfg, 0.60, free_bytes=20 * gb, total_bytes=180 * gb, min_tokens=32768) == 32768
    # context parallelism over 8 ranks: about 8 times the tokens in the same memory (the ratio-128 rows stay replicated)
    wide = memory_pool_tokens(cfg, 0.60, 155 * gb, 180 * gb, 32768, dcp_size=8)
    assert 7.0 < wide / got < 8.01
