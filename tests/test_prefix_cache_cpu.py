"""Prefix caching over the hybrid KV: a request that shares a cached 256-token-aligned prefix skips that
part of its prefill and still produces exactly the text of a cold engine."""
import pytest
import torch

from stkernel_b200.config import CacheConfig, EngineConfig, SchedulerConfig, tiny_config
from stkernel_b200.models.dsv4 import DictSource, build_model_weights
from stkernel_b200.models.weights import init_random_weights
from stkernel_b200.ops import functional as Fn
from stkernel_b200.runtime.engine import Engine, SamplingParams
from stkernel_b200.runtime.prefix_cache import BLOCK, chain_hashes


@pytest.fixture(autouse=True)
def fp32_acts():
    Fn.set_cpu_act_dtype(torch.float32)
    yield
    Fn.set_cpu_act_dtype(torch.bfloat16)


def _engine(w, cfg, caching, chunk=256, seqs=4):
    ec = EngineConfig(model=cfg, cache=CacheConfig(enable_prefix_caching=caching),
                      sched=SchedulerConfig(max_model_len=1536, max_num_seqs=seqs, max_num_batched_tokens=chunk, graph_cap=0)).validate()
    return Engine(ec, build_model_weights(cfg, DictSource(w), "cpu"), "cpu", max_context=1536)


def test_chain_hashes_are_prefix_stable():
    a = list(range(1000))
    b = list(range(600)) + [7] * 400
    ha, hb = chain_hashes(a), chain_hashes(b)
    assert len(ha) == 3 and ha[:2] == hb[:2] and ha[2] != hb[2]
    assert chain_hashes(a, limit=512) == ha[:2] and chain_hashes(a[:255]) == []


def test_shared_prefix_is_reused_and_text_is_unchanged():
    torch.manual_seed(0)
    cfg = tiny_config()
    w = init_random_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(5)
    common = torch.randint(0, cfg.vocab_size, (2 * BLOCK + 40,), generator=g).tolist()
    p1 = common + torch.randint(0, cfg.vocab_size, (30,), generator=g).tolist()
    p2 = common + torch.randint(0, cfg.vocab_size, (55,), generator=g).tolist()
    p3 = common[:BLOCK + 10] + torch.randint(0, cfg.vocab_size, (20,), generator=g).tolist()     # shares one block only
    sp = SamplingParams(temperature=0.7, seed=3, max_tokens=10)
    cold = _engine(w, cfg, caching=False)
    ref = [cold.generate([p], sp)[0] for p in (p1, p2, p3)]
    warm = _engine(w, cfg, caching=True)
    assert warm.prefix_cache is not None
    out1 = warm.generate([p1], sp)[0]
    computed1 = warm.metrics.prompt_tokens_total
    assert computed1 == len(p1) and len(warm.prefix_cache.entries) == 2          # boundaries 256 and 512
    out2 = warm.generate([p2], sp)[0]
    computed2 = warm.metrics.prompt_tokens_total - computed1
    assert computed2 == len(p2) - 2 * BLOCK and warm.prefix_cache.hits == 1
    out3 = warm.generate([p3], sp)[0]
    computed3 = warm.metrics.prompt_tokens_total - computed1 - computed2
    assert computed3 == len(p3) - BLOCK and warm.prefix_cache.hit_tokens == 3 * BLOCK
    assert [out1, out2, out3] == ref
    # an identical prompt still computes at least its last token
    before = warm.metrics.prompt_tokens_total
    again = warm.generate([p1], sp)[0]
    assert again == ref[0] and warm.metrics.prompt_tokens_total - before == len(p1) - 2 * BLOCK
    # all pages come back: request rows freed, entries dropped
    n = warm.reset_prefix_cache()
    assert n == 2 and warm.kv.swa.pages_in_use == 0 and warm.kv.c4.pages_in_use == 0
    assert all(r == 0 for r in warm.kv.swa.ref) and all(r == 0 for r in warm.kv.c4.ref)


def test_concurrent_requests_share_pages_and_eviction_under_pressure():
    torch.manual_seed(1)
    cfg = tiny_config()
    w = init_random_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(9)
    common = torch.randint(0, cfg.vocab_size, (BLOCK + 5,), generator=g).tolist()
    prompts = [common + torch.randint(0, cfg.vocab_size, (8 + i,), generator=g).tolist() for i in range(3)]
    sp = SamplingParams(temperature=0.0, max_tokens=6)
    cold = _engine(w, cfg, caching=False)
    ref = cold.generate(prompts, sp)
    warm = _engine(w, cfg, caching=True)
    warm.generate([prompts[0]], sp)
    shared_c4 = list(next(iter(warm.prefix_cache.entries.values())).c4_pages)
    out = warm.generate(prompts[1:], sp)                        # two requests adopt the same pages at once
    assert out == ref[1:] and warm.prefix_cache.hits == 2
    assert all(warm.kv.c4.ref[pg] == 1 for pg in shared_c4)    # only the entry still owns them
    # pressure: an allocation that finds no free page evicts cached prefixes instead of failing
    free_before = len(warm.kv.swa.free)
    held = [warm.kv.swa.free.pop() for _ in range(free_before)]
    row = warm.kv.alloc_row()
    warm.kv.swa.ensure(row, 0, 0)                               # must take a page back from the cache
    assert len(warm.prefix_cache.entries) == 0
    warm.kv.swa.free.extend(held)
    warm.kv.free_row(row)


def test_http_reset_endpoint_drops_entries():
    from fastapi.testclient import TestClient
    from stkernel_b200.serve.api_server import create_app
    from stkernel_b200.serve.tokenizer import ByteTokenizer, ChatTokenizer
    cfg = tiny_config()
    eng = _engine(init_random_weights(cfg, seed=0), cfg, caching=True)
    with TestClient(create_app(eng, ChatTokenizer(ByteTokenizer(cfg.vocab_size)), "tiny")) as c:
        body = {"prompt": "x" * 300, "max_tokens": 2, "temperature": 0}
        c.post("/v1/completions", json=body)
        assert len(eng.prefix_cache.entries) == 1
        u = c.post("/v1/completions", json=body).json()["usage"]
        assert eng.prefix_cache.hits == 1 and u["prompt_tokens"] == 300
        assert c.post("/reset_prefix_cache").json()["reset"] is True
        assert len(eng.prefix_cache.entries) == 0


def test_eviction_takes_the_longest_prefix_first_and_strands_nothing():
    """After any eviction every remaining entry must still be reachable through `match` (an entry is found only by
    walking its chain from the root), whatever order chains were offered and matched in."""
    cfg = tiny_config()
    g = torch.Generator().manual_seed(2)
    long_prompt = torch.randint(0, cfg.vocab_size, (4 * BLOCK + 3,), generator=g).tolist()
    other = long_prompt[:BLOCK] + torch.randint(0, cfg.vocab_size, (2 * BLOCK + 3,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=1)
    eng2 = _engine(init_random_weights(cfg, seed=0), cfg, caching=True, chunk=256)
    pc = eng2.prefix_cache
    eng2.generate([long_prompt], sp)            # boundaries 256 .. 1024
    eng2.generate([other], sp)                  # shares the first block, adds two entries of its own
    assert len(pc.entries) == 6
    pc.match(long_prompt)                       # a lookup must not make the root the oldest entry

    def reachable():
        seen = set()
        for p in (long_prompt, other):
            for h in chain_hashes(p, pc.block, limit=len(p) - 1):
                if h not in pc.entries:
                    break
                seen.add(h)
        return seen

    while pc.entries:
        assert reachable() == set(pc.entries.keys())
        pc.evict_one()
    assert eng2.kv.swa.pages_in_use == 0 and eng2.kv.c4.pages_in_use == 0


def test_prefix_cache_with_ratio_128_layers_copies_the_partial_page():
    """A model with a ratio-128 layer (the production layer mix): the cut at 256 tokens falls inside a ratio-128 page,
    whose two rows travel with the entry; the adopting request produces the text of a cold engine."""
    torch.manual_seed(0)
    cfg = tiny_config(num_hidden_layers=3, compress_ratios=(4, 128, 0))
    w = init_random_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(11)
    common = torch.randint(0, cfg.vocab_size, (BLOCK + 150,), generator=g).tolist()
    p1 = common + torch.randint(0, cfg.vocab_size, (20,), generator=g).tolist()
    p2 = common + torch.randint(0, cfg.vocab_size, (140,), generator=g).tolist()     # crosses the next ratio-128 window
    sp = SamplingParams(temperature=0.7, seed=5, max_tokens=8)
    cold = _engine(w, cfg, caching=False)
    ref = [cold.generate([p], sp)[0] for p in (p1, p2)]
    warm = _engine(w, cfg, caching=True)
    assert warm.prefix_cache is not None and warm.prefix_cache.c128_layers == [1]
    out1 = warm.generate([p1], sp)[0]
    e = next(iter(warm.prefix_cache.entries.values()))
    assert e.pos == BLOCK and e.c128_pages == [] and list(e.c128_tail) == [1]
    before = warm.metrics.prompt_tokens_total
    out2 = warm.generate([p2], sp)[0]
    assert warm.prefix_cache.hits == 1 and warm.metrics.prompt_tokens_total - before == len(p2) - BLOCK
    assert [out1, out2] == ref
    warm.reset_prefix_cache()
    assert warm.kv.c128.pages_in_use == 0 and all(r == 0 for r in warm.kv.c128.ref)
