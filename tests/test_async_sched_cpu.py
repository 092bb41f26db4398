"""Asynchronous scheduling: step k+1 is scheduled and launched before the tokens of step k are read.  The texts, the
finish reasons and the prefix-cache behaviour must be those of the engine that reads every step before the next."""
import pytest
import torch

from stkernel_b200.config import EngineConfig, SchedulerConfig, SpecConfig, tiny_config
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
    w = init_random_weights(cfg, seed=0)
    return cfg, build_model_weights(cfg, DictSource(w), "cpu")


def _engine(model, async_on, seqs=3, chunk=48):
    cfg, tw = model
    ec = EngineConfig(model=cfg, sched=SchedulerConfig(max_model_len=1024, max_num_seqs=seqs, max_num_batched_tokens=chunk,
                                                       graph_cap=0, async_scheduling=async_on)).validate()
    return Engine(ec, tw, "cpu", max_context=1024)


def _run(eng, prompts, params):
    ids = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
    steps = 0
    while eng.has_work():
        eng.step()
        steps += 1
    return [eng.requests[i].output for i in ids], [eng.requests[i].finish_reason for i in ids], steps


def test_texts_and_finish_reasons_match_the_synchronous_engine(model):
    cfg, _ = model
    torch.manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (100, 7, 61, 300, 20)]
    params = [SamplingParams(temperature=0.7, seed=i, max_tokens=3 + 4 * i) for i in range(5)]
    want = _run(_engine(model, False), prompts, params)
    eng = _engine(model, True)
    got = _run(eng, prompts, params)
    assert got[:2] == want[:2]
    assert want[2] < got[2] <= want[2] + 3                         # the last step is read one call later
    assert all(Engine.PENDING not in o for o in got[0])
    assert eng.kv.c4.pages_in_use == 0 or eng.prefix_cache is not None
    # an end-of-sequence token in the middle of an answer: the surplus row of the step in flight is dropped
    eos = want[0][4][5]
    params = [SamplingParams(temperature=0.7, seed=i, max_tokens=3 + 4 * i, eos_token_id=eos) for i in range(5)]
    want = _run(_engine(model, False), prompts, params)
    got = _run(_engine(model, True), prompts, params)
    assert got[:2] == want[:2] and "stop" in want[1]
    assert [len(o) for o in got[0]] == [len(o) for o in want[0]]


def test_cached_prefix_state_is_taken_before_the_next_step_changes_it(model):
    cfg, _ = model
    torch.manual_seed(1)
    base = torch.randint(0, cfg.vocab_size, (600,)).tolist()
    tail = torch.randint(0, cfg.vocab_size, (40,)).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=5)
    outs = {}
    for mode in (False, True):
        eng = _engine(model, mode, chunk=128)
        first = eng.generate([base], sp)
        second = eng.generate([base[:520] + tail], sp)              # 512 tokens come from the cache
        assert eng.prefix_cache.hit_tokens == 512
        outs[mode] = (first, second)
    assert outs[True] == outs[False]
    # and the cached run equals a run without any cache hit
    cold = _engine(model, False, chunk=128).generate([base[:520] + tail], sp)
    assert outs[True][1] == cold


def test_with_a_capped_pool_requests_wait_and_texts_match(model):
    """Asynchronous scheduling over a compressed-KV pool that cannot hold every request at once."""
    from stkernel_b200.config import CacheConfig
    cfg, tw = model
    torch.manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (300, 280, 270, 20, 290, 33)]
    params = [SamplingParams(temperature=0.5, seed=i, max_tokens=4 + i) for i in range(6)]
    outs = {}
    for mode in (False, True):
        ec = EngineConfig(model=cfg, cache=CacheConfig(kv_pool_tokens=700),
                          sched=SchedulerConfig(max_model_len=1024, max_num_seqs=4, max_num_batched_tokens=96,
                                                graph_cap=0, async_scheduling=mode)).validate()
        eng = Engine(ec, tw, "cpu", max_context=1024)
        ids = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
        waited = False
        while eng.has_work():
            eng.step()
            waited = waited or eng.sched.num_waiting > 0
            assert len(eng.kv.c4.free) - eng.kv.promised() >= 0
        assert waited and not eng.kv.reserved
        outs[mode] = [eng.requests[i].output for i in ids]
    assert outs[True] == outs[False]


def test_abort_while_a_step_is_in_flight(model):
    cfg, _ = model
    torch.manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (30, 40)]
    sp = SamplingParams(temperature=0.0, max_tokens=12)
    want = _run(_engine(model, False), prompts[1:], [sp])[0][0]
    eng = _engine(model, True)
    a, b = eng.add_request(prompts[0], sp), eng.add_request(prompts[1], sp)
    for _ in range(4):
        eng.step()
    assert eng.abort(a)
    eng.release(a)
    while eng.has_work():
        eng.step()
    assert eng.requests[b].output == want and Engine.PENDING not in eng.requests[b].output


def test_not_with_speculative_decoding_or_forced_tokens(model):
    cfg, tw = model
    eng = _engine(model, True)
    eng.add_request([1, 2, 3], SamplingParams(max_tokens=2))
    with pytest.raises(ValueError):
        eng.step(forced=[5])
    from stkernel_b200.spec import dspark as DS
    scfg = tiny_config(n_mtp_layers=2, dspark_target_layer_ids=(0, 1), dspark_markov_rank=16)
    w = init_random_weights(scfg, seed=0)
    stw = build_model_weights(scfg, DictSource(w), "cpu")
    ec = EngineConfig(model=scfg, spec=SpecConfig(method="dspark", num_speculative_tokens=3, markov_topk=8),
                      sched=SchedulerConfig(max_model_len=256, max_num_seqs=2, max_num_batched_tokens=64, graph_cap=0,
                                            async_scheduling=True)).validate()
    spec = Engine(ec, stw, "cpu", max_context=256, draft_weights=DS.build_draft_weights(scfg, DictSource(w), stw, "cpu"))
    assert spec.async_scheduling is False                           # the accept count decides what the next step holds


def test_http_server_on_an_asynchronously_scheduled_engine():
    import json
    from fastapi.testclient import TestClient
    from stkernel_b200.serve.api_server import create_app
    from stkernel_b200.serve.tokenizer import ByteTokenizer, ChatTokenizer
    cfg = tiny_config()
    tw = build_model_weights(cfg, DictSource(init_random_weights(cfg, seed=0)), "cpu")
    res = {}
    for mode in (False, True):
        ec = EngineConfig(model=cfg, sched=SchedulerConfig(max_model_len=512, max_num_seqs=4, max_num_batched_tokens=256,
                                                           graph_cap=0, async_scheduling=mode)).validate()
        app = create_app(Engine(ec, tw, "cpu", max_context=512), ChatTokenizer(ByteTokenizer(cfg.vocab_size)), "tiny")
        with TestClient(app) as c:
            body = {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0.9, "seed": 4,
                    "ignore_eos": True, "n": 2}
            r = c.post("/v1/chat/completions", json=body).json()
            with c.stream("POST", "/v1/chat/completions", json={**body, "stream": True}) as resp:
                lines = [x[6:] for x in resp.iter_lines() if x.startswith("data: ")]
            streamed = ["", ""]
            for x in lines[:-1]:
                for ch in json.loads(x)["choices"]:
                    streamed[ch["index"]] += ch["delta"].get("content", "")
            res[mode] = ([ch["message"]["content"] or "" for ch in r["choices"]], r["usage"], streamed)
    assert res[True] == res[False] and res[True][0] == res[True][2]
