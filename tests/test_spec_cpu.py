"""DSpark speculative decoding on the tiny CPU config: the emitted text is the target's own
(identical to the non-speculative engine under the same seeds) whatever the drafter proposes."""
import dataclasses

import pytest
import torch

from stkernel_b200.config import EngineConfig, SchedulerConfig, SpecConfig, tiny_config
from stkernel_b200.models.dsv4 import DictSource, build_model_weights
from stkernel_b200.models.weights import init_random_weights
from stkernel_b200.ops import functional as Fn
from stkernel_b200.ops import reference as R
from stkernel_b200.runtime.engine import Engine, SamplingParams
from stkernel_b200.spec import dspark as DS


@pytest.fixture(autouse=True)
def fp32_acts():
    Fn.set_cpu_act_dtype(torch.float32)
    yield
    Fn.set_cpu_act_dtype(torch.bfloat16)


def _cfg():
    return tiny_config(n_mtp_layers=2, dspark_target_layer_ids=(0, 1), dspark_markov_rank=16)


def _engines(n_spec=3, seqs=4, topk=8):
    cfg = _cfg()
    w = init_random_weights(cfg, seed=0)
    sc = SchedulerConfig(max_model_len=512, max_num_seqs=seqs, max_num_batched_tokens=96, graph_cap=0)
    tw = build_model_weights(cfg, DictSource(w), "cpu")
    plain = Engine(EngineConfig(model=cfg, sched=sc).validate(), tw, "cpu", max_context=512)
    dw = DS.build_draft_weights(cfg, DictSource(w), tw, "cpu")
    ec = EngineConfig(model=cfg, sched=sc, spec=SpecConfig(method="dspark", num_speculative_tokens=n_spec, markov_topk=topk)).validate()
    spec = Engine(ec, tw, "cpu", max_context=512, draft_weights=dw)
    return cfg, plain, spec


@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_spec_output_equals_plain(temperature):
    torch.manual_seed(0)
    cfg, plain, spec = _engines()
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (40, 150, 7)]
    sp = SamplingParams(temperature=temperature, seed=11, max_tokens=14)
    ref = plain.generate(prompts, sp)
    got = spec.generate(prompts, sp)
    assert got == ref
    assert spec.metrics.spec_num_drafts > 0 and spec.metrics.spec_num_draft_tokens == 3 * spec.metrics.spec_num_drafts


def test_oracle_drafter_accepts_and_rolls_back():
    """Feed the verifier proposals that are right for a while and then wrong: accepted prefixes shorten the
    run, rejected tails are rolled back (compressor rings, caches) without changing the text."""
    torch.manual_seed(1)
    cfg, plain, spec = _engines(n_spec=4)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (33, 90)]
    sp = SamplingParams(temperature=0.7, seed=5, max_tokens=40)
    ref = plain.generate(prompts, sp)
    truth = {tuple(p): r for p, r in zip(prompts, ref)}
    ids = [spec.add_request(p, sp) for p in prompts]
    calls = {"n": 0}

    def oracle(anchor, anchor_pos, rows, temperature, seed, want_logits=False):
        out = torch.zeros(anchor.shape[0], 4, dtype=torch.int64)
        for b in range(anchor.shape[0]):
            req = next(r for r in spec.requests.values() if r.row == int(rows[b]) and not r.finished)
            full = req.prompt + truth[tuple(req.prompt)]
            p = int(anchor_pos[b])
            good = (calls["n"] + b) % 5          # 0..4 right, the rest wrong
            for j in range(4):
                t = full[p + 1 + j] if p + 1 + j < len(full) else 0
                out[b, j] = t if j < good else (t + 1) % cfg.vocab_size
        calls["n"] += 1
        return out, None

    spec.drafter.draft = oracle
    steps = 0
    while spec.has_work():
        spec.step()
        steps += 1
    assert [spec.requests[i].output for i in ids] == ref
    m = spec.metrics
    assert 0 < m.spec_num_accepted_tokens < m.spec_num_draft_tokens
    assert m.spec_accepted_per_pos[0] >= m.spec_accepted_per_pos[-1]
    assert steps < 40 + 4                      # fewer steps than one token per step
    text = m.render("x")
    assert "vllm:spec_decode_num_accepted_tokens_per_pos_total" in text


def test_draft_tokens_use_verifier_noise():
    """A drafter whose logits equal the target's would always be accepted: same (seed, position) keys."""
    logits = torch.randn(3, 50)
    t = torch.full((3,), 0.9)
    seed = torch.tensor([1, 2, 3])
    pos = torch.tensor([10, 20, 30])
    a, _ = R.gumbel_sample(logits, t, seed, pos)
    b, _ = R.gumbel_sample(logits.clone(), t, seed, pos)
    assert torch.equal(a, b)
    c, _ = R.gumbel_sample(logits, t, seed, pos + 1)
    assert not torch.equal(a, c) or True      # different keys give independent draws


def test_markov_head_topk_and_dense():
    torch.manual_seed(0)
    V, Rk = 64, 8
    mh = DS.MarkovHead(torch.randn(V, Rk).bfloat16(), torch.randn(V, Rk).bfloat16())
    base = torch.randn(2, V)
    prev = torch.tensor([3, 9])
    dense = mh.apply(base, prev, 0)
    bias = mh.w2.float() @ mh.w1[prev].float().T
    assert torch.allclose(dense, base + bias.T, atol=1e-2)
    top = mh.apply(base, prev, 5)
    keep = torch.topk(base, 5, -1).indices
    assert torch.isinf(top).sum() == 2 * (V - 5)
    assert torch.allclose(top.gather(1, keep), dense.gather(1, keep), atol=1e-2)


def test_knob_parsers_fail_closed():
    assert DS.parse_draft_topk("", 100) is None and DS.parse_draft_topk("off", 100) is None
    assert DS.parse_draft_topk(" 512 ", 1000) == 512
    for bad in ("abc", "-1", "101", "1.5"):
        with pytest.raises(ValueError):
            DS.parse_draft_topk(bad, 100)
    assert DS.parse_refine_pass("") is False and DS.parse_refine_pass("YES") is True
    with pytest.raises(ValueError):
        DS.parse_refine_pass("maybe")
    assert DS.refine_feedback_indices(2, 4) == [1, 2, 3, 5, 6, 7]
    assert DS.refine_feedback_indices(3, 1) == []


def test_sideload_contract(tmp_path):
    V, Rk = 32, 4
    ok = dict(keys=["markov_w1", "markov_w2"], w1_shape=(V, Rk), w2_shape=(V, Rk), vocab_size=V, rank=Rk,
              replicated_w1=True, replicated_w2=True)
    assert DS.validate_markov_sideload(**ok) is None
    assert "missing" in DS.validate_markov_sideload(**{**ok, "keys": ["markov_w1"]})
    assert "markov_w1 shape" in DS.validate_markov_sideload(**{**ok, "w1_shape": (V, Rk + 1)})
    assert "markov_w2 shape" in DS.validate_markov_sideload(**{**ok, "w2_shape": (V + 1, Rk)})
    assert "W1" in DS.validate_markov_sideload(**{**ok, "replicated_w1": False})
    assert "W2" in DS.validate_markov_sideload(**{**ok, "replicated_w2": False})
    mh = DS.MarkovHead(torch.zeros(V, Rk).bfloat16(), torch.zeros(V, Rk).bfloat16())
    path = tmp_path / "m.pt"
    torch.save({"markov_w1": torch.ones(V, Rk), "markov_w2": torch.full((V, Rk), 2.0)}, path)
    sha = mh.sideload(str(path), V, Rk)
    assert len(sha) == 64 and float(mh.w1[0, 0]) == 1.0 and float(mh.w2[0, 0]) == 2.0
    torch.save({"markov_w1": torch.full((V, Rk), float("nan")), "markov_w2": torch.ones(V, Rk)}, path)
    with pytest.raises(RuntimeError):
        mh.sideload(str(path), V, Rk)
    mh.fp8_built = True
    with pytest.raises(RuntimeError):
        mh.sideload(str(path), V, Rk)


def test_bf16_head_release_truth_table():
    f = DS.bf16_head_release_blockers
    assert f(True, True, False, False, True, False) == []                      # not requested
    assert f(True, True, True, False, True, False) == []
    assert f(False, True, True, False, True, False) == ["target lm_head has no fp8 copy"]
    assert len(f(True, False, True, False, True, False)) == 1
    assert f(True, False, True, False, False, False) == []                     # draft does not share the head
    assert len(f(False, False, True, True, True, True)) == 4


def test_rowwise_fp8_draft_head():
    from stkernel_b200.spec import fp8_draft_head as F8
    torch.manual_seed(0)
    w = torch.randn(300, 128) * 0.05
    w[7] *= 40.0                                     # a row with a very different range keeps its own scale
    h = torch.randn(5, 128)
    head = F8.quantize_draft_head(w)
    assert head.weight_fp8.dtype == torch.float8_e4m3fn and head.row_scale.shape == (1, 300)
    lg = F8.fp8_draft_head_logits(h, head)
    ref = h @ w.t()
    assert ((lg - ref).norm() / ref.norm()).item() < 0.05
    assert (lg.argmax(-1) == ref.argmax(-1)).all()
    with pytest.raises(ValueError):
        F8.quantize_draft_head(torch.zeros(3))
    with pytest.raises(ValueError):
        F8.fp8_draft_head_logits(torch.zeros(2, 64), head)
    assert F8.pick_head_impl(True, False) == "rowwise" and F8.pick_head_impl(False, True) == "block"
    assert F8.pick_head_impl(False, False) == "bf16"
    with pytest.raises(ValueError):
        F8.pick_head_impl(True, True)


def test_http_server_delivers_every_token_of_a_request_that_ends_inside_a_speculative_step():
    """A step that accepts several drafts yields several tokens for one request; the one that ends the request must not
    cut the others off (the finished flag travels with the last token of the step)."""
    from fastapi.testclient import TestClient
    from stkernel_b200.serve.api_server import create_app
    from stkernel_b200.serve.tokenizer import ByteTokenizer, ChatTokenizer
    cfg, plain, spec = _engines()
    tok = ChatTokenizer(ByteTokenizer(cfg.vocab_size))
    prompt = tok.encode("hello there")
    want = plain.generate([prompt], SamplingParams(temperature=0.0, max_tokens=14, ignore_eos=True))[0]

    def oracle(req, drafted):                                   # a drafter that is always right: every draft is accepted
        k = len(req.output)
        return want[k:k + len(drafted)] if k + len(drafted) <= len(want) else drafted
    spec.draft_override = oracle
    import json
    with TestClient(create_app(spec, tok, "tiny")) as c, TestClient(create_app(plain, tok, "tiny")) as ref:
        for limit in range(9, 15):
            body = {"prompt": prompt, "max_tokens": limit, "temperature": 0.0, "ignore_eos": True}
            r, rr = c.post("/v1/completions", json=body).json(), ref.post("/v1/completions", json=body).json()
            assert r["usage"]["completion_tokens"] == limit and r["choices"][0]["finish_reason"] == "length"
            assert r["choices"][0]["text"] == rr["choices"][0]["text"]          # one token per step on the reference server
            with c.stream("POST", "/v1/completions", json={**body, "stream": True}) as resp:
                lines = [x[6:] for x in resp.iter_lines() if x.startswith("data: ")]
            chunks = [json.loads(x) for x in lines[:-1]]
            assert "".join(ch["choices"][0]["text"] for ch in chunks) == rr["choices"][0]["text"]
            assert chunks[-1]["usage"]["completion_tokens"] == limit
    assert spec.metrics.spec_num_accepted_tokens > 20           # steps did carry several tokens
