"""The paged, batched engine against the naive oracle on the tiny CPU config."""
import pytest
import torch

from stkernel_b200.config import CacheConfig, EngineConfig, SchedulerConfig, tiny_config
from stkernel_b200.models.dsv4 import DictSource, build_model_weights
from stkernel_b200.models.dsv4_oracle import OracleModel, index_cache_computes
from stkernel_b200.models.weights import init_random_weights
from stkernel_b200.ops import functional as Fn
from stkernel_b200.runtime.engine import Engine, SamplingParams


@pytest.fixture(autouse=True)
def fp32_acts():
    Fn.set_cpu_act_dtype(torch.float32)
    yield
    Fn.set_cpu_act_dtype(torch.bfloat16)


def close(got, ref, tol=5e-3, frac=0.9):
    """The layer input is rounded to bf16 by design, so a 1e-6 difference upstream can move an
    element by one bf16 ulp and, rarely, flip a router or top-k choice for one token.  Require
    most positions to agree tightly and the whole tensor to agree in norm."""
    err = (got.float() - ref).abs().amax(-1)
    assert (err < tol).float().mean().item() >= frac, err
    assert ((got.float() - ref).norm() / ref.norm()).item() < 5e-2


def make_engine(cfg, w, chunk=4096, seqs=4):
    ec = EngineConfig(model=cfg, sched=SchedulerConfig(max_model_len=512, max_num_seqs=seqs, max_num_batched_tokens=chunk,
                                                       graph_cap=0)).validate()
    weights = build_model_weights(cfg, DictSource(w), "cpu")
    return Engine(ec, weights, "cpu", max_context=512)


def test_index_cache_rule():
    cfg = tiny_config(num_hidden_layers=8, compress_ratios=(4, 0, 4, 4, 0, 4, 4, 4), index_topk_freq=3)
    flags = [index_cache_computes(cfg, i) for i in range(8)]
    assert flags == [True, False, False, False, False, True, False, False]
    cfg1 = tiny_config(num_hidden_layers=3, compress_ratios=(0, 4, 4), index_topk_freq=7)
    assert [index_cache_computes(cfg1, i) for i in range(3)] == [False, True, False]   # first C4A always computes


@pytest.mark.parametrize("chunk", [4096, 24])
def test_prefill_and_greedy_decode_match_oracle(chunk):
    torch.manual_seed(0)
    cfg = tiny_config()
    w = init_random_weights(cfg, seed=0)
    oracle = OracleModel(cfg, w)
    eng = make_engine(cfg, w, chunk=chunk)
    prompts = [torch.randint(0, cfg.vocab_size, (64,)).tolist() for _ in range(2)]
    steps = 32 if chunk == 4096 else 8
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=steps))
    for p, o in zip(prompts, outs):
        ref_ids, ref_logits = oracle.greedy_decode(torch.tensor(p), steps)
        assert o == ref_ids.tolist()


def test_logits_match_oracle_mixed_batch():
    torch.manual_seed(1)
    cfg = tiny_config(num_hidden_layers=3, compress_ratios=(4, 0, 4), index_topk_freq=2)
    w = init_random_weights(cfg, seed=3)
    oracle = OracleModel(cfg, w)
    eng = make_engine(cfg, w)
    a = torch.randint(0, cfg.vocab_size, (50,))
    b = torch.randint(0, cfg.vocab_size, (37,))
    # drive the model directly through two ragged steps to compare full logits
    from stkernel_b200.runtime.engine import Request, ScheduledSeq
    ra, rb = Request(0, a.tolist(), SamplingParams()), Request(1, b.tolist(), SamplingParams())
    ra.row, rb.row = eng.kv.alloc_row(), eng.kv.alloc_row()
    seqs = [ScheduledSeq(ra, 0, 30, False), ScheduledSeq(rb, 0, 37, True)]
    t, n, ns = eng._stage(seqs)
    eng._upload(t, n, ns)
    meta = eng._build_meta(t, n, 16)
    lg1 = eng.model.forward(meta)
    seqs = [ScheduledSeq(ra, 30, 20, True)]
    t, n, ns = eng._stage(seqs)
    eng._upload(t, n, ns)
    meta = eng._build_meta(t, n, 16)
    lg2 = eng.model.forward(meta)
    ref_a, ref_b = oracle.logits(a), oracle.logits(b)
    close(lg1[:30], ref_a[:30])
    close(lg1[30:], ref_b)
    close(lg2, ref_a[30:])


def test_quantised_storage_matches_quant_aware_oracle():
    torch.manual_seed(2)
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="fp8_ds_mla", expert_dtype="nvfp4")
    w = init_random_weights(cfg, seed=5)
    oracle = OracleModel(cfg, w)
    eng = make_engine(cfg, w)
    p = torch.randint(0, cfg.vocab_size, (48,))
    from stkernel_b200.runtime.engine import Request, ScheduledSeq
    r = Request(0, p.tolist(), SamplingParams())
    r.row = eng.kv.alloc_row()
    t, n, ns = eng._stage([ScheduledSeq(r, 0, 48, True)])
    eng._upload(t, n, ns)
    lg = eng.model.forward(eng._build_meta(t, n, 16))
    ref = oracle.logits(p)
    close(lg, ref, tol=1e-2)


def test_padded_decode_bucket_ignores_stale_sample_rows():
    """A decode bucket wider than the step (3 requests in a 4-row bucket) must not read the staged row list: the
    entries past the uploaded ones still hold the row numbers of an earlier, larger step (here a 4-prompt prefill
    whose last sampling row is far beyond the bucket)."""
    torch.manual_seed(3)
    cfg = tiny_config()
    w = init_random_weights(cfg, seed=0)
    eng = make_engine(cfg, w)
    lens = (40, 33, 21, 50)
    ids = [eng.add_request(torch.randint(0, cfg.vocab_size, (n,)).tolist(),
                           SamplingParams(max_tokens=1 if i == 3 else 4)) for i, n in enumerate(lens)]
    eng.step()                                    # one mixed step: all four prompts prefill and sample
    assert eng.requests[ids[3]].finished
    stale = eng.buf.d_logit_rows[:4].tolist()
    assert max(stale) >= 4                        # what a 4-row decode graph would have indexed with
    seqs = eng.sched.schedule()
    assert len(seqs) == 3 and all(s.n == 1 for s in seqs)
    t, n_req, ns = eng._stage(seqs)
    eng._upload(t, n_req, ns)
    eng.buf.d_qstart[n_req + 1:5].fill_(n_req)    # the padding rule of `_decode_graph`
    ref = eng._run_model(t, n_req, ns, 16)
    eng.buf.d_logit_rows.fill_(10 ** 6)           # poison: any read of it would raise on this path
    got = eng._run_model(4, 4, 4, 16, identity_rows=True)
    assert got[:3].tolist() == ref.tolist()


def test_nonzero_device_status_fails_step_and_disables_symmetric_path():
    """Host-side injection: the status word the engine reads after a step says a peer-flag wait ran out.  The step
    must raise, be counted, and switch the symmetric collectives off so that later all-reduces take the library path."""
    from stkernel_b200.runtime.engine import DeviceStatusError

    class FakeSymm:
        enabled = True
        reason = None

        def eligible(self, x):
            return self.enabled

        def all_reduce(self, x):
            return x if self.enabled else None

        def disable(self, reason):
            self.enabled, self.reason = False, reason

    class FakeComm:
        def __init__(self):
            self.symm, self.world_size, self.library_calls = FakeSymm(), 2, 0

        def all_reduce(self, x):
            if self.symm.eligible(x) and self.symm.all_reduce(x) is not None:
                return x
            self.library_calls += 1
            return x

    torch.manual_seed(4)
    cfg = tiny_config()
    eng = make_engine(cfg, init_random_weights(cfg, seed=0))
    eng.model.comm = FakeComm()
    eng.add_request(torch.randint(0, cfg.vocab_size, (12,)).tolist(), SamplingParams(max_tokens=4))
    eng.step()
    assert eng.metrics.device_status_errors == 0
    eng._read_status = lambda: (2, 5)
    with pytest.raises(DeviceStatusError) as ei:
        eng.step()
    assert ei.value.code == 2 and ei.value.detail == 5
    assert eng.metrics.device_status_errors == 1
    assert eng.model.comm.symm.enabled is False and "device status 2" in eng.model.comm.symm.reason
    eng.model.comm.all_reduce(torch.zeros(4))
    assert eng.model.comm.library_calls == 1
    assert "stk:device_status_errors_total" in eng.metrics.render()


def test_indexer_scoring_in_query_subchunks_under_a_logits_budget():
    """With a logits budget of a few hundred bytes the indexer scores a prefill chunk a handful of query rows at a
    time; the selected rows, hence the text, must not change."""
    torch.manual_seed(5)
    cfg = tiny_config()
    w = init_random_weights(cfg, seed=0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (90, 41)]
    sp = SamplingParams(temperature=0.0, max_tokens=6)
    ref = make_engine(cfg, w).generate(prompts, sp)
    eng = make_engine(cfg, w)
    eng.model.indexer_logits_bytes = 256
    calls = []
    from stkernel_b200.ops import attention as A
    orig = A.indexer_scores
    try:
        A.indexer_scores = lambda q, *a, **k: (calls.append(q.shape[0]), orig(q, *a, **k))[1]
        out = eng.generate(prompts, sp)
    finally:
        A.indexer_scores = orig
    assert out == ref
    assert len(calls) > 20 and max(calls) * 4 * 22 <= 256 + 4 * 22          # rows x compressed rows x 4 bytes within budget


def test_log_probabilities_match_the_oracle_and_do_not_change_the_text():
    torch.manual_seed(0)
    cfg = tiny_config()
    w = init_random_weights(cfg, seed=0)
    eng = make_engine(cfg, w, chunk=48)
    p = torch.randint(0, cfg.vocab_size, (30,)).tolist()
    a = eng.add_request(p, SamplingParams(temperature=0.0, max_tokens=5, logprobs=3))
    b = eng.add_request(p, SamplingParams(temperature=0.0, max_tokens=5))            # same batch, not asking
    while eng.has_work():
        eng.step()
    ra, rb = eng.requests[a], eng.requests[b]
    assert ra.output == rb.output and len(ra.logprobs) == 5 and rb.logprobs == []
    _, logits = OracleModel(cfg, w).greedy_decode(torch.tensor(p), 5)
    ref = torch.log_softmax(logits.float(), -1)
    for i, (lp, top) in enumerate(ra.logprobs):
        assert abs(lp - float(ref[i, ra.output[i]])) < 2e-3
        assert len(top) == 3 and top[0][0] == ra.output[i]
        assert [t for t, _ in top] == ref[i].topk(3).indices.tolist()
    # sampled (temperature 1): the reported value is the model's log-probability of the token that was drawn
    c = eng.add_request(p, SamplingParams(temperature=1.0, seed=5, max_tokens=4, logprobs=0))
    while eng.has_work():
        eng.step()
    rc = eng.requests[c]
    assert len(rc.logprobs) == 4 and all(top == [] and lp <= 0 for lp, top in rc.logprobs)
