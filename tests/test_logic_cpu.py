"""Pure-logic tests: chunker budgets, SP coverage, DCP index math, trace/bench tooling, n-gram ceiling,
Markov refit."""
import json
import random

import pytest
import torch

from stkernel_b200.bench import check_quality, ngram_ceiling, streamgap, trace_tools
from stkernel_b200.bench.http_client import acceptance, spec_counters, summarize, unique_prompt
from stkernel_b200.bench.kernel_table import bucket_of, interval_union
from stkernel_b200.config import tiny_config
from stkernel_b200.models.dsv4_oracle import index_cache_computes
from stkernel_b200.runtime import planning as P
from stkernel_b200.runtime.metrics import Metrics, parse_prometheus
from stkernel_b200.tools import markov_refit


# ---- prefill chunker ---------------------------------------------------------------------------
def _validate(seq_lens, query_lens, ws, logits_bytes, offset=0):
    chunks = P.split_indexer_prefill_chunks(list(seq_lens), list(query_lens), ws, logits_bytes, request_offset=offset)
    max_elems = logits_bytes // 4
    covered = {i: 0 for i in range(len(seq_lens))}
    for req_slice, q_slice in chunks:
        reqs = list(range(req_slice.start - offset, req_slice.stop - offset))
        n = sum(seq_lens[r] for r in reqs)
        m = q_slice.stop - q_slice.start
        assert m >= 1
        if len(reqs) > 1:
            assert n <= ws and sum(query_lens[r] for r in reqs) * n <= max_elems
        elif n <= ws and query_lens[reqs[0]] * n > max_elems:
            assert m * n <= max_elems or m == 1
        for r in reqs:
            covered[r] += m if len(reqs) == 1 else query_lens[r]
    assert all(covered[r] == q for r, q in enumerate(query_lens))
    return chunks


def test_prefill_chunker_budgets():
    _validate([100, 200, 300], [10, 20, 30], 10_000, 4 * 10 ** 9)
    assert len(_validate([500, 500, 500], [50, 50, 50], 600, 4 * 10 ** 9)) == 3          # tight workspace: one each
    assert len(_validate([100_000], [4_096], 200_000, 4 * 10_000_000)) > 1                # query sub-chunking
    ch = P.split_indexer_prefill_chunks([10], [5], 100, 4 * 10 ** 9, request_offset=7)
    assert (ch[0][0].start, ch[0][0].stop) == (7, 8)
    rng = random.Random(0)
    for _ in range(200):
        n = rng.randint(1, 8)
        seq = [rng.randint(1, 5000) for _ in range(n)]
        q = [rng.randint(1, s) for s in seq]
        _validate(seq, q, rng.randint(100, 20000), 4 * rng.randint(1000, 10 ** 7), rng.randint(0, 5))


# ---- sequence-parallel indexer ranges --------------------------------------------------------------
def test_indexer_sp_coverage():
    tp = 4
    for a, b in ((140, 4236), (4236, 4801), (0, 3), (7, 7)):
        sizes = P.sp_gather_sizes((a, b), tp)
        n = b - a
        assert sum(sizes) == n and len(sizes) == tp
        assert all(x <= -(-n // tp) for x in sizes) and sizes == sorted(sizes, reverse=True)      # ceil split, short tail


# ---- DCP / PP / helpers ---------------------------------------------------------------------------
def test_dcp_index_math_and_topk_merge():
    for dcp, il in ((2, 1), (4, 1), (4, 64), (8, 16)):
        n = 1000
        counts = [0] * dcp
        for row in range(n):
            r = P.dcp_owner(row, dcp, il)
            assert P.dcp_local_index(row, dcp, il) == counts[r]                      # local rows are dense and in order
            assert P.dcp_global_row(counts[r], dcp, r, il) == row
            counts[r] += 1
        assert [P.dcp_local_rows(n, dcp, r, il) for r in range(dcp)] == counts
    rng = random.Random(1)
    scores = [rng.random() for _ in range(500)]
    per_rank = []
    for r in range(4):
        mine = [(scores[i], i) for i in range(500) if P.dcp_owner(i, 4) == r]
        per_rank.append(sorted(mine, key=lambda c: -c[0])[:32])
    want = [i for _, i in sorted(((scores[i], i) for i in range(500)), key=lambda c: (-c[0], c[1]))[:32]]
    assert P.merge_topk_candidates(per_rank, 32) == want
    # the model's tensor merge follows the same rule, ties included
    from stkernel_b200.models.dsv4 import dcp_merge_candidates
    tied = [round(x, 1) for x in scores]
    per_rank = []
    for r in range(4):
        mine = sorted(((tied[i], i) for i in range(500) if P.dcp_owner(i, 4) == r), key=lambda c: (-c[0], c[1]))[:32]
        per_rank.append(mine + [(float("-inf"), -1)] * 3)                            # short lists are padded
    gids = torch.tensor([[i for lst in per_rank for _, i in lst]], dtype=torch.int32)
    vals = torch.tensor([[v for lst in per_rank for v, _ in lst]], dtype=torch.float32)
    want = P.merge_topk_candidates([[c for c in lst if c[1] >= 0] for lst in per_rank], 32)
    assert dcp_merge_candidates(gids, vals, 32)[0].tolist() == want
    few = dcp_merge_candidates(gids[:, :35], vals[:, :35], 34)[0].tolist()          # one rank's 32 candidates + padding
    assert few[:32] == [i for _, i in per_rank[0][:32]] and few[32:] == [-1, -1]


def test_pp_ranges_and_index_cache_pattern():
    for n, pp in ((48, 4), (43, 4), (6, 8)):
        spans = [P.pp_layer_range(n, pp, r) for r in range(pp)]
        assert spans[0][0] == 0 and spans[-1][1] == n and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
    ratios = (4, 0, 4, 4, 0, 4, 4, 4)
    pat = P.index_cache_pattern(ratios, 8, 3)
    assert pat == [True, None, False, False, None, True, False, False]
    cfg = tiny_config(num_hidden_layers=8, compress_ratios=ratios, index_topk_freq=3)
    assert [p if p is not None else False for p in pat] == [index_cache_computes(cfg, i) for i in range(8)]
    for freq in (1, 2, 7, 100):
        assert P.index_cache_pattern((0, 4, 4), 3, freq)[1] is True                   # first C4A always computes


# ---- profiling tools ---------------------------------------------------------------------------
def _trace():
    ev = []
    t = 0.0
    for i in range(10):
        ev.append({"cat": "kernel", "name": "stk::gemm_kernel<64>", "ts": t, "dur": 10.0, "args": {"stream": 7}})
        t += 10.0 + (30.0 if i == 4 else 2.0)
        ev.append({"cat": "kernel", "name": "stk::sparse_mla_tc_kernel<64>", "ts": t, "dur": 5.0, "args": {"stream": 7}})
        t += 5.0 + 1.0
    ev.append({"cat": "kernel", "name": "ncclDevKernel_AllReduce", "ts": 80.0, "dur": 25.0, "args": {"stream": 9}})
    ev.append({"cat": "cpu_op", "name": "aten::mm", "ts": 0.0, "dur": 999.0})
    return {"traceEvents": ev}


def test_bucket_regex_and_interval_union():
    assert bucket_of("ncclDevKernel_AllReduce_Sum") == "comms" and bucket_of("stk::oneshot_allreduce_kernel") == "comms"
    assert bucket_of("stk::expert_fc1_kernel<4>") == "moe" and bucket_of("stk::sparse_mla_tc_kernel<64>") == "attn/indexer"
    assert bucket_of("stk::gemm_kernel<64, true>") == "gemm" and bucket_of("stk::mhc_cluster_kernel<24>") == "mhc"
    assert bucket_of("stk::rmsnorm_kernel") == "norm/rope/quant" and bucket_of("Memcpy HtoD") == "memops"
    assert bucket_of("something_else") == "other"
    assert interval_union([(0, 10), (5, 15), (20, 30)]) == 25 and interval_union([]) == 0
    assert interval_union([(0, 10), (2, 3), (10, 12)]) == 12


def test_trace_tools_reports():
    evs = trace_tools.gpu_events(_trace())
    assert len(evs) == 21
    tab = trace_tools.bucket_table(evs)
    assert tab["buckets"]["gemm"] == 100.0 and tab["buckets"]["attn/indexer"] == 50.0 and tab["buckets"]["comms"] == 25.0
    assert tab["busy_us"] == 173.0                             # the collective overlaps a kernel: not counted twice
    assert abs(tab["busy_us"] + tab["idle_us"] - tab["span_us"]) < 1e-6
    g = trace_tools.gap_report(evs)
    assert g["stream"] == 7 and g["n_kernels"] == 20
    assert g["largest"][0][0] == 30.0 and "gemm" in g["largest"][0][1] and "sparse_mla" in g["largest"][0][2]
    assert sum(g["hist"]) == 19
    st = g["kernel_stats"]["stk::gemm_kernel<64>"]
    assert st["n"] == 10 and st["min"] == st["max"] == 10.0
    c = trace_tools.concurrent_report(evs)
    assert c[0]["gap_us"] == 30.0 and c[0]["other"][0][0].startswith("nccl") and c[0]["covered_us"] == 23.0
    assert "bucket gemm" in trace_tools.format_table(tab, steps=10)
    assert trace_tools.percentile([1, 2, 3, 4, 100], 0.5) == 3


def test_nccl_fingerprint_ignores_volatile_fields():
    a = ("host1:123:456 [0] NCCL INFO Channel 00/24 : 0 1 2 3\nhost1:123:456 [0] NCCL INFO Trees [0] 1/-1/-1->0->-1\n"
         "host1:123:456 [0] NCCL INFO comm 0x55aa rank 0 nranks 4 cudaDev 0 - Init COMPLETE\nhost1:1:2 [0] NCCL INFO Using network Socket\n")
    b = a.replace("host1:123:456", "host9:9:9").replace("0x55aa", "0x7f00")
    fa, na = trace_tools.nccl_fingerprint(a)
    assert na == 3 and (fa, na) == trace_tools.nccl_fingerprint(b)
    assert trace_tools.nccl_fingerprint(a.replace("0 1 2 3", "0 2 1 3"))[0] != fa


def test_prometheus_and_acceptance_formulas():
    m = Metrics()
    m.record_spec(5, 3); m.record_spec(5, 0); m.record_spec(5, 5)
    after = spec_counters(parse_prometheus(m.render("x")))
    assert after["vllm:spec_decode_num_drafts_total"] == 3 and after["vllm:spec_decode_num_draft_tokens_total"] == 15
    assert after["vllm:spec_decode_num_accepted_tokens_total"] == 8
    assert after["vllm:spec_decode_num_accepted_tokens_per_pos_total"] == 8            # labels collapsed: 2+2+2+1+1
    acc = acceptance({}, after)
    assert abs(acc["raw"] - 8 / 15) < 1e-9 and abs(acc["accepted_per_step"] - 8 / 3) < 1e-9
    assert abs(acc["acc"] - (8 + 8) / (3 + 15)) < 1e-9                               # the legacy substring convention
    assert acceptance({}, {}) == {"acc": 0.0, "raw": 0.0, "accepted_per_step": 0.0}
    assert summarize([3, 1, 2]) == {"mean": 2.0, "median": 2, "min": 1, "max": 3}
    assert unique_prompt(1, 5) == unique_prompt(1, 5) != unique_prompt(2, 5)


def test_quality_document_and_grading():
    doc = check_quality.build_document(2000, 3)
    pos = [doc.index(s) / len(doc) for s, _, _ in check_quality.FACTS]
    assert all(abs(p - d) < 0.05 for p, d in zip(pos, (0.25, 0.5, 0.75)))
    assert check_quality.grade("It was Dr. Halvorsen, on 14 March 1997.", ("halvorsen", "14 march 1997"))
    assert not check_quality.grade("Halvorsen in 1998", ("halvorsen", "14 march 1997"))
    st = [0.0, 0.1, 0.2, 0.3, 5.0, 5.1, 9.0, 9.1, 9.2]
    r = streamgap.window_rates(st, 0.0, 0.35, 8.0)
    assert r["before"] > r["during"] and r["after"] > r["during"]
    assert streamgap.largest_gaps(st, 0.0, 2)[0][0] == pytest.approx(4.7)


# ---- n-gram ceiling ---------------------------------------------------------------------------
def test_ngram_ceiling_pmf_index_and_no_future_leak():
    pmf = ngram_ceiling.accept_len_pmf(ngram_ceiling.parse_curve("78.5,56.4,39.6,28.6,21.5"))
    assert abs(sum(pmf) - 1) < 1e-9 and abs(pmf[0] - 0.215) < 1e-9 and abs(pmf[5] - 0.215) < 1e-9
    with pytest.raises(ValueError):
        ngram_ceiling.parse_curve("50,60")
    with pytest.raises(ValueError):
        ngram_ceiling.parse_curve("150")
    toks = [1, 2, 3, 4, 5, 9, 1, 2, 3, 4, 5, 7]
    idx = ngram_ceiling.GramIndex(toks, 3)
    idx.advance(9)                                          # suffix ending at 9 is (1,2,3) again
    assert idx.longest(9, 16) == (3, 3)
    idx2 = ngram_ceiling.GramIndex(toks, 3)
    idx2.advance(3)
    assert idx2.longest(3, 16) == (0, -1)                  # the only other (1,2,3) ends at 9, in the future of t=3
    rep = list(range(50)) * 6
    st = ngram_ceiling.simulate(rep[:60], rep[60:], pmf, threshold=4)
    assert st["steps"]["hybrid"] < st["steps"]["drafter"] and st["steps"]["oracle"] <= st["steps"]["hybrid"]
    assert st["copy_accepted"] / st["copy_steps"] > 4.0
    r3 = random.Random(3)
    rnd = [r3.randrange(10 ** 6) for _ in range(400)]
    st2 = ngram_ceiling.simulate(rnd[:100], rnd[100:], pmf)
    assert st2["copy_steps"] == 0 and st2["steps"]["hybrid"] == st2["steps"]["drafter"]
    assert ngram_ceiling.simulate([1], [2], pmf) is None


# ---- Markov refit ---------------------------------------------------------------------------
def test_markov_refit_recovers_bigram_structure(tmp_path):
    V = 64
    rng = random.Random(0)
    nxt = {i: (i * 7 + 3) % V for i in range(V)}              # a deterministic successor for every token
    docs = []
    for _ in range(200):
        t = rng.randrange(V)
        seq = [t]
        for _ in range(30):
            t = nxt[t] if rng.random() < 0.8 else rng.randrange(V)
            seq.append(t)
        docs.append(seq)
    pairs, uni, total = markov_refit.count_bigrams(docs)
    out = markov_refit.refit(pairs, uni, total, V, rank=48)
    bias = out["markov_w1"] @ out["markov_w2"].T
    hit = sum(int(bias[i].argmax()) == nxt[i] for i in range(V))
    assert hit >= 0.9 * V and out["meta"]["blend"] == 1.0 and out["meta"]["energy"] > 0.5
    # blending with a shipped head moves the result between the two
    base = (torch.randn(V, 8) * 0.1, torch.randn(V, 8) * 0.1)
    keep = markov_refit.refit(pairs, uni, total, V, rank=8, blend=0.0, base=base)
    assert torch.allclose(keep["markov_w1"] @ keep["markov_w2"].T, base[0] @ base[1].T, atol=1e-3)
    with pytest.raises(ValueError):
        markov_refit.refit(pairs, uni, total, V, rank=8, blend=1.5)
    with pytest.raises(ValueError):
        markov_refit.pmi_operator(pairs, uni, total, V, min_count=10 ** 6)
    # the payload passes the serving loader's sideload contract
    from stkernel_b200.spec.dspark import MarkovHead
    p = tmp_path / "m.pt"
    torch.save({"markov_w1": out["markov_w1"], "markov_w2": out["markov_w2"], "meta": out["meta"]}, p)
    MarkovHead(torch.zeros(V, 48).bfloat16(), torch.zeros(V, 48).bfloat16()).sideload(str(p), V, 48)


def test_span_recorder_accounting():
    from stkernel_b200.utils import spans
    r = spans.SpanRecorder(decode_rows=6)
    assert r.phase(6) == "decode" and r.phase(7) == "prefill"
    r.add_ms("decode", "attention", 1.5)
    r.add_ms("decode", "attention", 0.5)
    r.add_ms("decode", "moe", 1.0)
    r.add_ms("prefill", "moe", 10.0)
    rep = r.report()
    assert "[decode] 3.00 ms in 3 spans" in rep and "attention" in rep and "[prefill] 10.00 ms" in rep
    assert rep.index("attention") < rep.index("moe")           # sorted by time within a phase
    with spans.span("x"):                                       # disabled (STK_PROF unset): a null context
        pass
    with r.span("cpu-only", 1):                                 # no CUDA here: passes through without recording
        pass
    assert ("decode", "cpu-only") not in r.totals


def test_mhc_split_weight_cache_follows_the_tensor_not_its_address():
    """The bf16 hi/lo split of an mHC mix matrix is cached per weight tensor; a new tensor that the allocator places at a
    freed tensor's address must get its own split."""
    import torch
    from stkernel_b200.ops import functional as Fn
    seen = []
    for seed in range(6):
        fn = torch.randn(24, 256, generator=torch.Generator().manual_seed(seed)) * 0.02
        w = Fn._mhc_wcat(fn, 24)
        assert torch.equal(w[:24].float() + w[32:56].float(), (fn.to(torch.bfloat16).float() + (fn - fn.to(torch.bfloat16).float()).to(torch.bfloat16).float()))
        assert Fn._mhc_wcat(fn, 24) is w                     # second call: cached
        seen.append(fn.data_ptr())
        del fn, w
    # (the CPU allocator usually hands the same block out again: the case the cache has to survive)


def test_c_api_header_is_generated_from_the_sources():
    """`stk_c_api.h` lists every exported entry point and is regenerated whenever a signature changes."""
    from stkernel_b200.csrc import gen_c_api
    from stkernel_b200.ops import _lib
    text = gen_c_api.HEADER.read_text()
    assert text == gen_c_api.render(), "run `python -m stkernel_b200.csrc.gen_c_api`"
    for name in _lib._parse_signatures():
        assert f" {name}(" in text


def test_replay_drafter_counts_only_steps_drafted_from_a_valid_oracle():
    """The bench's stand-in drafter replays a recorded text; once the request emits something else the recording is no
    oracle any more, and neither its steps nor its tokens may enter the acceptance figures."""
    from types import SimpleNamespace
    from stkernel_b200.bench.decode_bench import ReplayDrafter
    rec = {7: list(range(100, 160))}
    d = ReplayDrafter(rec, vocab=1000, acceptance=(1.0, 1.0, 1.0), seed=0)
    d.counting = True
    req = SimpleNamespace(params=SimpleNamespace(seed=7), output=[])
    assert d(req, [1, 2, 3]) == [100, 101, 102]                 # acceptance 1.0: the recorded continuation
    req.output = [100, 101, 102, 103]                           # three accepted + the bonus token
    assert d(req, [1, 2, 3]) == [104, 105, 106]
    assert (d.steps_in_sync, d.tokens_in_sync) == (1, 4)
    req.output = req.output + [104, 999]                        # the engine emitted a token the recording does not have
    assert d(req, [1, 2, 3]) == [1, 2, 3]                       # out of sync: the device drafts go through
    assert (d.steps_in_sync, d.tokens_in_sync) == (2, 6)        # the step that just ended was still drafted validly
    req.output = req.output + [5]
    d(req, [1, 2, 3])
    assert (d.steps_in_sync, d.tokens_in_sync) == (2, 6)        # steps after the divergence are not counted


def test_model_config_rejects_wrongly_typed_fields_as_configuration_errors():
    """A `config.json` with a string where a number belongs (or a scalar where a list belongs) fails with a
    configuration error that names the field; randomised over all fields."""
    import dataclasses
    from stkernel_b200.config import ConfigError, model_config_from_hf
    base = {k: (list(v) if isinstance(v, tuple) else v) for k, v in dataclasses.asdict(tiny_config()).items()}
    assert model_config_from_hf(base) == tiny_config()
    for name, value in (("hidden_size", "4096"), ("compress_ratios", 4), ("norm_topk_prob", 1), ("rope_theta", "x"),
                        ("scoring_func", 3), ("num_hidden_layers", 0), ("hc_eps", float("nan")), ("o_groups", True)):
        with pytest.raises(ConfigError) as e:
            model_config_from_hf({**base, name: value})
        assert name in str(e.value)
    rng = random.Random(0)
    vals = [None, 0, -1, 2, 64, 0.5, "", "fp8", [], [4, 0], True, {}, 10 ** 9]
    for _ in range(3000):
        hf = dict(base)
        for k in rng.sample(list(base), rng.randint(1, 4)):
            hf[k] = rng.choice(vals)
        try:
            cfg = model_config_from_hf(hf)
            [cfg.layer_kind(i) for i in range(cfg.num_hidden_layers)]
        except ConfigError:
            pass
