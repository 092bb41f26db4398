"""The engine on a B200: tiny config against the quantisation-aware oracle, CUDA-graph replay
against eager execution, and a Flash-shaped single layer smoke test."""
import pytest
import torch

from stkernel_b200.config import EngineConfig, SchedulerConfig, flash_config, tiny_config
from stkernel_b200.models.dsv4 import DictSource, RandomSource, build_model_weights
from stkernel_b200.models.dsv4_oracle import OracleModel
from stkernel_b200.models.weights import init_random_weights
from stkernel_b200.ops import _lib
from stkernel_b200.runtime.engine import Engine, Request, SamplingParams, ScheduledSeq

pytestmark = pytest.mark.gpu


def make_engine(cfg, src, graph_cap=0, seqs=4, ctx=512, chunk=4096):
    ec = EngineConfig(model=cfg, sched=SchedulerConfig(max_model_len=ctx, max_num_seqs=seqs,
                                                       max_num_batched_tokens=chunk, graph_cap=graph_cap)).validate()
    weights = build_model_weights(cfg, src, "cuda:0")
    return Engine(ec, weights, "cuda:0", max_context=ctx)


@pytest.mark.parametrize("dense,kv", [("bf16", "bf16"), ("fp8", "fp8_ds_mla")])
def test_tiny_logits_match_oracle(dense, kv):
    torch.manual_seed(0)
    # dims chosen so that every fused weight (wq_a|wkv, wq_b|indexer wq_b, w1|w3) splits on 128-row
    # block boundaries, as in the production shape: joint and separate block quantisation then agree
    cfg = tiny_config(dense_dtype=dense, kv_cache_dtype=kv, expert_dtype="nvfp4", num_hidden_layers=3,
                      compress_ratios=(4, 0, 4), index_topk_freq=2, head_dim=144, num_attention_heads=8,
                      q_lora_rank=128, o_lora_rank=128)
    w = init_random_weights(cfg, seed=7)
    oracle = OracleModel(cfg, w)
    eng = make_engine(cfg, DictSource(w))
    p = torch.randint(0, cfg.vocab_size, (70,))
    r = Request(0, p.tolist(), SamplingParams())
    r.row = eng.kv.alloc_row()
    t, n, ns = eng._stage([ScheduledSeq(r, 0, 40, False)])
    eng._upload(t, n, ns)
    lg1 = eng.model.forward(eng._build_meta(t, n, 32))
    t, n, ns = eng._stage([ScheduledSeq(r, 40, 30, True)])
    eng._upload(t, n, ns)
    lg2 = eng.model.forward(eng._build_meta(t, n, 32))
    torch.cuda.synchronize()
    _lib.check_status()
    got = torch.cat([lg1, lg2]).float().cpu()
    ref = oracle.logits(p)
    rel = ((got - ref).norm() / ref.norm()).item()
    agree = (got.argmax(-1) == ref.argmax(-1)).float().mean().item()
    print(f"oracle check {dense}/{kv}: rel {rel:.4f} argmax {agree:.3f}")
    # measured on B200: bf16 1.2 % / 0.986, fp8 (weights, activations and KV all quantised; the oracle keeps the
    # activations unquantised) 8.7 % / 0.87 over three layers of a 256-wide model with nearly flat random logits
    assert rel < (0.02 if dense == "bf16" else 0.12), rel
    assert agree > (0.95 if dense == "bf16" else 0.8), agree


def test_graph_replay_matches_eager_and_is_deterministic():
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="fp8_ds_mla", expert_dtype="nvfp4")
    w = init_random_weights(cfg, seed=1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (33, 64, 17)]
    outs = []
    for cap in (0, 8, 8):
        eng = make_engine(cfg, DictSource(w), graph_cap=cap)
        outs.append(eng.generate(prompts, SamplingParams(temperature=0.7, seed=5, max_tokens=24)))
        torch.cuda.synchronize()
        _lib.check_status()
    assert outs[1] == outs[2]
    assert outs[0] == outs[1]


def test_stream_fork_and_dependent_launch_do_not_change_tokens():
    """The second-stream fork of the decode sub-blocks and programmatic dependent launch only reorder independent work:
    sampled tokens equal those of the plain single-stream chain — compared eagerly and, separately, under graph replay
    (graph buckets pad the batch, which changes split counts and with them summation order, so eager and replayed runs
    are not compared with each other here)."""
    cfg = flash_config(num_layers=4, n_routed_experts=16, vocab_size=4096)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (300, 41)]
    for cap in (0, 4):
        outs = {}
        for fork, pdl in ((0, 0), (64, 0), (0, 1), (64, 1)):
            _lib.call("stk_set_pdl", pdl)
            try:
                eng = make_engine(cfg, RandomSource(3), graph_cap=cap, ctx=2048, chunk=512)
                eng.model.fork_max_t = fork
                outs[(fork, pdl)] = eng.generate(prompts, SamplingParams(temperature=0.8, seed=11, max_tokens=12))
                torch.cuda.synchronize()
                _lib.check_status()
            finally:
                _lib.call("stk_set_pdl", 1)
        base = outs[(0, 0)]
        for k, v in outs.items():
            assert v == base, (cap, k)


def test_flash_shaped_layer_runs():
    cfg = flash_config(num_layers=2, n_routed_experts=16, vocab_size=4096)
    eng = make_engine(cfg, RandomSource(0), graph_cap=4, ctx=4096, chunk=1024)
    prompts = [torch.randint(0, cfg.vocab_size, (1500,)).tolist(), torch.randint(0, cfg.vocab_size, (300,)).tolist()]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))
    torch.cuda.synchronize()
    _lib.check_status()
    assert all(len(o) == 6 for o in outs)
    assert all(0 <= t < cfg.vocab_size for o in outs for t in o)


def test_dspark_speculative_engine_runs_and_agrees_with_plain_prefix():
    """Draft + coupled verify on the device.  Kernel selection differs between a 1-row decode step and a
    (1+N)-row verify step, so bitwise-equal text is not guaranteed; the first tokens (same prefill) are,
    and with greedy sampling on well-separated logits most of the text agrees."""
    from stkernel_b200.config import SpecConfig
    from stkernel_b200.spec.dspark import build_draft_weights
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="fp8_ds_mla", expert_dtype="nvfp4", n_mtp_layers=2,
                      dspark_target_layer_ids=(0, 1), dspark_markov_rank=16)
    w = init_random_weights(cfg, seed=3)
    sc = SchedulerConfig(max_model_len=512, max_num_seqs=4, max_num_batched_tokens=256, graph_cap=0)
    tw = build_model_weights(cfg, DictSource(w), "cuda:0")
    plain = Engine(EngineConfig(model=cfg, sched=sc).validate(), tw, "cuda:0", max_context=512)
    dw = build_draft_weights(cfg, DictSource(w), tw, "cuda:0")
    ec = EngineConfig(model=cfg, sched=sc, spec=SpecConfig(method="dspark", num_speculative_tokens=3, markov_topk=8)).validate()
    spec = Engine(ec, tw, "cuda:0", max_context=512, draft_weights=dw)
    torch.manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (40, 150, 7)]
    sp = SamplingParams(temperature=0.0, max_tokens=24)
    ref = plain.generate(prompts, sp)
    got = spec.generate(prompts, sp)
    torch.cuda.synchronize()
    _lib.check_status()
    assert [len(g) for g in got] == [24, 24, 24]
    assert [g[0] for g in got] == [r[0] for r in ref]
    m = spec.metrics
    assert m.spec_num_drafts > 0 and m.spec_num_accepted_tokens <= m.spec_num_draft_tokens


def test_dspark_step_graph_replay_matches_eager():
    """The captured speculative step (verify + context insert + draft block + Markov chain) gives the same text
    as the eager one: same kernels, same inputs."""
    from stkernel_b200.config import SpecConfig
    from stkernel_b200.spec.dspark import build_draft_weights
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="fp8_ds_mla", expert_dtype="nvfp4", n_mtp_layers=2,
                      dspark_target_layer_ids=(0, 1), dspark_markov_rank=16)
    w = init_random_weights(cfg, seed=4)
    tw = build_model_weights(cfg, DictSource(w), "cuda:0")
    dw = build_draft_weights(cfg, DictSource(w), tw, "cuda:0")
    torch.manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (30, 70)]
    sp = SamplingParams(temperature=0.8, seed=9, max_tokens=20)
    outs = []
    for cap in (0, 64):
        sc = SchedulerConfig(max_model_len=512, max_num_seqs=4, max_num_batched_tokens=256, graph_cap=cap)
        ec = EngineConfig(model=cfg, sched=sc, spec=SpecConfig(method="dspark", num_speculative_tokens=3, markov_topk=8)).validate()
        eng = Engine(ec, tw, "cuda:0", max_context=512, draft_weights=dw)
        outs.append(eng.generate(prompts, sp))
        torch.cuda.synchronize()
        _lib.check_status()
        if cap:
            assert any(isinstance(k, tuple) and k[0] == "spec" for k in eng._graphs)
    assert outs[0] == outs[1]


def test_dspark_text_does_not_depend_on_what_the_drafter_proposes():
    """Losslessness on the GPU, with the kernels held fixed: two speculative engines that differ only in their proposals
    (one never accepted, one replaying the other's text so that nearly every draft is accepted) emit the same text for
    the same seeds.  Both run the same verify-row kernels, so this isolates the accept / rollback / context-insert
    logic from the kernel-selection differences between 1-row and (1+N)-row steps."""
    from stkernel_b200.bench.decode_bench import ReplayDrafter
    from stkernel_b200.config import SpecConfig
    from stkernel_b200.spec.dspark import build_draft_weights
    cfg = tiny_config(dense_dtype="bf16", kv_cache_dtype="fp8_ds_mla", expert_dtype="nvfp4", n_mtp_layers=2,
                      dspark_target_layer_ids=(0, 1), dspark_markov_rank=16)
    w = init_random_weights(cfg, seed=5)
    tw = build_model_weights(cfg, DictSource(w), "cuda:0")
    dw = build_draft_weights(cfg, DictSource(w), tw, "cuda:0")
    torch.manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (33, 90)]
    sc = SchedulerConfig(max_model_len=512, max_num_seqs=4, max_num_batched_tokens=256, graph_cap=0)
    ec = EngineConfig(model=cfg, sched=sc, spec=SpecConfig(method="dspark", num_speculative_tokens=3, markov_topk=8)).validate()

    def run(override_factory):
        eng = Engine(ec, tw, "cuda:0", max_context=512, draft_weights=dw)
        eng.draft_override = override_factory()
        ids = [eng.add_request(p, SamplingParams(temperature=0.7, seed=40 + i, max_tokens=24)) for i, p in enumerate(prompts)]
        while eng.has_work():
            eng.step()
        torch.cuda.synchronize()
        _lib.check_status()
        return [list(eng.requests[i].output) for i in ids], eng.metrics

    never, m0 = run(lambda: (lambda req, drafts: [(cfg.vocab_size - 1)] * len(drafts)))
    recorded = {40 + i: t for i, t in enumerate(never)}
    replay, m1 = run(lambda: ReplayDrafter(recorded, cfg.vocab_size, acceptance=(1.0, 1.0, 1.0)))
    assert m1.spec_num_accepted_tokens > m0.spec_num_accepted_tokens + 10      # the second run really accepted drafts
    assert replay == never
