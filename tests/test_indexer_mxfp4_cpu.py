"""MXFP4 indexer operands (e2m1 values, one ue8m0 scale per 32) on the reference path: the q preparation, the paged
key cache, and the engine against the naive oracle."""
import pytest
import torch

from stkernel_b200.config import ConfigError, EngineConfig, SchedulerConfig, tiny_config
from stkernel_b200.models.dsv4 import DictSource, build_model_weights
from stkernel_b200.models.dsv4_oracle import OracleModel
from stkernel_b200.models.weights import init_random_weights
from stkernel_b200.ops import attention as A
from stkernel_b200.ops import cache as C
from stkernel_b200.ops import functional as Fn
from stkernel_b200.ops import reference as R
from stkernel_b200.runtime.engine import Engine, SamplingParams


@pytest.fixture(autouse=True)
def fp32_acts():
    Fn.set_cpu_act_dtype(torch.float32)
    yield
    Fn.set_cpu_act_dtype(torch.bfloat16)


def test_q_preparation_blocks_and_weights():
    torch.manual_seed(0)
    t, ih, d, rd = 5, 4, 128, 64
    q = torch.randn(t, ih, d) * torch.logspace(-2, 1, d)          # a wide range inside a row: block scales matter
    w = torch.randn(t, ih)
    pos = torch.arange(t) + 100
    inv = Fn.inv_freq(rd, 10000.0, "cpu")
    qq, wf = C.indexer_q_prep(q.to(torch.bfloat16), w, pos, inv, rd, True, fmt="mxfp4")
    assert qq.packed.shape == (t, ih, d // 2) and qq.scales.shape == (t, ih, d // 32) and qq.shape == (t, ih, d)
    assert torch.allclose(wf, w * d ** -0.5 * ih ** -0.5)         # no q scale folded in: the block scales stay with q
    # against the unquantised roped q: every block within the 4-bit step of its own scale
    ang = pos.float()[:, None] * inv[None, :]
    ref, _ = R.indexer_q_prepare(q.to(torch.bfloat16), w, torch.cos(ang), torch.sin(ang), rd, quantize=False)
    deq = qq.dequant()
    blocks_ref, blocks = ref.view(t, ih, d // 32, 32), deq.view(t, ih, d // 32, 32)
    step = torch.exp2(qq.scales.float() - 127.0)[..., None]        # spacing of the coarsest e2m1 interval is 2 steps
    assert ((blocks - blocks_ref).abs() <= step + 1e-6).all()
    amax = blocks_ref.abs().amax(-1, keepdim=True)
    assert (6.0 * step >= amax - 1e-6).all() and (3.0 * step < amax + 1e-6).all()     # the smallest scale that fits
    # row slices keep values and scales together
    assert torch.equal(qq[1:3].dequant(), deq[1:3])


def test_paged_key_cache_roundtrip_and_size():
    d, rd = 128, 64
    fp8 = C.PagedCache.allocate(3, d, rd, True, "indexer", "cpu")
    fp4 = C.PagedCache.allocate(3, d, rd, True, "indexer", "cpu", fp4=True)
    assert fp4.data_bytes == 64 and fp4.page_stride < 0.55 * fp8.page_stride      # 68 against 132 bytes per row
    rows = torch.randn(7, d) * 3
    slots = torch.tensor([0, 5, 63, 64, 130, -1, 191])
    fp4.write_rows_cpu(slots, rows)
    got, sc = fp4.read_rows_cpu(slots)
    assert sc is None
    want = R.dequant_mxfp4(*R.quant_mxfp4(rows))
    keep = slots >= 0
    assert torch.equal(got[keep], want[keep]) and got[~keep].abs().sum() == 0
    with pytest.raises(AssertionError):
        C.PagedCache.page_bytes(d, rd, True, "latent", fp4=True)


def test_config_checks_block_structure():
    with pytest.raises(ConfigError):
        tiny_config(indexer_dtype="mxfp4").validate()                 # rope 16 / index dim 32: not whole blocks
    with pytest.raises(ConfigError):
        tiny_config(indexer_dtype="int4").validate()
    tiny_config(indexer_dtype="mxfp4", qk_rope_head_dim=32, index_head_dim=64, head_dim=96).validate()


@pytest.mark.parametrize("kv_dtype", ["bf16", "fp8_ds_mla"])
def test_engine_matches_oracle_with_mxfp4_indexer(kv_dtype):
    torch.manual_seed(0)
    cfg = tiny_config(indexer_dtype="mxfp4", qk_rope_head_dim=32, index_head_dim=64, head_dim=96,
                      kv_cache_dtype=kv_dtype, num_hidden_layers=3, compress_ratios=(4, 0, 4), index_topk_freq=2)
    w = init_random_weights(cfg, seed=0)
    oracle = OracleModel(cfg, w)
    ec = EngineConfig(model=cfg, sched=SchedulerConfig(max_model_len=512, max_num_seqs=4, max_num_batched_tokens=48,
                                                       graph_cap=0)).validate()
    eng = Engine(ec, build_model_weights(cfg, DictSource(w), "cpu"), "cpu", max_context=512)
    assert all(c.fp4 for c in eng.kv.idx_cache.values())
    prompts = [torch.randint(0, cfg.vocab_size, (n,)).tolist() for n in (100, 71)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
    for p, o in zip(prompts, outs):
        ref_ids, _ = oracle.greedy_decode(torch.tensor(p), 8)
        assert o == ref_ids.tolist()
    # the 4-bit operands select mostly the rows the 8-bit ones select
    cfg8 = tiny_config(qk_rope_head_dim=32, index_head_dim=64, head_dim=96, kv_cache_dtype=kv_dtype,
                       num_hidden_layers=3, compress_ratios=(4, 0, 4), index_topk_freq=2)
    eng8 = Engine(EngineConfig(model=cfg8, sched=ec.sched).validate(), build_model_weights(cfg8, DictSource(w), "cpu"), "cpu",
                  max_context=512)
    eng8.generate(prompts[:1], SamplingParams(temperature=0.0, max_tokens=1))
    eng4 = Engine(ec, build_model_weights(cfg, DictSource(w), "cpu"), "cpu", max_context=512)
    eng4.generate(prompts[:1], SamplingParams(temperature=0.0, max_tokens=1))
    a, b = eng8.model.topk_buffer[0].tolist(), eng4.model.topk_buffer[0].tolist()
    overlap = len(set(a) & set(b)) / len(set(a))
    assert overlap >= 0.6, (a, b)
