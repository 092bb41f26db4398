"""Checkpoint layout: safetensors reader/writer, fp8 + MXFP4 expansion, bit-exact re-quantisation,
TP shard plan."""
import json
import os

import pytest
import torch

from stkernel_b200.config import tiny_config, flash_config
from stkernel_b200.models import loader as L
from stkernel_b200.models.dsv4 import DictSource, build_model_weights
from stkernel_b200.models.weights import init_random_weights, weight_shapes
from stkernel_b200.ops import reference as R


def test_safetensors_roundtrip_all_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(4, 4).bfloat16(), "c": torch.arange(6, dtype=torch.int32).view(2, 3),
         "d": torch.randn(8, 8).to(torch.float8_e4m3fn), "e": torch.randint(0, 255, (2, 4), dtype=torch.uint8),
         "f": torch.empty(0, 3)}
    p = str(tmp_path / "x.safetensors")
    L.write_safetensors(p, t, {"e": "F8_E8M0"})
    idx = L.SafetensorsIndex(p)
    assert set(idx.keys()) == set(t)
    for k, v in t.items():
        got = idx.get(k)
        assert got.shape == v.shape
        assert torch.equal(got.view(torch.uint8), v.view(torch.uint8)) if v.numel() else True
    assert idx.dtype_name("e") == "F8_E8M0"
    from safetensors import safe_open                     # the file is a valid safetensors file for other readers
    with safe_open(p, "pt") as f:
        assert torch.equal(f.get_tensor("a"), t["a"]) and torch.equal(f.get_tensor("b"), t["b"])
    bad = str(tmp_path / "bad.safetensors")
    open(bad, "wb").write((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(ValueError):
        L.SafetensorsIndex(bad)


@pytest.mark.parametrize("rule", ["ue8m0", "absmax"])
def test_checkpoint_source_reproduces_codes(tmp_path, rule):
    cfg = tiny_config(dense_dtype="fp8", expert_dtype="mxfp4", n_mtp_layers=1, dspark_target_layer_ids=(1,), dspark_markov_rank=8)
    masters = init_random_weights(cfg, seed=3)
    path = str(tmp_path / "ckpt")
    L.write_checkpoint(path, cfg, masters, shards=3, scale_rule=rule)
    assert L.load_model_config(path) == cfg
    src = L.CheckpointSource(path)
    assert src.fp8_scale_rule == rule
    assert src.missing(cfg) == [] and src.unexpected(cfg) == []
    # an fp8 tensor expands to exactly q * scale, and quantising that again gives the stored codes
    name = "layers.0.attn.wq_b.weight"
    q_disk, s_disk = src.raw(name)
    w = src.get(name, weight_shapes(cfg)[name][0], "cpu")
    q2, s2 = R.quant_fp8_block128_weight(w, ue8m0=(rule == "ue8m0"))
    assert torch.equal(q2.view(torch.uint8), q_disk.view(torch.uint8))
    # experts: the MXFP4 values survive expansion and re-quantisation exactly (a group whose largest code
    # is below 4 re-encodes with a smaller exponent and larger codes: other bits, same numbers)
    en = "layers.0.ffn.experts.2.w1.weight"
    p_disk, sb_disk = src.raw(en)
    we = src.get(en, weight_shapes(cfg)[en][0], "cpu")
    assert torch.equal(we, R.dequant_mxfp4(p_disk, sb_disk))
    p2, sb2 = R.quant_mxfp4(we)
    assert torch.equal(R.dequant_mxfp4(p2, sb2), we)
    with pytest.raises(ValueError):
        src.get(name, (1, 1), "cpu")
    with pytest.raises(KeyError):
        src.get("nope.weight", (1,), "cpu")
    # the model built from the checkpoint equals the model built from the expanded masters
    a = build_model_weights(cfg, src, "cpu")
    expanded = {n: src.get(n, sh, "cpu") for n, (sh, _) in weight_shapes(cfg).items()}
    d = DictSource(expanded)
    d.fp8_scale_rule = rule
    b = build_model_weights(cfg, d, "cpu")
    assert torch.equal(a.layers[0].w_qb.w.view(torch.uint8), b.layers[0].w_qb.w.view(torch.uint8))
    assert torch.equal(a.layers[1].experts.w13, b.layers[1].experts.w13)
    wa, _ = a.layers[0].experts.dequant()
    e0 = torch.cat([src.get(f"layers.0.ffn.experts.0.w{i}.weight", weight_shapes(cfg)[f"layers.0.ffn.experts.0.w{i}.weight"][0], "cpu")
                    for i in (1, 3)], 0)
    assert torch.allclose(wa[0], e0, rtol=0, atol=0)                 # NVFP4 storage holds the checkpoint's values exactly


def test_shard_plan_covers_and_partitions():
    cfg = flash_config(2)
    shapes = weight_shapes(cfg)
    for tp in (1, 2, 4, 8):
        plans = [L.shard_plan(cfg, tp, r) for r in range(tp)]
        for name, (shape, kind) in shapes.items():
            sh = [p[name] for p in plans]
            if sh[0].dim is None and ".experts." not in name:
                assert all(s.dim is None for s in sh)
                continue
            if ".experts." in name:
                owners = [r for r, s in enumerate(sh) if s.dim is None]
                assert len(owners) == 1                                   # every expert lives on exactly one rank
                continue
            d = sh[0].dim
            spans = sorted((s.start, s.stop) for s in sh)
            assert spans[0][0] == 0 and spans[-1][1] == shape[d]
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0                                           # no gap, no overlap
            if kind == "dense" and name.endswith(("wo_b.weight", "w2.weight", "w1.weight", "w3.weight")):
                assert all(s.start % 128 == 0 for s in sh)               # fp8 block boundaries
        per_rank = [L.plan_bytes(cfg, tp, r) for r in range(tp)]
        assert max(per_rank) - min(per_rank) <= 0.02 * max(per_rank)
    # 48 layers fit 8 GPUs of 180 GB with room for the caches, but not one GPU
    full = flash_config(48)
    assert L.plan_bytes(full, 8, 0) < 40e9 and L.plan_bytes(full, 1, 0) > 150e9
    with pytest.raises(ValueError):
        L.shard_plan(cfg, 3, 0)


def test_damaged_shards_fail_as_value_errors_that_name_the_file(tmp_path):
    """Truncated files, flipped header bytes, absurd header lengths and malformed tensor entries: a ValueError at index
    time (or when the tensor is read), never another exception from deep inside a view."""
    import json
    import random
    import struct
    from stkernel_b200.models.loader import SafetensorsIndex, write_safetensors
    good = tmp_path / "good"
    good.mkdir()
    write_safetensors(str(good / "model-00001-of-00001.safetensors"),
                      {"a": torch.randn(4, 8), "b": torch.arange(10, dtype=torch.int32)})
    raw = (good / "model-00001-of-00001.safetensors").read_bytes()
    assert set(SafetensorsIndex(str(good)).keys()) == {"a", "b"}
    rng = random.Random(0)
    bad = tmp_path / "bad"
    bad.mkdir()
    refused = 0
    for _ in range(300):
        b = bytearray(raw)
        op = rng.choice(["trunc", "flip", "hdrlen", "json"])
        if op == "trunc":
            b = b[:rng.randrange(len(b))]
        elif op == "flip":
            for _ in range(rng.randint(1, 5)):
                b[rng.randrange(min(len(b), 200))] = rng.randrange(256)
        elif op == "hdrlen":
            b[:8] = struct.pack("<Q", rng.choice([0, 1, 7, 10 ** 6, 2 ** 63, len(b)]))
        else:
            n = struct.unpack("<Q", bytes(b[:8]))[0]
            hdr = json.loads(bytes(b[8:8 + n]))
            hdr[rng.choice(list(hdr))] = rng.choice([None, 1, {"dtype": "F32"},
                                                     {"dtype": "XX", "shape": [1], "data_offsets": [0, 4]},
                                                     {"dtype": "F32", "shape": [4, 8], "data_offsets": [0, 10 ** 9]},
                                                     {"dtype": "F32", "shape": [-1], "data_offsets": [4, 0]}])
            h = json.dumps(hdr).encode()
            b = bytearray(struct.pack("<Q", len(h)) + h + bytes(b[8 + n:]))
        (bad / "model-00001-of-00001.safetensors").write_bytes(bytes(b))
        try:
            idx = SafetensorsIndex(str(bad))
            for name in list(idx.keys()):
                idx.get(name)
        except (ValueError, KeyError):
            refused += 1
    assert refused > 200
