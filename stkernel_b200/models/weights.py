"""Weight naming (DeepSeek-V4 checkpoint layout) and random initialisation.

Tensors are keyed by their *checkpoint* names: ``embed.weight``, ``head.weight``,
``norm.weight``, ``hc_head_fn|base|scale``, ``layers.N.attn.{wq_a,wkv,wq_b,wo_a,wo_b}.weight``,
``layers.N.attn.{q_norm,kv_norm}.weight``, ``layers.N.attn.attn_sink``,
``layers.N.attn.compressor.{wkv,wgate}.weight|ape|norm.weight``,
``layers.N.attn.indexer.{wq_b,weights_proj}.weight``, ``layers.N.attn.indexer.compressor.*``,
``layers.N.{attn_norm,ffn_norm}.weight``, ``layers.N.hc_{attn,ffn}_{fn,base,scale}``,
``layers.N.ffn.gate.{weight,bias,tid2eid}``, ``layers.N.ffn.experts.E.w{1,2,3}.weight``,
``layers.N.ffn.shared_experts.w{1,2,3}.weight``, and ``mtp.K.*`` for draft layers
(name map of overlay/nvidia_model.py:1843-1953,2002-2036 and overlay/dspark_v2.py:616-764).
Quantised tensors carry a sibling ``.scale`` entry.
"""
from __future__ import annotations

from typing import Dict, Iterator, List, Tuple

import torch

from ..config import ModelConfig


def compressor_slots(ratio: int) -> int:
    """Ratio-4 compressors pool overlapped windows (two value/gate slots per token)."""
    return 2 if ratio == 4 else 1


def weight_shapes(cfg: ModelConfig, include_mtp: bool = True) -> Dict[str, Tuple[Tuple[int, ...], str]]:
    """name -> (shape, kind); kind in {dense, expert, fp32, bf16, int} decides dtype/quantisation."""
    H, D, R = cfg.hidden_size, cfg.head_dim, cfg.qk_rope_head_dim
    nh, hc = cfg.num_attention_heads, cfg.hc_mult
    out: Dict[str, Tuple[Tuple[int, ...], str]] = {}
    out["embed.weight"] = ((cfg.vocab_size, H), "bf16")
    out["head.weight"] = ((cfg.vocab_size, H), "bf16")
    out["norm.weight"] = ((H,), "bf16")
    out["hc_head_fn"] = ((hc, hc * H), "fp32")
    out["hc_head_base"] = ((hc,), "fp32")
    out["hc_head_scale"] = ((1,), "fp32")

    def layer(prefix: str, li: int) -> None:
        p = prefix
        out[f"{p}.attn_norm.weight"] = ((H,), "bf16")
        out[f"{p}.ffn_norm.weight"] = ((H,), "bf16")
        for blk in ("attn", "ffn"):
            out[f"{p}.hc_{blk}_fn"] = ((cfg.mix_hc, hc * H), "fp32")
            out[f"{p}.hc_{blk}_base"] = ((cfg.mix_hc,), "fp32")
            out[f"{p}.hc_{blk}_scale"] = ((3,), "fp32")
        a = f"{p}.attn"
        out[f"{a}.wq_a.weight"] = ((cfg.q_lora_rank, H), "dense")
        out[f"{a}.wkv.weight"] = ((D, H), "dense")
        out[f"{a}.q_norm.weight"] = ((cfg.q_lora_rank,), "bf16")
        out[f"{a}.kv_norm.weight"] = ((D,), "bf16")
        out[f"{a}.wq_b.weight"] = ((nh * D, cfg.q_lora_rank), "dense")
        out[f"{a}.wo_a.weight"] = ((cfg.o_groups * cfg.o_lora_rank, (nh // cfg.o_groups) * D), "dense")
        out[f"{a}.wo_b.weight"] = ((H, cfg.o_groups * cfg.o_lora_rank), "dense")
        out[f"{a}.attn_sink"] = ((nh,), "fp32")
        ratio = cfg.compress_ratio(li) if li < cfg.num_hidden_layers else 0
        if ratio:
            c = compressor_slots(ratio)
            out[f"{a}.compressor.wkv.weight"] = ((c * D, H), "bf16")
            out[f"{a}.compressor.wgate.weight"] = ((c * D, H), "bf16")
            out[f"{a}.compressor.ape"] = ((ratio, c * D), "fp32")
            out[f"{a}.compressor.norm.weight"] = ((D,), "bf16")
        if ratio == 4:
            di = cfg.index_head_dim
            out[f"{a}.indexer.wq_b.weight"] = ((cfg.index_n_heads * di, cfg.q_lora_rank), "dense")
            out[f"{a}.indexer.weights_proj.weight"] = ((cfg.index_n_heads, H), "bf16")
            out[f"{a}.indexer.compressor.wkv.weight"] = ((2 * di, H), "bf16")
            out[f"{a}.indexer.compressor.wgate.weight"] = ((2 * di, H), "bf16")
            out[f"{a}.indexer.compressor.ape"] = ((ratio, 2 * di), "fp32")
            out[f"{a}.indexer.compressor.norm.weight"] = ((di,), "bf16")
        f = f"{p}.ffn"
        out[f"{f}.gate.weight"] = ((cfg.n_routed_experts, H), "bf16")
        if li < cfg.num_hash_layers:
            out[f"{f}.gate.tid2eid"] = ((cfg.vocab_size, cfg.num_experts_per_tok), "int")
        else:
            out[f"{f}.gate.bias"] = ((cfg.n_routed_experts,), "fp32")
        I = cfg.moe_intermediate_size
        for e in range(cfg.n_routed_experts):
            out[f"{f}.experts.{e}.w1.weight"] = ((I, H), "expert")
            out[f"{f}.experts.{e}.w3.weight"] = ((I, H), "expert")
            out[f"{f}.experts.{e}.w2.weight"] = ((H, I), "expert")
        if cfg.n_shared_experts:
            Is = I * cfg.n_shared_experts
            out[f"{f}.shared_experts.w1.weight"] = ((Is, H), "dense")
            out[f"{f}.shared_experts.w3.weight"] = ((Is, H), "dense")
            out[f"{f}.shared_experts.w2.weight"] = ((H, Is), "dense")

    for li in range(cfg.num_hidden_layers):
        layer(f"layers.{li}", li)
    if include_mtp and cfg.n_mtp_layers:
        n_aux = max(1, len(cfg.dspark_target_layer_ids))
        out["mtp.main_proj.weight"] = ((H, H * n_aux), "bf16")
        out["mtp.main_norm.weight"] = ((H,), "bf16")
        out["mtp.markov_w1.weight"] = ((cfg.vocab_size, cfg.dspark_markov_rank), "bf16")
        out["mtp.markov_w2.weight"] = ((cfg.vocab_size, cfg.dspark_markov_rank), "bf16")
        out["mtp.norm.weight"] = ((H,), "bf16")
        out["mtp.hc_head_fn"] = ((hc, hc * H), "fp32")
        out["mtp.hc_head_base"] = ((hc,), "fp32")
        out["mtp.hc_head_scale"] = ((1,), "fp32")
        for k in range(cfg.n_mtp_layers):
            layer(f"mtp.{k}", cfg.num_hidden_layers + k)     # draft layers are SWA-only
    return out


def init_random_weights(cfg: ModelConfig, seed: int = 0, device: str = "cpu", std: float = 0.02
                        ) -> Dict[str, torch.Tensor]:
    """fp32 master weights ~N(0, std); norms at 1, sinks at 0, hc scales at 1, router bias U[-0.1, 0.1]."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    w: Dict[str, torch.Tensor] = {}
    for name, (shape, kind) in weight_shapes(cfg).items():
        if kind == "int":
            t = torch.randint(0, cfg.n_routed_experts, shape, generator=g, dtype=torch.int32)
        elif name.endswith("norm.weight"):
            t = torch.ones(shape)
        elif name.endswith("_scale"):
            t = torch.ones(shape)
        elif name.endswith("_base"):
            t = torch.zeros(shape)
        elif name.endswith("attn_sink"):
            t = torch.zeros(shape)
        elif name.endswith("gate.bias"):
            t = torch.rand(shape, generator=g) * 0.2 - 0.1
        elif name.endswith("_fn"):
            t = torch.randn(shape, generator=g) * std
        elif name.endswith(".ape"):
            t = torch.randn(shape, generator=g) * std
        else:
            t = torch.randn(shape, generator=g) * std
        w[name] = t.to(device)
    return w


def stacked_expert_weights(w: Dict[str, torch.Tensor], prefix: str, n_experts: int
                           ) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (w13 [E, 2I, H] gate rows then up rows, w2 [E, H, I])."""
    w13 = torch.stack([torch.cat([w[f"{prefix}.experts.{e}.w1.weight"], w[f"{prefix}.experts.{e}.w3.weight"]], 0)
                       for e in range(n_experts)])
    w2 = torch.stack([w[f"{prefix}.experts.{e}.w2.weight"] for e in range(n_experts)])
    return w13, w2
