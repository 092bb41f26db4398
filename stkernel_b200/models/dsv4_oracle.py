"""Naive fp32 DeepSeek-V4-style decoder: the correctness oracle.

Whole-sequence, cache-free, one sequence at a time; every position recomputes
its own row sets.  It states the model semantics (layer order of
overlay/nvidia_model.py:1509-1572,1713-1841; attention data flow of
overlay/attention.py:541-670) with none of the engine's machinery, so the paged,
batched, kernel-backed engine can be checked against it.

When the config asks for quantised storage the oracle applies the same
quantise->dequantise round trips (fp8 block weights and per-token-group
activations, NVFP4/MXFP4 experts, fp8_ds_mla KV rows, fp8 indexer operands) so
that a GPU run can be compared within tensor-core accumulation error.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config import ModelConfig
from ..ops import reference as R
from .weights import compressor_slots, stacked_expert_weights

F32 = torch.float32


def index_cache_computes(cfg: ModelConfig, layer: int) -> bool:
    """True when `layer` (a C4A layer) runs its own indexer (F-layer); False when it
    reuses the most recent F-layer's top-k (S-layer).  The first C4A layer always
    computes (overlay/attention.py:179-205)."""
    if cfg.layer_kind(layer) != "c4a":
        return False
    if not cfg.use_index_cache:
        return True
    ordinal = sum(1 for i in range(layer) if cfg.layer_kind(i) == "c4a")
    return ordinal % cfg.index_topk_freq == 0


class OracleModel:
    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.w = weights
        self._deq: Dict[str, torch.Tensor] = {}

    # ---- weight access with storage-format round trips ----------------
    def dense_w(self, name: str) -> torch.Tensor:
        if name not in self._deq:
            w = self.w[name].to(F32)
            if self.cfg.dense_dtype == "fp8":
                w = R.dequant_fp8_block128_weight(*R.quant_fp8_block128_weight(w))
            else:
                w = w.to(torch.bfloat16).to(F32) if self.cfg.dense_dtype == "bf16" else w
            self._deq[name] = w
        return self._deq[name]

    def bf16_w(self, name: str) -> torch.Tensor:
        if name not in self._deq:
            self._deq[name] = self.w[name].to(torch.bfloat16).to(F32)
        return self._deq[name]

    def expert_w(self, name: str) -> torch.Tensor:
        if name not in self._deq:
            w = self.w[name].to(F32)
            if self.cfg.expert_dtype == "nvfp4":
                w = R.dequant_nvfp4(*R.quant_nvfp4(w))
            elif self.cfg.expert_dtype == "mxfp4":
                w = R.dequant_mxfp4(*R.quant_mxfp4(w))
            else:
                w = w.to(torch.bfloat16).to(F32)
            self._deq[name] = w
        return self._deq[name]

    def dense_linear(self, x: torch.Tensor, name: str) -> torch.Tensor:
        if self.cfg.dense_dtype == "fp8":
            x = R.dequant_fp8_group128_act(*R.quant_fp8_group128_act(x))
        return x.to(F32) @ self.dense_w(name).t()

    def kvq(self, rows: torch.Tensor) -> torch.Tensor:
        if self.cfg.kv_cache_dtype == "fp8_ds_mla":
            return R.kv_fake_quant(rows, self.cfg.qk_rope_head_dim)
        return rows.to(torch.bfloat16).to(F32)

    # ---- sub-blocks ------------------------------------------------------
    def _compress(self, y: torch.Tensor, prefix: str, ratio: int, out_dim: int, positions: torch.Tensor
                  ) -> torch.Tensor:
        """Compressed rows [S//ratio, out_dim] (normed + roped, unquantised)."""
        cfg = self.cfg
        c = 2 if prefix.endswith("indexer.compressor") else compressor_slots(ratio)
        s = y.shape[0]
        n = s // ratio
        if n == 0:
            return torch.zeros(0, out_dim, dtype=F32)
        kv = (y @ self.bf16_w(f"{prefix}.wkv.weight").t())[: n * ratio].view(n * ratio, c, out_dim)
        sc = (y @ self.bf16_w(f"{prefix}.wgate.weight").t())[: n * ratio].view(n * ratio, c, out_dim)
        ape = self.w[f"{prefix}.ape"].to(F32).view(ratio, c, out_dim)
        pooled = R.compressor_pool(kv, sc, ape, ratio, overlap=(c == 2))
        pooled = R.rms_norm(pooled, self.bf16_w(f"{prefix}.norm.weight"), cfg.rms_norm_eps)
        rd = cfg.qk_rope_head_dim
        cpos = torch.arange(n, dtype=torch.int64) * ratio
        cos, sin = R.rope_cos_sin(cpos, rd, cfg.rope_theta)
        pooled = pooled.clone()
        pooled[:, out_dim - rd:] = R.apply_rope_interleaved(pooled[:, out_dim - rd:], cos, sin)
        return pooled

    def _attention(self, li: int, prefix: str, y: torch.Tensor, positions: torch.Tensor,
                   shared_topk: Dict[str, torch.Tensor], kind: str, causal: bool = True) -> torch.Tensor:
        cfg = self.cfg
        s = y.shape[0]
        D, Rd, nh = cfg.head_dim, cfg.qk_rope_head_dim, cfg.num_attention_heads
        a = f"{prefix}.attn"
        qr = R.rms_norm(self.dense_linear(y, f"{a}.wq_a.weight"), self.bf16_w(f"{a}.q_norm.weight"), cfg.rms_norm_eps)
        kv = R.rms_norm(self.dense_linear(y, f"{a}.wkv.weight"), self.bf16_w(f"{a}.kv_norm.weight"), cfg.rms_norm_eps)
        q = self.dense_linear(qr, f"{a}.wq_b.weight").view(s, nh, D)
        q = R.rms_norm(q, None, cfg.rms_norm_eps)
        cos, sin = R.rope_cos_sin(positions, Rd, cfg.rope_theta)
        q = torch.cat([q[..., :D - Rd], R.apply_rope_interleaved(q[..., D - Rd:], cos, sin)], -1)
        kv = torch.cat([kv[:, :D - Rd], R.apply_rope_interleaved(kv[:, D - Rd:], cos, sin)], -1)
        swa_rows = self.kvq(kv)

        ratio = cfg.compress_ratio(li) if kind != "swa" else 0
        comp_rows = None
        topk = None
        if ratio:
            comp_rows = self.kvq(self._compress(y, f"{a}.compressor", ratio, D, positions))
            n_valid = (positions + 1) // ratio
            if kind == "c4a":
                if index_cache_computes(cfg, li):
                    i = f"{a}.indexer"
                    di, ih = cfg.index_head_dim, cfg.index_n_heads
                    qi = self.dense_linear(qr, f"{i}.wq_b.weight").view(s, ih, di)
                    wi = y @ self.bf16_w(f"{i}.weights_proj.weight").t()
                    quant = cfg.kv_cache_dtype == "fp8_ds_mla"
                    ki = self._compress(y, f"{i}.compressor", ratio, di, positions)
                    if cfg.indexer_dtype == "mxfp4":
                        qp, qs, wf = R.indexer_q_prepare_mxfp4(qi, wi, cos, sin, Rd)
                        kd = R.dequant_mxfp4(*R.quant_mxfp4(ki.to(F32)))
                        scores = R.indexer_scores(R.dequant_mxfp4(qp, qs), wf, kd, None)
                    else:
                        qq, wf = R.indexer_q_prepare(qi, wi, cos, sin, Rd, quantize=quant)
                        if quant:
                            kq, ks = R.indexer_k_quant(ki)
                            scores = R.indexer_scores(qq, wf, kq.to(F32), ks)
                        else:
                            scores = R.indexer_scores(qq, wf, ki.to(torch.bfloat16).to(F32), None)
                    topk = R.topk_rows(scores, n_valid, cfg.index_topk)
                    shared_topk["topk"] = topk
                else:
                    topk = shared_topk["topk"]
            else:  # c128a: every complete window, most recent index_topk of them
                topk = torch.full((s, cfg.index_topk), -1, dtype=torch.int32)
                for t in range(s):
                    nv = int(n_valid[t])
                    lo = max(0, nv - cfg.index_topk)
                    topk[t, : nv - lo] = torch.arange(lo, nv, dtype=torch.int32)

        W = cfg.sliding_window
        out = torch.zeros(s, nh, D, dtype=F32)
        sink = self.w[f"{a}.attn_sink"].to(F32)
        for t in range(s):
            p = int(positions[t])
            if causal:
                lo = max(0, t - W + 1)
                rows = [swa_rows[lo:t + 1]]
            else:
                rows = [swa_rows]
            if topk is not None:
                idx = topk[t]
                idx = idx[idx >= 0].long()
                if idx.numel():
                    rows.append(comp_rows[idx])
            rr = torch.cat(rows, 0)[None]
            valid = torch.ones(1, rr.shape[1], dtype=torch.bool)
            out[t] = R.sparse_mla(q[t:t + 1], rr, valid, sink, D ** -0.5)[0]
        # inverse rope on the rope dims of the output, grouped low-rank o-proj
        o = torch.cat([out[..., :D - Rd], R.apply_rope_interleaved(out[..., D - Rd:], cos, sin, inverse=True)], -1)
        G = cfg.o_groups
        og = o.reshape(s, G, (nh // G) * D)
        if cfg.dense_dtype == "fp8":
            og = R.dequant_fp8_group128_act(*R.quant_fp8_group128_act(og.reshape(s * G, -1))).view(s, G, -1)
        woa = self.dense_w(f"{a}.wo_a.weight").view(G, cfg.o_lora_rank, (nh // G) * D)
        z = torch.einsum("tgi,gri->tgr", og, woa).reshape(s, G * cfg.o_lora_rank)
        return self.dense_linear(z, f"{a}.wo_b.weight")

    def _moe(self, prefix: str, li: int, y: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        f = f"{prefix}.ffn"
        logits = y.to(torch.bfloat16).to(F32) @ self.bf16_w(f"{f}.gate.weight").t()
        hash_ids = None
        bias = None
        if f"{f}.gate.tid2eid" in self.w:
            hash_ids = self.w[f"{f}.gate.tid2eid"][token_ids.long()]
        else:
            bias = self.w[f"{f}.gate.bias"]
        ids, wts = R.route(logits, bias, cfg.num_experts_per_tok, cfg.scoring_func, cfg.norm_topk_prob,
                           cfg.routed_scaling_factor, hash_ids)
        key = f"{f}.__stacked"
        if key not in self._deq:
            E = cfg.n_routed_experts
            def q(t):
                if cfg.expert_dtype == "nvfp4":
                    return R.dequant_nvfp4(*R.quant_nvfp4(t))
                if cfg.expert_dtype == "mxfp4":
                    return R.dequant_nvfp4(*R.mxfp4_to_nvfp4(*R.quant_mxfp4(t)))
                return t.to(torch.bfloat16).to(F32)
            # gate and up rows are stored as one [2I, H] matrix with one global scale
            w13 = torch.stack([q(torch.cat([self.w[f"{f}.experts.{e}.w1.weight"].to(F32),
                                            self.w[f"{f}.experts.{e}.w3.weight"].to(F32)], 0)) for e in range(E)])
            w2 = torch.stack([q(self.w[f"{f}.experts.{e}.w2.weight"].to(F32)) for e in range(E)])
            self._deq[key] = (w13, w2)
        w13, w2 = self._deq[key]
        out = R.moe_experts(y, ids, wts, w13, w2, cfg.swiglu_limit)
        if cfg.n_shared_experts:
            g = self.dense_linear(y, f"{f}.shared_experts.w1.weight")
            u = self.dense_linear(y, f"{f}.shared_experts.w3.weight")
            out = out + self.dense_linear(R.swiglu_clamp(g, u, cfg.swiglu_limit), f"{f}.shared_experts.w2.weight")
        return out

    def _layer(self, li: int, prefix: str, X: torch.Tensor, positions: torch.Tensor, token_ids: torch.Tensor,
               shared_topk: Dict[str, torch.Tensor], kind: str, causal: bool = True) -> torch.Tensor:
        cfg = self.cfg
        w = self.w
        y, post, comb = R.mhc_pre(X, w[f"{prefix}.hc_attn_fn"], w[f"{prefix}.hc_attn_base"], w[f"{prefix}.hc_attn_scale"],
                                  self.bf16_w(f"{prefix}.attn_norm.weight"), cfg.rms_norm_eps, cfg.hc_eps,
                                  cfg.hc_sinkhorn_iters, round_bf16=True)
        a = self._attention(li, prefix, y, positions, shared_topk, kind, causal)
        X = R.mhc_post(a, X, post, comb)
        y, post, comb = R.mhc_pre(X, w[f"{prefix}.hc_ffn_fn"], w[f"{prefix}.hc_ffn_base"], w[f"{prefix}.hc_ffn_scale"],
                                  self.bf16_w(f"{prefix}.ffn_norm.weight"), cfg.rms_norm_eps, cfg.hc_eps,
                                  cfg.hc_sinkhorn_iters, round_bf16=True)
        f = self._moe(prefix, li, y, token_ids)
        return R.mhc_post(f, X, post, comb)

    # ---- public ------------------------------------------------------------
    def hidden_states(self, token_ids: torch.Tensor, aux_layers: Tuple[int, ...] = ()
                      ) -> Tuple[torch.Tensor, List[torch.Tensor]]:
        """token_ids [S] -> (final residual streams [S, hc, H], aux hidden states of `aux_layers`)."""
        cfg = self.cfg
        s = token_ids.shape[0]
        positions = torch.arange(s, dtype=torch.int64)
        x = self.bf16_w("embed.weight")[token_ids.long()]
        X = x[:, None, :].repeat(1, cfg.hc_mult, 1)
        shared: Dict[str, torch.Tensor] = {}
        aux: List[torch.Tensor] = []
        for li in range(cfg.num_hidden_layers):
            X = self._layer(li, f"layers.{li}", X, positions, token_ids, shared, cfg.layer_kind(li))
            if li in aux_layers:
                aux.append(X.mean(1))
        return X, aux

    def logits(self, token_ids: torch.Tensor) -> torch.Tensor:
        """token_ids [S] -> logits [S, V] for every position."""
        cfg = self.cfg
        X, _ = self.hidden_states(token_ids)
        h = R.hc_head(X, self.w["hc_head_fn"], self.w["hc_head_base"], self.w["hc_head_scale"],
                      cfg.rms_norm_eps, cfg.hc_eps)
        h = R.rms_norm(h, self.bf16_w("norm.weight"), cfg.rms_norm_eps)
        return h @ self.bf16_w("head.weight").t()

    def greedy_decode(self, prompt: torch.Tensor, steps: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """-> (generated ids [steps], logits used for each generated id [steps, V])."""
        ids = prompt.clone()
        outs, lgs = [], []
        for _ in range(steps):
            lg = self.logits(ids)[-1]
            nxt = int(lg.argmax())
            outs.append(nxt)
            lgs.append(lg)
            ids = torch.cat([ids, torch.tensor([nxt], dtype=ids.dtype)])
        return torch.tensor(outs), torch.stack(lgs)
