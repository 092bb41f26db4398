"""MoE ops: router, pair alignment, NVFP4 expert MLP (weight-streaming path), combine."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib
from . import reference as R
from .scratch import scratch
from .functional import cpu_act_dtype

BF16 = torch.bfloat16
F32 = torch.float32
I32 = torch.int32
DIRECT_MAX_PAIRS = 48
# tcgen05 grouped GEMM for batches beyond a handful of pairs (False: weight-streaming kernels, for A/B checks)
USE_GROUPED_GEMM = True


@dataclass
class ExpertWeights:
    """Local experts of one layer.

    NVFP4: w13 [E, 2I, H/2] uint8, s13 [E, 2I, H/16] e4m3 bytes, g13 [E] fp32; w2 [E, H, I/2], s2 [E, H, I/16], g2 [E].
    bf16 (debug dtype): w13 [E, 2I, H], w2 [E, H, I] with the scale fields None."""
    w13: torch.Tensor
    w2: torch.Tensor
    s13: Optional[torch.Tensor] = None
    s2: Optional[torch.Tensor] = None
    g13: Optional[torch.Tensor] = None
    g2: Optional[torch.Tensor] = None
    expert_start: int = 0

    @property
    def is_fp4(self) -> bool:
        return self.s13 is not None

    @property
    def num_local(self) -> int:
        return self.w13.shape[0]

    @staticmethod
    def from_master(w13: torch.Tensor, w2: torch.Tensor, expert_dtype: str, device, expert_start: int = 0
                    ) -> "ExpertWeights":
        """w13 [E, 2I, H], w2 [E, H, I] fp32 master -> storage format (one global scale per expert matrix)."""
        if expert_dtype == "bf16":
            return ExpertWeights(w13.to(device=device, dtype=BF16), w2.to(device=device, dtype=BF16),
                                 expert_start=expert_start)
        p13, s13, g13, p2, s2, g2 = [], [], [], [], [], []
        for e in range(w13.shape[0]):
            if expert_dtype == "mxfp4":
                a, b, c = R.mxfp4_to_nvfp4(*R.quant_mxfp4(w13[e].to(device)))
                d, f, g = R.mxfp4_to_nvfp4(*R.quant_mxfp4(w2[e].to(device)))
            else:
                a, b, c = R.quant_nvfp4(w13[e].to(device))
                d, f, g = R.quant_nvfp4(w2[e].to(device))
            p13.append(a); s13.append(b.view(torch.uint8)); g13.append(c)
            p2.append(d); s2.append(f.view(torch.uint8)); g2.append(g)
        return ExpertWeights(torch.stack(p13), torch.stack(p2), torch.stack(s13), torch.stack(s2),
                             torch.stack(g13).to(F32), torch.stack(g2).to(F32), expert_start)

    def dequant(self) -> Tuple[torch.Tensor, torch.Tensor]:
        if not self.is_fp4:
            return self.w13.to(F32), self.w2.to(F32)
        f8 = torch.float8_e4m3fn
        w13 = torch.stack([R.dequant_nvfp4(self.w13[e], self.s13[e].view(f8), self.g13[e]) for e in range(self.num_local)])
        w2 = torch.stack([R.dequant_nvfp4(self.w2[e], self.s2[e].view(f8), self.g2[e]) for e in range(self.num_local)])
        return w13, w2


def router(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, scoring: str, renorm: bool, scaling: float,
           tid2eid: Optional[torch.Tensor] = None, token_ids: Optional[torch.Tensor] = None
           ) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 gate logits [T, E] -> (expert ids i32 [T, k], weights f32 [T, k])."""
    t, e = logits.shape
    if not logits.is_cuda:
        hash_ids = tid2eid[token_ids.long()] if tid2eid is not None else None
        return R.route(logits, bias, top_k, scoring, renorm, scaling, hash_ids)
    ids = torch.empty(t, top_k, dtype=I32, device=logits.device)
    w = torch.empty(t, top_k, dtype=F32, device=logits.device)
    vocab = tid2eid.shape[0] if tid2eid is not None else 0
    _lib.call("stk_router", logits, logits.stride(0), bias, tid2eid, token_ids, vocab, ids, w, t, e, top_k,
              0 if scoring == "sigmoid" else 1, 1 if renorm else 0, float(scaling), _lib.status_buffer(), _lib.stream())
    return ids, w


def moe_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, ew: ExpertWeights, limit: float,
                shared: Optional[torch.Tensor] = None, total_experts: int = 0, shared_ready=None, ll=None):
    """x [T, H] bf16 -> sum_k w_k * expert_k(x) (+ shared) as bf16 [T, H]; experts that are not local add nothing.
    shared_ready: CUDA event after which `shared` (computed on another stream) may be read.
    ll: an `LLExchange`; this rank's sum is pushed into the folded all-reduce by the combine kernel and an
    `LLPending` is returned (GPU, NVFP4 experts only)."""
    t, h = x.shape
    k = ids.shape[1]
    if not x.is_cuda or not ew.is_fp4:
        w13, w2 = ew.dequant()
        out = R.moe_experts(x.to(cpu_act_dtype()), ids, weights, w13, w2, limit, ew.expert_start)
        if shared is not None:
            out = out + shared.to(F32)
        return out.to(cpu_act_dtype())
    dev = x.device
    n_pairs = t * k
    inter = ew.w2.shape[2] * 2
    st = _lib.stream()
    act = scratch("moe.act", (n_pairs, inter), torch.float16, dev)
    y = scratch("moe.y", (n_pairs, h), BF16, dev)
    if n_pairs <= DIRECT_MAX_PAIRS:
        # a handful of pairs: skip the sort, row = pair index
        pair_row = None
        _lib.call("stk_moe_expert_fc1", x, x.stride(0), ew.w13, ew.s13, ew.g13, None, None, None, ew.num_local, k, act,
                  n_pairs, h, inter, float(limit), ids, ew.expert_start, st)
        _lib.call("stk_moe_expert_fc2", act, ew.w2, ew.s2, ew.g2, None, None, ew.num_local, y, n_pairs, h, inter, ids,
                  ew.expert_start, st)
    else:
        sorted_p = scratch("moe.sorted", (n_pairs,), I32, dev)
        pair_row = scratch("moe.pair_row", (n_pairs,), I32, dev)
        offsets = scratch("moe.offsets", (ew.num_local + 1,), I32, dev)
        sorted_e = scratch("moe.sorted_e", (n_pairs,), I32, dev)
        counts = scratch("moe.counts", (((n_pairs + 255) // 256) * ew.num_local,), I32, dev) if n_pairs > 2048 else None
        _lib.call("stk_moe_align", ids, n_pairs, ew.expert_start, ew.num_local, sorted_p, pair_row, offsets, sorted_e,
                  counts, st)
        if USE_GROUPED_GEMM and h % 64 == 0 and inter % 128 == 0 and h % 128 == 0:
            # tensor-core path: permute the activations into expert order, then two grouped GEMMs
            avg = max(1, n_pairs // max(1, total_experts or ew.num_local))
            bt = 16 if avg <= 8 else 32 if avg <= 24 else 64 if avg <= 48 else 128
            xs = scratch("moe.xs", (n_pairs + 128, h), torch.float16, dev, zero=True)
            act_p = scratch("moe.act_p", (n_pairs + 128, inter), torch.float16, dev, zero=True)
            _lib.call("stk_moe_permute", x, x.stride(0), sorted_p, offsets, ew.num_local, k, xs, n_pairs, h, st)
            _lib.call("stk_moe_grouped", xs, n_pairs + 128, ew.w13, ew.s13, ew.g13, offsets, ew.num_local, inter, h, act_p, 1,
                      float(limit), bt, _lib.status_buffer(), _lib.sm_count(), st)
            _lib.call("stk_moe_grouped", act_p, n_pairs + 128, ew.w2, ew.s2, ew.g2, offsets, ew.num_local, h, inter, y, 0,
                      0.0, bt, _lib.status_buffer(), _lib.sm_count(), st)
        else:
            _lib.call("stk_moe_expert_fc1", x, x.stride(0), ew.w13, ew.s13, ew.g13, sorted_p, sorted_e, offsets,
                      ew.num_local, k, act, n_pairs, h, inter, float(limit), None, 0, st)
            _lib.call("stk_moe_expert_fc2", act, ew.w2, ew.s2, ew.g2, sorted_e, offsets, ew.num_local, y, n_pairs, h,
                      inter, None, 0, st)
    if shared_ready is not None:
        torch.cuda.current_stream().wait_event(shared_ready)
    if ll is not None:
        from .functional import LLPending
        _lib.call("stk_moe_combine", y, weights, pair_row, shared, None, t, h, k, ll.ctx, st)
        return LLPending(ll, t, h, dev)
    out = torch.empty(t, h, dtype=BF16, device=dev)
    _lib.call("stk_moe_combine", y, weights, pair_row, shared, out, t, h, k, None, st)
    return out
