"""Row-wise FP8 draft head (experiment, off by default).

One e4m3 scale per vocabulary row for the weights and one dynamic scale per token for the activations:
``logits[t, v] = (a_q[t] . w_q[v]) * a_scale[t] * w_scale[v]``.  The reference measured this variant and
rejected it in favour of the block-scaled head (overlay/fp8_draft_head.py:59-112); it is kept here behind
`FP8HEAD=1` for the same A/B.  The production path is the 128x128 block-scaled fp8 head on the tcgen05 GEMM
(`build_model_weights(head_fp8=True)`); exactly one of the two may be armed (`pick_head_impl`).
On a GPU the contraction is a plain library fp8 GEMM (`torch._scaled_mm`), which is what a row-scaled
epilogue needs and nothing more; on CPU it is the fp32 statement of the same arithmetic.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

FP8_MAX = 448.0


@dataclass
class Fp8DraftHead:
    weight_fp8: torch.Tensor      # [V_local, H] e4m3
    row_scale: torch.Tensor       # [1, V_local]
    unit_scale: torch.Tensor      # [1] fp32 (the GEMM itself runs unscaled)


def quantize_draft_head(weight: torch.Tensor) -> Fp8DraftHead:
    if weight.ndim != 2:
        raise ValueError(f"draft lm_head weight must be two-dimensional, got shape={tuple(weight.shape)}")
    w = weight.detach()
    row_max = w.abs().amax(dim=1, keepdim=True).float().clamp(min=1e-6)
    q = (w.float() * (FP8_MAX / row_max)).to(torch.float8_e4m3fn)
    return Fp8DraftHead(q, (row_max / FP8_MAX).to(w.dtype).reshape(1, -1), torch.ones(1, dtype=torch.float32, device=w.device))


def fp8_draft_head_logits(hidden: torch.Tensor, head: Fp8DraftHead) -> torch.Tensor:
    if hidden.shape[-1] != head.weight_fp8.shape[-1]:
        raise ValueError(f"draft hidden/head dimension mismatch: hidden={hidden.shape[-1]}, head={head.weight_fp8.shape[-1]}")
    act_max = hidden.abs().amax(dim=-1, keepdim=True).clamp(min=1e-6)
    act_q = (hidden * (FP8_MAX / act_max)).to(torch.float8_e4m3fn)
    if hidden.is_cuda and hasattr(torch, "_scaled_mm") and hidden.shape[0] % 16 == 0 and hidden.shape[-1] % 16 == 0:
        logits = torch._scaled_mm(act_q, head.weight_fp8.t(), scale_a=head.unit_scale, scale_b=head.unit_scale,
                                  out_dtype=hidden.dtype)
    else:
        logits = (act_q.float() @ head.weight_fp8.float().t()).to(hidden.dtype)
    return logits * head.row_scale * (act_max / FP8_MAX).to(hidden.dtype)


def pick_head_impl(fp8_draft_head: bool, fp8_lm_head: bool) -> str:
    """Exactly one fp8 draft-head implementation may be armed; both at once is a configuration error."""
    if fp8_draft_head and fp8_lm_head:
        raise ValueError("row-wise FP8 draft head and block-scaled FP8 lm_head copy must not be armed together")
    return "rowwise" if fp8_draft_head else "block" if fp8_lm_head else "bf16"
