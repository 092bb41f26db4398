"""Plain PyTorch fp32 statements of every op in the engine.

These functions are (a) the numerics oracle that each sm_100a kernel is tested
against and (b) the CPU execution path of the engine (gloo ranks, unit tests).
They define the semantics that the reference only names but does not ship
(KV compressor pooling, hc_head, indexer activation, mhc_post index order):

* mHC pre: restates overlay/mhc_tilelang.py:206-325.
* mHC post: ``out[j] = post[j]*x + sum_k comb[j,k]*res[k]`` — the index order of
  the torch path in overlay/nvidia_model.py:1779-1785.
* fp8_ds_mla row quantisation: restates overlay/ops_cache_utils.py:97-152.
* indexer Q rope/quant/fold: restates overlay/ops_fused_indexer_q.py:93-172.
* indexer activation: ReLU (the published DSA indexer).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from ..config import FP8_BLOCK, FP8_MAX, KV_QUANT_BLOCK, KV_SCALE_BYTES, MXFP4_GROUP, NVFP4_GROUP

F32 = torch.float32

# ----------------------------------------------------------------------------
# number formats
# ----------------------------------------------------------------------------
_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def e2m1_table(device=None) -> torch.Tensor:
    pos = torch.tensor(_E2M1_VALUES, dtype=F32, device=device)
    return torch.cat([pos, -pos])          # code 0..7 positive, 8..15 negative


def round_to_e2m1_code(x: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 code (ties to even mantissa, saturating), as uint8 in [0, 15]."""
    a = x.abs().clamp(max=6.0)
    # thresholds between consecutive magnitudes; ties resolve to the even code
    code = torch.zeros_like(a, dtype=torch.uint8)
    bounds = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
    tie_up = (False, True, False, True, False, True, False)  # tie goes to even code
    for i, (b, up) in enumerate(zip(bounds, tie_up)):
        code = torch.where((a > b) | ((a == b) & up), torch.full_like(code, i + 1), code)
    sign = (x < 0) | ((x == 0) & torch.signbit(x))
    return code | (sign.to(torch.uint8) << 3)


def to_fp8_e4m3(x: torch.Tensor) -> torch.Tensor:
    """Saturating round-to-nearest-even cast to e4m3 (finite max 448)."""
    return x.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


def ue8m0_scale_from_amax(amax: torch.Tensor, floor: float = 1e-4) -> Tuple[torch.Tensor, torch.Tensor]:
    """Power-of-two scale 2^ceil(log2(max(amax, floor)/448)) and its biased exponent byte."""
    amax = amax.to(F32).clamp(min=floor)
    exponent = torch.ceil(torch.log2(amax / FP8_MAX))
    byte = (exponent + 127.0).clamp(0, 255).to(torch.uint8)
    return torch.exp2(exponent), byte


def quant_fp8_block128_weight(w: torch.Tensor, ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Weight [N, K] -> e4m3 [N, K] + fp32 scales [ceil(N/128), ceil(K/128)] (dequant = q*scale).
    ue8m0: scales rounded up to a power of two (the checkpoint's exponent-byte scale format)."""
    n, k = w.shape
    nb, kb = -(-n // FP8_BLOCK), -(-k // FP8_BLOCK)
    wp = torch.zeros(nb * FP8_BLOCK, kb * FP8_BLOCK, dtype=F32, device=w.device)
    wp[:n, :k] = w.to(F32)
    blocks = wp.view(nb, FP8_BLOCK, kb, FP8_BLOCK)
    amax = blocks.abs().amax(dim=(1, 3)).clamp(min=1e-12)
    scale = amax / FP8_MAX
    if ue8m0:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = to_fp8_e4m3(blocks / scale[:, None, :, None]).view(nb * FP8_BLOCK, kb * FP8_BLOCK)
    return q[:n, :k].contiguous(), scale.contiguous()


def dequant_fp8_block128_weight(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    n, k = q.shape
    s = scale.repeat_interleave(FP8_BLOCK, 0)[:n].repeat_interleave(FP8_BLOCK, 1)[:, :k]
    return q.to(F32) * s


def quant_fp8_group128_act(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Activation [T, K] -> e4m3 [T, K] + fp32 scale [T, ceil(K/128)] (per-token 1x128 groups)."""
    t, k = x.shape
    kb = -(-k // FP8_BLOCK)
    xp = torch.zeros(t, kb * FP8_BLOCK, dtype=F32, device=x.device)
    xp[:, :k] = x.to(F32)
    g = xp.view(t, kb, FP8_BLOCK)
    scale = g.abs().amax(-1).clamp(min=1e-10) / FP8_MAX
    q = to_fp8_e4m3(g / scale[..., None]).view(t, kb * FP8_BLOCK)[:, :k]
    return q.contiguous(), scale.contiguous()


def dequant_fp8_group128_act(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    k = q.shape[-1]
    return q.to(F32) * scale.repeat_interleave(FP8_BLOCK, -1)[..., :k]


def quant_nvfp4(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """NVFP4: [.., K] -> packed e2m1 [.., K/2] uint8 (low nibble = even index),
    e4m3 scales [.., K/16] (as float8 tensor), per-tensor fp32 global scale.

    dequant = e2m1 * fp32(scale_e4m3) * global_scale.
    """
    assert w.shape[-1] % NVFP4_GROUP == 0
    wf = w.to(F32)
    gmax = wf.abs().amax().clamp(min=1e-12)
    global_scale = gmax / (6.0 * FP8_MAX)
    g = wf.view(*wf.shape[:-1], -1, NVFP4_GROUP)
    amax = g.abs().amax(-1)
    s = to_fp8_e4m3(amax / 6.0 / global_scale)
    sf = s.to(F32) * global_scale
    sf_safe = torch.where(sf == 0, torch.ones_like(sf), sf)
    code = round_to_e2m1_code(g / sf_safe[..., None]).view(*wf.shape)
    packed = (code[..., 0::2] | (code[..., 1::2] << 4)).contiguous()
    return packed, s.contiguous(), global_scale.reshape(())


def dequant_nvfp4(packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor) -> torch.Tensor:
    tbl = e2m1_table(packed.device)
    lo = tbl[(packed & 0xF).long()]
    hi = tbl[(packed >> 4).long()]
    v = torch.stack([lo, hi], dim=-1).flatten(-2)
    sf = scales.to(F32).repeat_interleave(NVFP4_GROUP, -1) * global_scale.to(F32)
    return v * sf


def quant_mxfp4(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """MXFP4 checkpoint layout: packed e2m1 [.., K/2] + ue8m0 exponent bytes [.., K/32]."""
    assert w.shape[-1] % MXFP4_GROUP == 0
    g = w.to(F32).view(*w.shape[:-1], -1, MXFP4_GROUP)
    amax = g.abs().amax(-1).clamp(min=2.0 ** -120)
    exponent = torch.ceil(torch.log2(amax / 6.0))
    byte = (exponent + 127).clamp(0, 255).to(torch.uint8)
    code = round_to_e2m1_code(g / torch.exp2(exponent)[..., None]).view(*w.shape)
    packed = (code[..., 0::2] | (code[..., 1::2] << 4)).contiguous()
    return packed, byte.contiguous()


def dequant_mxfp4(packed: torch.Tensor, scale_bytes: torch.Tensor) -> torch.Tensor:
    tbl = e2m1_table(packed.device)
    v = torch.stack([tbl[(packed & 0xF).long()], tbl[(packed >> 4).long()]], dim=-1).flatten(-2)
    sf = torch.exp2(scale_bytes.to(F32) - 127.0).repeat_interleave(MXFP4_GROUP, -1)
    return v * sf


def mxfp4_to_nvfp4(packed: torch.Tensor, scale_bytes: torch.Tensor
                   ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Re-express an MXFP4 tensor as NVFP4 without touching the 4-bit codes.

    Power-of-two scales are exactly representable in e4m3 after one global
    shift, so each ue8m0 scale is duplicated to the two 16-element groups it
    covers.  Exponents that fall below the e4m3 range flush to the smallest
    subnormal (2^-9 relative to the global scale)."""
    e = scale_bytes.to(F32) - 127.0
    emax = e.amax()
    global_scale = torch.exp2(emax - 8.0)            # largest group scale -> 2^8 (<= 448)
    rel = torch.exp2((e - emax + 8.0).clamp(min=-9.0))
    s = rel.to(torch.float8_e4m3fn).repeat_interleave(MXFP4_GROUP // NVFP4_GROUP, -1)
    return packed, s.contiguous(), global_scale.reshape(())


# ----------------------------------------------------------------------------
# norms, rope, activations
# ----------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    xf = x.to(F32)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return y * w.to(F32) if w is not None else y


def rope_cos_sin(positions: torch.Tensor, rope_dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, rope_dim, 2, dtype=F32, device=positions.device) / rope_dim))
    ang = positions.to(F32)[:, None] * inv[None, :]
    return torch.cos(ang), torch.sin(ang)


def apply_rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """GPT-J style: pairs (x[2i], x[2i+1]) rotate by angle_i.  x [T, ..., R]; cos/sin [T, R/2]."""
    xf = x.to(F32)
    x0, x1 = xf[..., 0::2], xf[..., 1::2]
    shape = [cos.shape[0]] + [1] * (xf.dim() - 2) + [cos.shape[1]]
    c, s = cos.view(shape), sin.view(shape)
    if inverse:
        s = -s
    return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1).flatten(-2)


def swiglu_clamp(gate: torch.Tensor, up: torch.Tensor, limit: float) -> torch.Tensor:
    g = gate.to(F32)
    u = up.to(F32)
    if limit and limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(-limit, limit)
    return torch.nn.functional.silu(g) * u


# ----------------------------------------------------------------------------
# mHC (manifold hyper-connections)
# ----------------------------------------------------------------------------
def mhc_pre(residual: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor,
            norm_w: Optional[torch.Tensor], rms_eps: float, hc_eps: float, sinkhorn_iters: int,
            post_mult: float = 2.0, round_bf16: bool = False
            ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """residual [T, hc, H] -> (layer_input [T, H], post [T, hc], comb [T, hc, hc])."""
    t, hc, h = residual.shape
    x = residual.to(F32).reshape(t, hc * h)
    mixes = x @ fn.to(F32).t()
    rms = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + rms_eps)
    mixes = mixes * rms
    base = base.to(F32)
    scale = scale.to(F32)
    pre = torch.sigmoid(mixes[:, :hc] * scale[0] + base[:hc]) + hc_eps
    post = torch.sigmoid(mixes[:, hc:2 * hc] * scale[1] + base[hc:2 * hc]) * post_mult
    cm = mixes[:, 2 * hc:].reshape(t, hc, hc) * scale[2] + base[2 * hc:].reshape(hc, hc)
    cm = torch.softmax(cm, dim=-1) + hc_eps
    cm = cm / (cm.sum(1, keepdim=True) + hc_eps)
    for _ in range(sinkhorn_iters - 1):
        cm = cm / (cm.sum(2, keepdim=True) + hc_eps)
        cm = cm / (cm.sum(1, keepdim=True) + hc_eps)
    y = (pre[:, :, None] * residual.to(F32)).sum(1)
    if round_bf16:
        y = y.to(torch.bfloat16).to(F32)
    if norm_w is not None:
        y = rms_norm(y, norm_w, rms_eps)
    return y, post, cm


def mhc_post(x: torch.Tensor, residual: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """out[t, j] = post[t, j] * x[t] + sum_k comb[t, j, k] * residual[t, k]."""
    return post[:, :, None] * x.to(F32)[:, None, :] + torch.einsum("tjk,tkh->tjh", comb, residual.to(F32))


def hc_head(residual: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor,
            rms_eps: float, hc_eps: float) -> torch.Tensor:
    """Collapse hc streams: w = sigmoid(rms*(x_flat @ fn^T)*scale + base) + eps; out = sum_j w_j x_j."""
    t, hc, h = residual.shape
    x = residual.to(F32).reshape(t, hc * h)
    mixes = (x @ fn.to(F32).t()) * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + rms_eps)
    w = torch.sigmoid(mixes * scale.to(F32)[0] + base.to(F32)) + hc_eps
    return (w[:, :, None] * residual.to(F32)).sum(1)


# ----------------------------------------------------------------------------
# fp8_ds_mla KV rows
# ----------------------------------------------------------------------------
def kv_row_quant(kv: torch.Tensor, rope_dim: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """kv [T, D] -> (fp8 nope [T, D-R] float8, rope [T, R] bf16, scale bytes [T, 8] uint8)."""
    t, d = kv.shape
    nope = d - rope_dim
    nb = nope // KV_QUANT_BLOCK
    x = kv[:, :nope].to(F32).view(t, nb, KV_QUANT_BLOCK)
    scale, byte = ue8m0_scale_from_amax(x.abs().amax(-1))
    q = to_fp8_e4m3(x / scale[..., None]).view(t, nope)
    scales = torch.zeros(t, KV_SCALE_BYTES, dtype=torch.uint8, device=kv.device)
    scales[:, :nb] = byte
    return q, kv[:, nope:].to(torch.bfloat16), scales


def kv_row_dequant(q: torch.Tensor, rope: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    t, nope = q.shape
    nb = nope // KV_QUANT_BLOCK
    s = torch.exp2(scales[:, :nb].to(F32) - 127.0)
    x = (q.to(F32).view(t, nb, KV_QUANT_BLOCK) * s[..., None]).view(t, nope)
    return torch.cat([x, rope.to(F32)], dim=-1)


def kv_fake_quant(kv: torch.Tensor, rope_dim: int) -> torch.Tensor:
    """Quantise + dequantise a latent row the way the paged cache stores it."""
    return kv_row_dequant(*kv_row_quant(kv, rope_dim))


def indexer_k_quant(k: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Indexer K rows [S, d] -> e4m3 [S, d] + fp32 scale [S] (power of two, ue8m0-rounded)."""
    scale, _ = ue8m0_scale_from_amax(k.to(F32).abs().amax(-1))
    return to_fp8_e4m3(k.to(F32) / scale[:, None]), scale


# ----------------------------------------------------------------------------
# lightning indexer
# ----------------------------------------------------------------------------
def indexer_q_prepare(q: torch.Tensor, weights: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                      rope_dim: int, quantize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [T, ih, d] (pre-rope), weights [T, ih] -> (q values [T, ih, d], folded weights [T, ih]).

    RoPE (interleaved) on the last rope_dim dims, round to bf16, per-(token, head)
    ue8m0 fp8 quantisation; the scale, the softmax scale d^-0.5 and ih^-0.5 fold
    into the head weights."""
    t, ih, d = q.shape
    qf = q.to(F32).clone()
    qf[..., d - rope_dim:] = apply_rope_interleaved(qf[..., d - rope_dim:], cos, sin)
    qf = qf.to(torch.bfloat16).to(F32)
    fold = (d ** -0.5) * (ih ** -0.5)
    if not quantize:
        return qf, weights.to(F32) * fold
    scale, _ = ue8m0_scale_from_amax(qf.abs().amax(-1))
    qq = to_fp8_e4m3(qf / scale[..., None]).to(F32)
    return qq, weights.to(F32) * scale * fold


def indexer_q_prepare_mxfp4(q: torch.Tensor, weights: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                            rope_dim: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """q [T, ih, d] (pre-rope), weights [T, ih] -> (packed e2m1 [T, ih, d/2], ue8m0 bytes [T, ih, d/32], weights).

    RoPE on the last rope_dim dims, round to bf16, then one power-of-two scale per 32 values (the rope and non-rope
    parts are whole blocks).  The block scales stay with q, so only d^-0.5 and ih^-0.5 fold into the head weights
    (overlay/ops_fused_indexer_q.py:175-282)."""
    t, ih, d = q.shape
    qf = q.to(F32).clone()
    qf[..., d - rope_dim:] = apply_rope_interleaved(qf[..., d - rope_dim:], cos, sin)
    qf = qf.to(torch.bfloat16).to(F32)
    packed, scales = quant_mxfp4(qf)
    return packed, scales, weights.to(F32) * (d ** -0.5) * (ih ** -0.5)


def indexer_scores(q: torch.Tensor, w: torch.Tensor, k: torch.Tensor, k_scale: Optional[torch.Tensor]) -> torch.Tensor:
    """score[t, s] = sum_h w[t,h] * relu(q[t,h] . k[s]) * k_scale[s]."""
    dots = torch.einsum("thd,sd->ths", q.to(F32), k.to(F32))
    sc = (torch.relu(dots) * w.to(F32)[:, :, None]).sum(1)
    if k_scale is not None:
        sc = sc * k_scale.to(F32)[None, :]
    return sc


def topk_rows(scores: torch.Tensor, valid_len: torch.Tensor, k: int) -> torch.Tensor:
    """Per-row indices of the k largest scores among the first valid_len[t] columns, -1 padded.

    Order inside a row is unspecified for consumers; this statement returns them
    sorted by decreasing score (ties: lower index first)."""
    t, s = scores.shape
    out = torch.full((t, k), -1, dtype=torch.int32, device=scores.device)
    col = torch.arange(s, device=scores.device)
    for i in range(t):
        n = int(valid_len[i])
        if n <= 0:
            continue
        row = scores[i, :n]
        kk = min(k, n)
        idx = torch.argsort(row, descending=True, stable=True)[:kk]
        out[i, :kk] = col[idx].to(torch.int32)
    return out


# ----------------------------------------------------------------------------
# KV compressor (gated pooling over ratio-sized windows, optional overlap)
# ----------------------------------------------------------------------------
def compressor_pool(kv: torch.Tensor, score: torch.Tensor, ape: torch.Tensor, ratio: int, overlap: bool,
                    first_window: int = 0, prev_kv: Optional[torch.Tensor] = None,
                    prev_score: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Pool complete windows of one sequence.

    kv, score: [n_windows*ratio, c, D] for the tokens of windows first_window.. (c = 2 if overlap else 1)
    ape: [ratio, c, D] gate bias per in-window position.
    prev_kv/prev_score: [ratio, c, D] of window first_window-1 (overlap only, None at sequence start).
    Returns [n_windows, D].

    Window j pools, per channel, a softmax over: its own ratio tokens using slot 0,
    and (overlap) the ratio tokens of window j-1 using slot 1."""
    n = kv.shape[0] // ratio
    d = kv.shape[-1]
    kvw = kv.to(F32).view(n, ratio, -1, d)
    scw = score.to(F32).view(n, ratio, -1, d) + ape.to(F32)[None]
    vals = [kvw[:, :, 0]]
    logits = [scw[:, :, 0]]
    if overlap:
        pk = torch.zeros(n, ratio, d, dtype=F32, device=kv.device)
        ps = torch.full((n, ratio, d), float("-inf"), dtype=F32, device=kv.device)
        if n > 1:
            pk[1:] = kvw[:-1, :, 1]
            ps[1:] = scw[:-1, :, 1]
        if prev_kv is not None:
            pk[0] = prev_kv.to(F32)[:, 1]
            ps[0] = prev_score.to(F32)[:, 1] + ape.to(F32)[:, 1]
        vals.append(pk)
        logits.append(ps)
    v = torch.cat(vals, dim=1)
    l = torch.cat(logits, dim=1)
    p = torch.softmax(l, dim=1)
    return (p * v).sum(1)


# ----------------------------------------------------------------------------
# sparse MLA attention over gathered rows
# ----------------------------------------------------------------------------
def sparse_mla(q: torch.Tensor, rows: torch.Tensor, row_valid: torch.Tensor, sink: Optional[torch.Tensor],
               scale: float) -> torch.Tensor:
    """q [T, nh, D]; rows [T, L, D] gathered (dequantised) KV rows; row_valid [T, L] bool;
    sink [nh] logit that only joins the softmax denominator.  K = V = the row.  -> [T, nh, D]."""
    logits = torch.einsum("thd,tld->thl", q.to(F32), rows.to(F32)) * scale
    logits = logits.masked_fill(~row_valid[:, None, :], float("-inf"))
    if sink is not None:
        sk = sink.to(F32)[None, :, None].expand(logits.shape[0], -1, 1)
        logits = torch.cat([logits, sk], dim=-1)
    m = logits.amax(-1, keepdim=True)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(logits - m)
    denom = p.sum(-1, keepdim=True).clamp(min=1e-30)
    p = p / denom
    if sink is not None:
        p = p[..., :-1]
    return torch.einsum("thl,tld->thd", p, rows.to(F32))


# ----------------------------------------------------------------------------
# router
# ----------------------------------------------------------------------------
def router_scores(logits: torch.Tensor, scoring: str) -> torch.Tensor:
    lf = logits.to(F32)
    if scoring == "sigmoid":
        return torch.sigmoid(lf)
    if scoring == "sqrtsoftplus":
        return torch.sqrt(torch.nn.functional.softplus(lf))
    raise ValueError(scoring)


def route(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, scoring: str, renorm: bool,
          scaling: float, hash_ids: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (expert ids [T, k] int32, weights [T, k] fp32).  Selection uses score+bias,
    weights use the unbiased score.  hash_ids [T, k] (already looked up) overrides selection."""
    scores = router_scores(logits, scoring)
    if hash_ids is not None:
        ids = hash_ids.long()
    else:
        sel = scores + bias.to(F32)[None] if bias is not None else scores
        # ties broken toward the lower expert id
        ids = torch.argsort(sel, dim=-1, descending=True, stable=True)[:, :top_k]
    w = torch.gather(scores, 1, ids)
    if renorm:
        w = w / w.sum(-1, keepdim=True).clamp(min=1e-20)
    return ids.to(torch.int32), w * scaling


# ----------------------------------------------------------------------------
# sampling: counter-based Gumbel noise keyed by (seed, position, vocab id)
# ----------------------------------------------------------------------------
_M32 = 0xFFFFFFFF


def _mix32(x: torch.Tensor) -> torch.Tensor:
    """A 32-bit integer finaliser (xor-shift-multiply) on int64 tensors holding uint32 values."""
    x = x & _M32
    x = ((x ^ (x >> 16)) * 0x7FEB352D) & _M32
    x = ((x ^ (x >> 15)) * 0x846CA68B) & _M32
    x = (x ^ (x >> 16)) & _M32
    return x


def gumbel_noise(seed: torch.Tensor, pos: torch.Tensor, vocab: int) -> torch.Tensor:
    """g[b, v] = -log(-log(u)), u in (0,1) a pure function of (seed[b], pos[b], v).  seed/pos int64 [B]."""
    v = torch.arange(vocab, dtype=torch.int64, device=seed.device)[None, :]
    s = seed.to(torch.int64)[:, None]
    p = pos.to(torch.int64)[:, None]
    h = _mix32((s & _M32) ^ 0x9E3779B9)
    h = _mix32(h ^ _mix32(((s >> 32) & _M32) + 0x85EBCA6B))
    h = _mix32(h ^ _mix32((p & _M32) + 0xC2B2AE35))
    h = _mix32(h ^ _mix32(v + 0x27D4EB2F))
    u = ((h >> 8).to(F32) + 0.5) * (1.0 / 16777216.0)      # 24 random bits, never 0 or 1
    return -torch.log(-torch.log(u))


def truncation_mask(logits: torch.Tensor, temperature: torch.Tensor, top_k: Optional[torch.Tensor],
                    top_p: Optional[torch.Tensor]) -> torch.Tensor:
    """[B, V] bool: inside the top-k set and the top-p nucleus (of the top-k survivors, at temperature T); ties at
    either threshold are kept."""
    lf = logits.to(F32)
    b, v = lf.shape
    keep = torch.ones(b, v, dtype=torch.bool, device=lf.device)
    for i in range(b):
        row = lf[i]
        k = int(top_k[i]) if top_k is not None else 0
        if 0 < k < v:
            keep[i] &= row >= torch.topk(row, k).values[-1]
        p = float(top_p[i]) if top_p is not None else 1.0
        t = float(temperature[i])
        if p < 1.0 and t > 0:
            masked = torch.where(keep[i], row, torch.full_like(row, float("-inf")))
            pr = torch.softmax(masked / t, -1)
            srt, _ = torch.sort(pr, descending=True)
            cum = torch.cumsum(srt, 0)
            j = int((cum >= p).nonzero()[0]) if bool((cum >= p).any()) else v - 1
            keep[i] &= pr >= srt[j]
    return keep


def gumbel_sample(logits: torch.Tensor, temperature: torch.Tensor, seed: torch.Tensor, pos: torch.Tensor,
                  top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (token [B] int64, processed logits [B, V] = logits/T, -inf outside the top-k / top-p set).
    temperature 0 => greedy."""
    lf = logits.to(F32)
    t = temperature.to(F32)[:, None]
    greedy = t <= 0
    proc = lf / torch.where(greedy, torch.ones_like(t), t)
    if top_k is not None or top_p is not None:
        proc = torch.where(truncation_mask(lf, temperature.to(F32), top_k, top_p), proc, torch.full_like(proc, float("-inf")))
    noisy = torch.where(greedy, proc, proc + gumbel_noise(seed, pos, lf.shape[-1]))
    return noisy.argmax(-1), proc


def coupled_verify(draft_tokens: torch.Tensor, target_logits: torch.Tensor, temperature: torch.Tensor,
                   seed: torch.Tensor, pos0: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Seeded-Gumbel coupled acceptance.

    draft_tokens [B, N] (sampled as argmax(log q + g(seed, pos0+i)));
    target_logits [B, N+1, V] for positions pos0 .. pos0+N.
    The verifier token at offset i is argmax(log p_i + g(seed, pos0+i)); draft i is
    accepted iff all earlier ones were and it equals that token.  The emitted token at
    every offset is the verifier's, so the output follows the target distribution for any q
    (overlay/dspark_speculator_v2.py:32-38).
    -> (num_accepted [B], emitted tokens [B, N+1]; entries past num_accepted+1 are -1)."""
    b, n1, v = target_logits.shape
    n = n1 - 1
    emitted = torch.full((b, n1), -1, dtype=torch.int64, device=target_logits.device)
    ok = torch.ones(b, dtype=torch.bool, device=target_logits.device)
    n_acc = torch.zeros(b, dtype=torch.int64, device=target_logits.device)
    for i in range(n1):
        tok, _ = gumbel_sample(target_logits[:, i], temperature, seed, pos0 + i)
        emitted[:, i] = torch.where(ok, tok, emitted[:, i])
        if i < n:
            ok = ok & (tok == draft_tokens[:, i].to(torch.int64))
            n_acc = n_acc + ok.to(torch.int64)
    return n_acc, emitted


def markov_bias_topk(base_logits: torch.Tensor, w2: torch.Tensor, embed: torch.Tensor, topk: int
                     ) -> torch.Tensor:
    """DSpark first-order Markov head restricted to the base-logit top-k.

    base_logits [B, V]; w2 [V, R]; embed [B, R] (W1 row of the previous token).
    Returns logits [B, V] = base + W2[idx]·embed on the top-k set, -inf elsewhere
    (topk == 0: dense bias over the whole vocabulary).
    (overlay/dspark_v2.py:184-236, overlay/dspark_speculator_v2.py:255-259)"""
    lf = base_logits.to(F32)
    if topk <= 0 or topk >= lf.shape[-1]:
        return lf + embed.to(F32) @ w2.to(F32).t()
    val, idx = torch.topk(lf, topk, dim=-1)
    bias = torch.einsum("bkr,br->bk", w2.to(F32)[idx], embed.to(F32))
    out = torch.full_like(lf, float("-inf"))
    out.scatter_(1, idx, val + bias)
    return out


# ----------------------------------------------------------------------------
# dense / grouped linear
# ----------------------------------------------------------------------------
def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return x.to(F32) @ w.to(F32).t()


def moe_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor,
                limit: float, expert_offset: int = 0) -> torch.Tensor:
    """x [T, H]; ids/weights [T, k]; w13 [E_local, 2I, H] (gate rows then up rows); w2 [E_local, H, I].
    Experts outside [expert_offset, expert_offset+E_local) contribute nothing (expert parallel)."""
    t, h = x.shape
    e_local, two_i, _ = w13.shape
    inter = two_i // 2
    out = torch.zeros(t, h, dtype=F32, device=x.device)
    xf = x.to(F32)
    for e in range(e_local):
        mask = ids == (e + expert_offset)
        tok = mask.any(-1).nonzero().flatten()
        if tok.numel() == 0:
            continue
        wt = (weights * mask).sum(-1)[tok]
        gu = xf[tok] @ w13[e].to(F32).t()
        act = swiglu_clamp(gu[:, :inter], gu[:, inter:], limit)
        out[tok] += (act @ w2[e].to(F32).t()) * wt[:, None]
    return out
