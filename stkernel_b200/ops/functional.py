"""The op layer: every function runs the sm_100a kernel when its tensors live on
a GPU and the PyTorch reference statement (:mod:`.reference`) on CPU.

On a GPU there is no fallback: a missing library raises (see :mod:`._lib`).
Scratch buffers come from :mod:`.scratch`, so addresses are stable across steps
and the whole decode step can be captured in a CUDA graph.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ..config import FP8_BLOCK
from . import _lib
from . import reference as R
from .scratch import scratch

BF16 = torch.bfloat16
F32 = torch.float32
FP8 = torch.float8_e4m3fn

import os as _os
import weakref

# STK_CPU_ACT_FP32=1: fp32 activations on the CPU path (exact comparisons across TP degrees)
_CPU_ACT = [torch.float32 if _os.environ.get("STK_CPU_ACT_FP32") == "1" else torch.bfloat16]


def set_cpu_act_dtype(dtype: torch.dtype) -> None:
    """Activation dtype of the CPU reference path (bf16 mirrors the GPU; fp32 for exact oracle checks)."""
    _CPU_ACT[0] = dtype


def cpu_act_dtype() -> torch.dtype:
    return _CPU_ACT[0]


# ----------------------------------------------------------------------------
# dense linear
# ----------------------------------------------------------------------------
@dataclass
class LinearWeight:
    """[N, K] weight in its storage format: bf16, or e4m3 with 128x128 fp32 block scales."""
    w: torch.Tensor
    scale: Optional[torch.Tensor] = None

    @property
    def is_fp8(self) -> bool:
        return self.scale is not None

    @property
    def out_features(self) -> int:
        return self.w.shape[0]

    @property
    def in_features(self) -> int:
        return self.w.shape[1]

    @staticmethod
    def from_master(w: torch.Tensor, dense_dtype: str, device, ue8m0: bool = False) -> "LinearWeight":
        if dense_dtype == "fp8":
            q, s = R.quant_fp8_block128_weight(w.to(device=device, dtype=F32), ue8m0=ue8m0)
            return LinearWeight(q.contiguous(), s.contiguous())
        return LinearWeight(w.to(device=device, dtype=BF16).contiguous())

    def dequant(self) -> torch.Tensor:
        if self.is_fp8:
            return R.dequant_fp8_block128_weight(self.w, self.scale)
        return self.w.to(F32)


@dataclass
class QuantAct:
    """fp8 activation [T, K] with scales stored token-contiguous: [ceil(K/128), ld], ld % 4 == 0."""
    q: torch.Tensor
    scale: torch.Tensor


@dataclass
class LLPending:
    """A [T, H] bf16 activation that exists only as per-rank partial sums in the receive slots of a folded all-reduce
    (`parallel.symm.LLExchange`): the producer kernel pushed them, the consumer kernel (`mhc_post_pre`, or `ll_reduce`)
    adds the ranks.  Exactly one consumer must follow each producer on the same stream."""
    ex: "object"
    t: int
    h: int
    device: torch.device

    @property
    def shape(self):
        return (self.t, self.h)


def ll_push(x: torch.Tensor, ex) -> LLPending:
    """Producer on its own: push a finished [T, H] bf16 tensor into every rank's slot."""
    t, h = x.shape
    _lib.call("stk_ll_push", ex.ctx, x, x.stride(0), t, h, _lib.stream())
    return LLPending(ex, t, h, x.device)


def ll_reduce(p: LLPending) -> torch.Tensor:
    """Consumer on its own: the sum over ranks as a plain bf16 tensor."""
    out = torch.empty(p.t, p.h, dtype=BF16, device=p.device)
    _lib.call("stk_ll_reduce", p.ex.ctx, out, out.stride(0), p.t, p.h, _lib.status_buffer(), _lib.stream())
    return out


# largest batch served by the weight-streaming kernels: CUDA-core dot products up to four tokens, the eight-token
# warp-level tensor-core stream above (speculative verification rows, small decode batches)
SKINNY_MAX_T = min(8, int(_os.environ.get("STK_SKINNY_MAX_T", "8")))
MHC_CLUSTER_MAX_T = int(_os.environ.get("STK_MHC_CLUSTER_MAX_T", "64"))


def _skinny_rows(t: int) -> int:
    """Rows of the kernel instance that serves a batch of t tokens (its activation tile lives in shared memory)."""
    return t if t <= 4 else (6 if t <= 6 else 8)


def wants_quant_act(t: int, device) -> bool:
    """Whether fp8 layers should be fed pre-quantised activations for a step of t tokens (the
    weight-streaming kernel used for t <= 4 on a GPU takes bf16 activations)."""
    return not (torch.device(device).type == "cuda" and t <= SKINNY_MAX_T)


def _scale_ld(t: int) -> int:
    return max(4, (t + 3) // 4 * 4)


def quant_act(x: torch.Tensor, tag: str = "act") -> QuantAct:
    """Per-token 1x128 group quantisation of a bf16 activation."""
    t, k = x.shape
    if not x.is_cuda:
        q, s = R.quant_fp8_group128_act(x)
        return QuantAct(q, s.t().contiguous())
    kb = (k + FP8_BLOCK - 1) // FP8_BLOCK
    ld = _scale_ld(t)
    q = scratch(f"{tag}.q", (t, k), torch.uint8, x.device)
    s = scratch(f"{tag}.s", (kb, ld), F32, x.device)
    _lib.call("stk_quant_fp8_group128", x, x.stride(0), q, k, s, ld, t, k, _lib.stream())
    return QuantAct(q.view(FP8), s)


SKINNY_NARROW_BYTES = 4 << 20        # bf16 weights this small (the router gate) stay in L2 while groups of eight tokens stream them again
SKINNY_NARROW_MAX_T = 64
# Off by default: one rank's share of an 8-rank group gained 7 % per 64-token step with it (3507 -> 3277 us), the same
# step of the unsharded 6-layer model on one GPU lost 7 % (10057 -> 10789 us) without any one kernel accounting for it.
SKINNY_NARROW = _os.environ.get("STK_SKINNY_NARROW", "0") == "1"


def _skinny_ok(x, t: int, k: int, is_fp8: bool, n: Optional[int] = None, rows: Optional[int] = None) -> bool:
    """Whether the weight-streaming kernels serve x[t, k] @ W[n, k]^T.  `rows`: weight rows actually streamed (2n for the
    fused SwiGLU pair, n * groups for a block-diagonal weight)."""
    if not (isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == BF16):
        return False
    if t > SKINNY_MAX_T:
        # narrow bf16 weights (router gate, side projections): up to 64 tokens in groups of eight
        if not (SKINNY_NARROW and SKINNY_MAX_T >= 8 and not is_fp8 and t <= SKINNY_NARROW_MAX_T and n is not None
                and (rows or n) * k * 2 <= SKINNY_NARROW_BYTES):
            return False
    if t > 4:
        # five to eight tokens: the warp-level tensor-core stream (16 weight rows per CTA, 128-value scale groups,
        # eight activation rows in shared memory)
        return (k % 128 == 0 and (n is None or n % 16 == 0) and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
                and 8 * ((k if is_fp8 else 2 * k) + 64) + 8 * (k // 128) * 4 + 4096 + (2 * k * min(t, 8) if is_fp8 else 0) + 2 * k
                <= 200 * 1024)
    # a lane holds at most 32 16-byte chunks of a weight row: K <= 16384 for fp8, K <= 8192 for bf16
    return k % 16 == 0 and k <= (16384 if is_fp8 else 8192) and _skinny_rows(t) * k * 2 <= 160 * 1024


def linear(x, lw: LinearWeight, out: Optional[torch.Tensor] = None, out_dtype=BF16, tag: str = "lin",
           splits: Optional[int] = None, groups: int = 1, ar_ctx=None, norm=None, ll=None):
    """out[T, N] = x[T, K] @ W[N, K]^T.  x: bf16 tensor or a QuantAct (required format for fp8 weights
    is produced on the fly when a bf16 tensor is given).

    ar_ctx: symmetric-memory context; the kernel then all-reduces the output over the ranks in its
    epilogue (row-parallel layers).  The output must be contiguous.

    groups > 1: block-diagonal product.  W is [N, K] with N/groups rows per group, x is [T, groups*K];
    output columns of group g use x[:, g*K:(g+1)*K].

    norm = (weight, eps): x is RMS-normalised first (inside the weight-streaming kernel for decode-sized batches).
    ll: an `LLExchange`; the bf16 result is a per-rank partial sum that goes into the folded all-reduce and an
    `LLPending` is returned instead of a tensor (row-parallel layers at decode sizes)."""
    if (norm is not None or ll is not None) and not isinstance(x, QuantAct) and x.is_cuda:
        t0, (n0, k0) = x.shape[0], lw.w.shape
        if groups == 1 and ar_ctx is None and out_dtype == BF16 and _skinny_ok(x, t0, k0, lw.is_fp8, n0 // max(groups, 1), n0) and (ll is None or n0 % 2 == 0):
            o = out if out is not None else (None if ll is not None else torch.empty(t0, n0, dtype=BF16, device=x.device))
            _lib.call("stk_skinny_linear_fused", lw.w, lw.w.stride(0), 1 if lw.is_fp8 else 0, lw.scale,
                      lw.scale.stride(0) if lw.is_fp8 else 0, x, x.stride(0), o, o.stride(0) if o is not None else 0, t0, n0, k0,
                      0, _lib.sm_count(), norm[0] if norm is not None else None, float(norm[1]) if norm is not None else 0.0,
                      ll.ctx if ll is not None else None, 0, None, None, None, None, 0, None, None, 0, 0, 0, 0.0,
                      _lib.status_buffer(), _lib.stream())
            return LLPending(ll, t0, n0, x.device) if ll is not None else o
    if norm is not None:
        x = rms_norm(x, norm[0], norm[1])
    if ll is not None:
        return ll_push(linear(x, lw, out, out_dtype, tag, splits, groups, ar_ctx), ll)
    if isinstance(x, QuantAct):
        xa, dev, t = x, x.q.device, x.q.shape[0]
    else:
        xa, dev, t = None, x.device, x.shape[0]
    n, k = lw.w.shape
    if groups > 1 and dev.type != "cuda":
        xf = x if xa is None else R.dequant_fp8_group128_act(xa.q, xa.scale.t()[:t])
        if lw.is_fp8 and xa is None:
            xf = torch.cat([R.dequant_fp8_group128_act(*R.quant_fp8_group128_act(xf[:, g * k:(g + 1) * k]))
                            for g in range(groups)], 1)
        wd = lw.dequant().view(groups, n // groups, k)
        y = torch.einsum("tgk,gnk->tgn", xf.to(F32).view(t, groups, k), wd).reshape(t, n)
        y = y.to(out_dtype if out_dtype != BF16 else cpu_act_dtype())
        if out is not None:
            out.copy_(y)
            return out
        return y
    if dev.type != "cuda":
        if lw.is_fp8:
            if xa is None:
                xa = quant_act(x)
            xf = R.dequant_fp8_group128_act(xa.q, xa.scale.t()[:t])
        else:
            xf = (x if xa is None else R.dequant_fp8_group128_act(xa.q, xa.scale.t()[:t])).to(cpu_act_dtype()).to(F32)
        y = xf @ lw.dequant().t()
        y = y.to(out_dtype if out_dtype != BF16 else cpu_act_dtype())
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty(t, n, dtype=out_dtype, device=dev)
    if xa is None and ar_ctx is None and _skinny_ok(x, t, k, lw.is_fp8, n // max(groups, 1), n):
        # one to four tokens: weight-streaming kernel, activations unquantised
        _lib.call("stk_skinny_linear", lw.w, lw.w.stride(0), 1 if lw.is_fp8 else 0, lw.scale,
                  lw.scale.stride(0) if lw.is_fp8 else 0, x, x.stride(0), out, out.stride(0), t, n, k,
                  1 if out.dtype == F32 else 0, _lib.sm_count(), groups, 0, 0.0, _lib.stream())
        return out
    if lw.is_fp8 and xa is None:
        xa = quant_act(x, tag + ".xq")
    is_fp8 = 1 if lw.is_fp8 else 0
    sms = _lib.sm_count()
    if splits is None:
        splits = _lib.query("stk_gemm_pick_splits", t, n, k, is_fp8, sms)
    ws = cnt = None
    if splits > 1:
        ws = scratch("gemm.splitk", (splits * t * n,), F32, dev)
        cnt = scratch("gemm.counters", (4096,), torch.int32, dev, zero=True)
    xin = xa.q if is_fp8 else x
    if not is_fp8 and xin.dtype != BF16:
        xin = xin.to(BF16)
    _lib.call("stk_gemm", lw.w, lw.w.stride(0), xin, xin.stride(0), out, out.stride(0), t, n, k, is_fp8,
              1 if out.dtype == F32 else 0, lw.scale, lw.scale.stride(0) if is_fp8 else 0,
              xa.scale if is_fp8 else None, xa.scale.stride(0) if is_fp8 else 0, splits, ws, cnt,
              _lib.status_buffer(), sms, groups, ctypes.addressof(ar_ctx) if ar_ctx is not None else None,
              _lib.stream())
    return out


_route_counters: dict = {}


GATE_CLUSTER = _os.environ.get("STK_GATE_CLUSTER", "1") != "0"
_gate_cluster_state: dict = {}


def _gate_cluster_ok() -> bool:
    d = torch.cuda.current_device()
    if d not in _gate_cluster_state:
        _gate_cluster_state[d] = _lib.query("stk_gate_route_cluster_ok") == 1
    return _gate_cluster_state[d]


def gate_route(x: torch.Tensor, w_gate: LinearWeight, bias, top_k: int, scoring: str, renorm: bool, scaling: float,
               tid2eid=None, token_ids=None):
    """Router gate projection and expert selection in one launch for decode-sized batches (the CTA that finishes the
    projection last routes the tokens); returns (ids i32 [T, k], weights f32 [T, k]) or None when that kernel does
    not apply (the caller then runs the projection and the router separately)."""
    t, k = x.shape
    e = w_gate.w.shape[0]
    if not _skinny_ok(x, t, k, w_gate.is_fp8) or e > 512 or top_k > 32:
        return None
    dev = x.device
    ids = torch.empty(t, top_k, dtype=torch.int32, device=dev)
    wts = torch.empty(t, top_k, dtype=F32, device=dev)
    vocab = tid2eid.shape[0] if tid2eid is not None else 0
    w = w_gate.w
    if (GATE_CLUSTER and not w_gate.is_fp8 and w.dtype == BF16 and k <= 4096 and k % 8 == 0 and w.stride(0) % 8 == 0
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and _gate_cluster_ok()):
        # one 16-CTA cluster: the logits meet in distributed shared memory instead of global memory
        _lib.call("stk_gate_route_cluster", w, w.stride(0), x, x.stride(0), t, e, k, bias, tid2eid, token_ids, vocab, ids,
                  wts, top_k, 0 if scoring == "sigmoid" else 1, 1 if renorm else 0, float(scaling), _lib.status_buffer(),
                  _lib.stream())
        return ids, wts
    cnt = _route_counters.get(dev.index)
    if cnt is None:
        cnt = _route_counters[dev.index] = torch.zeros(1, dtype=torch.int32, device=dev)
    logits = scratch("gate.logits", (t, e), F32, dev, zero=True)      # zero on entry, left zero by the kernel
    _lib.call("stk_skinny_linear_fused", w_gate.w, w_gate.w.stride(0), 1 if w_gate.is_fp8 else 0, w_gate.scale,
              w_gate.scale.stride(0) if w_gate.is_fp8 else 0, x, x.stride(0), logits, logits.stride(0), t, e, k, 1,
              _lib.sm_count(), None, 0.0, None, 2, cnt, bias, tid2eid, token_ids, vocab, ids, wts, top_k,
              0 if scoring == "sigmoid" else 1, 1 if renorm else 0, float(scaling), _lib.status_buffer(), _lib.stream())
    return ids, wts


def linear_swiglu(x: torch.Tensor, lw13: LinearWeight, limit: float) -> Optional[torch.Tensor]:
    """act[T, I] = silu(min(x W1^T, lim)) * clamp(x W3^T) with W13 = [W1; W3] in one weight-streaming launch
    (decode-sized batches on a GPU); returns None when that kernel does not apply."""
    t, k = x.shape
    n2 = lw13.w.shape[0]
    if not x.is_cuda or t > SKINNY_MAX_T or x.dtype != BF16 or k % 16 or k > 8192 or n2 % 2 or _skinny_rows(t) * k * 2 > 160 * 1024:
        return None
    i = n2 // 2
    if t > 4 and not _skinny_ok(x, t, k, lw13.is_fp8, i, n2):
        return None
    if lw13.is_fp8 and i % 128:
        return None
    out = torch.empty(t, i, dtype=BF16, device=x.device)
    _lib.call("stk_skinny_linear", lw13.w, lw13.w.stride(0), 1 if lw13.is_fp8 else 0, lw13.scale,
              lw13.scale.stride(0) if lw13.is_fp8 else 0, x, x.stride(0), out, out.stride(0), t, i, k, 0, _lib.sm_count(),
              1, 1, float(limit), _lib.stream())
    return out


# ----------------------------------------------------------------------------
# norms / elementwise
# ----------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, quant: bool = False, tag: str = "norm"):
    """bf16 RMSNorm; with quant=True also returns the fp8 QuantAct of the normed row."""
    t, h = x.shape
    if not x.is_cuda:
        y = R.rms_norm(x, w, eps).to(cpu_act_dtype())
        return (y, quant_act(y)) if quant else y
    out = torch.empty(t, h, dtype=BF16, device=x.device)
    q = s = None
    ld = _scale_ld(t)
    if quant:
        q = scratch(f"{tag}.q", (t, h), torch.uint8, x.device)
        s = scratch(f"{tag}.s", ((h + 127) // 128, ld), F32, x.device)
    _lib.call("stk_rmsnorm", x, x.stride(0), w, out, h, h, q, h, s, ld,
              None, 0, None, None, 0, 0, t, eps, _lib.stream())
    return (out, QuantAct(q.view(FP8), s)) if quant else out


def rms_norm_pair(x0, w0, x1, w1, eps: float, quant0: bool = False, tag: str = "norm2"):
    """Two independent RMSNorms in one launch (q_lora row and kv row)."""
    t = x0.shape[0]
    if not x0.is_cuda:
        y0, y1 = R.rms_norm(x0, w0, eps).to(cpu_act_dtype()), R.rms_norm(x1, w1, eps).to(cpu_act_dtype())
        return (y0, y1, quant_act(y0)) if quant0 else (y0, y1)
    h0, h1 = x0.shape[1], x1.shape[1]
    o0 = torch.empty(t, h0, dtype=BF16, device=x0.device)
    o1 = torch.empty(t, h1, dtype=BF16, device=x0.device)
    q = s = None
    ld = _scale_ld(t)
    if quant0:
        q = scratch(f"{tag}.q", (t, h0), torch.uint8, x0.device)
        s = scratch(f"{tag}.s", ((h0 + 127) // 128, ld), F32, x0.device)
    _lib.call("stk_rmsnorm", x0, x0.stride(0), w0, o0, h0, h0, q, h0, s, ld,
              x1, x1.stride(0), w1, o1, h1, h1, t, eps, _lib.stream())
    return (o0, o1, QuantAct(q.view(FP8), s)) if quant0 else (o0, o1)


def swiglu_clamp(gu: torch.Tensor, limit: float, quant: bool = False, tag: str = "swiglu"):
    t, two_i = gu.shape
    i = two_i // 2
    if not gu.is_cuda:
        a = R.swiglu_clamp(gu[:, :i], gu[:, i:], limit).to(cpu_act_dtype())
        return (a, quant_act(a)) if quant else a
    act = torch.empty(t, i, dtype=BF16, device=gu.device)
    q = s = None
    ld = _scale_ld(t)
    if quant:
        q = scratch(f"{tag}.q", (t, i), torch.uint8, gu.device)
        s = scratch(f"{tag}.s", ((i + 127) // 128, ld), F32, gu.device)
    _lib.call("stk_swiglu_clamp", gu, gu.stride(0), act, i, t, i, float(limit), q, i, s, ld, _lib.stream())
    return (act, QuantAct(q.view(FP8), s)) if quant else act


def embed_hc(ids: torch.Tensor, embed: torch.Tensor, hc: int, vocab: int, vocab_start: int = 0) -> torch.Tensor:
    """ids [T] -> [T, hc, H] (each stream a copy of the embedding row; rows outside this rank's
    vocabulary shard are zero so a sum across ranks completes them)."""
    t = ids.shape[0]
    h = embed.shape[1]
    vend = vocab_start + embed.shape[0]
    if not ids.is_cuda:
        local = ids.long() - vocab_start
        ok = (local >= 0) & (local < embed.shape[0])
        x = torch.where(ok[:, None], embed[local.clamp(0, embed.shape[0] - 1)], torch.zeros_like(embed[:1]))
        return x[:, None, :].repeat(1, hc, 1).to(cpu_act_dtype())
    out = torch.empty(t, hc, h, dtype=BF16, device=ids.device)
    _lib.call("stk_embed_hc", ids, embed, out, t, h, hc, vocab, vocab_start, vend, _lib.status_buffer(), _lib.stream())
    return out


# ----------------------------------------------------------------------------
# mHC
# ----------------------------------------------------------------------------
MHC_GEMM_MIN_T = 256
_MHC_WCAT: dict = {}


def _mhc_wcat(fn: torch.Tensor, n_mix: int) -> torch.Tensor:
    """[128, hc*H] bf16: rows [0, n_mix) the bf16 rounding of fn, rows [32, 32 + n_mix) the bf16 rounding of the
    remainder, zeros elsewhere (a full 128-row weight tile).  Built once per weight tensor."""
    # keyed by the tensor object, not its address: a freed weight's address is reused by the allocator
    ent = _MHC_WCAT.get(id(fn))
    if ent is not None and ent[0]() is fn and ent[2] == fn._version:
        return ent[1]
    hi = fn.to(BF16)
    lo = (fn - hi.to(F32)).to(BF16)
    w = torch.zeros(128, fn.shape[1], dtype=BF16, device=fn.device)
    w[:n_mix] = hi
    w[32:32 + n_mix] = lo
    if len(_MHC_WCAT) > 4096:
        for k in [k for k, v in _MHC_WCAT.items() if v[0]() is None]:
            del _MHC_WCAT[k]
    _MHC_WCAT[id(fn)] = (weakref.ref(fn), w, fn._version)
    return w


def mhc_pre(residual: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor,
            norm_w: Optional[torch.Tensor], rms_eps: float, hc_eps: float, iters: int, quant: bool = False,
            tag: str = "mhc"):
    """residual [T, hc, H] bf16 -> (y [T, H] bf16, post [T, hc] f32, comb [T, hc*hc] f32[, QuantAct(y)])."""
    t, hc, h = residual.shape
    if not residual.is_cuda:
        y, post, comb = R.mhc_pre(residual, fn, base, scale, norm_w, rms_eps, hc_eps, iters, round_bf16=True)
        y = y.to(cpu_act_dtype())
        res = (y, post, comb.reshape(t, hc * hc))
        return res + (quant_act(y),) if quant else res
    dev = residual.device
    n_mix = (2 + hc) * hc
    if t <= MHC_CLUSTER_MAX_T and hc == 4 and h % 32 == 0 and h <= 4096:
        y = torch.empty(t, h, dtype=BF16, device=dev)
        post = torch.empty(t, hc, dtype=F32, device=dev)
        comb = torch.empty(t, hc * hc, dtype=F32, device=dev)
        _lib.call("stk_mhc_decode", residual, None, None, None, None, None, fn, base, scale, norm_w, post, comb, y, t, h,
                  rms_eps, hc_eps, iters, 2.0, None, _lib.status_buffer(), _lib.stream())
        return (y, post, comb, quant_act(y, tag + ".q")) if quant else (y, post, comb)
    if t <= MHC_CLUSTER_MAX_T and n_mix in (24, 8) and h <= 16384:
        # decode-sized batch: one launch, an 8-CTA cluster per token (DSMEM reductions); a quantised copy of the
        # few output rows, when the consumer wants one, is a second tiny launch
        y = torch.empty(t, h, dtype=BF16, device=dev)
        post = torch.empty(t, hc, dtype=F32, device=dev)
        comb = torch.empty(t, hc * hc, dtype=F32, device=dev)
        _lib.call("stk_mhc_cluster", residual, fn, base, scale, norm_w, post, comb, y, t, h, hc, n_mix, rms_eps, hc_eps,
                  iters, 2.0, 0, _lib.stream())
        return (y, post, comb, quant_act(y, tag + ".q")) if quant else (y, post, comb)
    if t >= MHC_GEMM_MIN_T and n_mix <= 32 and (hc * h) % 64 == 0:
        # many tokens: the [n_mix, hc*H] mix projection runs on the tensor cores.  fn (fp32) is split into a bf16 high
        # part and a bf16 remainder (two weight rows per mix, products accumulate in fp32: ~16 mantissa bits, more
        # than the tf32 the reference uses); narrow 32-token tiles supply the parallelism, no split-K.
        wcat = _mhc_wcat(fn, n_mix)
        x2d = residual.view(t, hc * h)
        prod = scratch("mhc.gemm", (t, 128), F32, dev)
        # one weight tile: the parallelism is token tiles x K splits (a sequence-parallel rank holds a few hundred tokens)
        tiles = (t + 31) // 32
        splits = max(1, min(16, _lib.sm_count() // tiles, (hc * h) // 256))
        ws = cnt = None
        if splits > 1:
            ws = scratch("mhc.gemm.splitk", (splits * t * 128,), F32, dev)
            cnt = scratch("gemm.counters", (4096,), torch.int32, dev, zero=True)
        _lib.call("stk_gemm_tile", wcat, wcat.stride(0), x2d, x2d.stride(0), prod, 128, t, 128, hc * h, 1, 32, splits, ws, cnt,
                  _lib.status_buffer(), _lib.sm_count(), _lib.stream())
        partial = scratch("mhc.partial", (t * (n_mix + 1),), F32, dev).view(t, n_mix + 1)
        torch.add(prod[:, :n_mix], prod[:, 32:32 + n_mix], out=partial[:, :n_mix])
        _lib.call("stk_row_sumsq", x2d, x2d.stride(0), partial[:, n_mix:], n_mix + 1, t, hc * h, _lib.stream())
        splits = 1
    else:
        splits = _lib.query("stk_mhc_pick_splits", t, hc * h)
        partial = scratch("mhc.partial", (splits * t * (n_mix + 1),), F32, dev)
        _lib.call("stk_mhc_dots", residual, fn, partial, t, h, hc, n_mix, splits, _lib.stream())
    y = torch.empty(t, h, dtype=BF16, device=dev)
    post = torch.empty(t, hc, dtype=F32, device=dev)
    comb = torch.empty(t, hc * hc, dtype=F32, device=dev)
    q = s = None
    ld = _scale_ld(t)
    if quant:
        q = scratch(f"{tag}.q", (t, h), torch.uint8, dev)
        s = scratch(f"{tag}.s", ((h + 127) // 128, ld), F32, dev)
    _lib.call("stk_mhc_finalize", residual, partial, splits, n_mix + 1, 1, base, scale, norm_w, post, comb, y, t, h, hc,
              rms_eps, hc_eps, iters, 2.0, 0, q, s, ld, _lib.stream())
    return (y, post, comb, QuantAct(q.view(FP8), s)) if quant else (y, post, comb)


def mhc_post(x, residual: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    t, hc, h = residual.shape
    if isinstance(x, LLPending):
        x = ll_reduce(x)
    if not residual.is_cuda:
        return R.mhc_post(x, residual, post, comb.reshape(t, hc, hc)).to(cpu_act_dtype())
    out = torch.empty_like(residual)
    _lib.call("stk_mhc_post", x, residual, post, comb, out, t, h, hc, _lib.stream())
    return out


def mhc_post_pre(x: torch.Tensor, residual: torch.Tensor, post_old: torch.Tensor, comb_old: torch.Tensor,
                 fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor, norm_w: Optional[torch.Tensor], rms_eps: float,
                 hc_eps: float, iters: int, quant: bool = False, tag: str = "mhc"):
    """The post-mix of one sub-block followed by the pre-mix of the next: -> (new residual [T, hc, H], mhc_pre outputs).
    Decode-sized batches run both in one cluster launch (the new streams are formed on the fly from x and the old
    streams and never re-read); otherwise the two ops run back to back."""
    t, hc, h = residual.shape
    n_mix = (2 + hc) * hc
    if residual.is_cuda and t <= MHC_CLUSTER_MAX_T and hc == 4 and h % 32 == 0 and h <= 4096:
        dev = residual.device
        new_res = torch.empty_like(residual)
        y = torch.empty(t, h, dtype=BF16, device=dev)
        post = torch.empty(t, hc, dtype=F32, device=dev)
        comb = torch.empty(t, hc * hc, dtype=F32, device=dev)
        pend = isinstance(x, LLPending)
        _lib.call("stk_mhc_decode", None, None if pend else x, residual, post_old, comb_old, new_res, fn, base, scale, norm_w,
                  post, comb, y, t, h, rms_eps, hc_eps, iters, 2.0, x.ex.ctx if pend else None, _lib.status_buffer(),
                  _lib.stream())
        r = (y, post, comb, quant_act(y, tag + ".q")) if quant else (y, post, comb)
        return new_res, r
    if isinstance(x, LLPending):
        x = ll_reduce(x)
    if (residual.is_cuda and t <= MHC_CLUSTER_MAX_T and n_mix == 24 and h <= 16384 and h % 32 == 0):
        dev = residual.device
        new_res = torch.empty_like(residual)
        y = torch.empty(t, h, dtype=BF16, device=dev)
        post = torch.empty(t, hc, dtype=F32, device=dev)
        comb = torch.empty(t, hc * hc, dtype=F32, device=dev)
        _lib.call("stk_mhc_post_pre", x, residual, post_old, comb_old, new_res, fn, base, scale, norm_w, post, comb, y, t,
                  h, hc, n_mix, rms_eps, hc_eps, iters, 2.0, 0, _lib.stream())
        r = (y, post, comb, quant_act(y, tag + ".q")) if quant else (y, post, comb)
        return new_res, r
    new_res = mhc_post(x, residual, post_old, comb_old)
    return new_res, mhc_pre(new_res, fn, base, scale, norm_w, rms_eps, hc_eps, iters, quant=quant, tag=tag)


def hc_head(residual: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor, rms_eps: float,
            hc_eps: float) -> torch.Tensor:
    t, hc, h = residual.shape
    if not residual.is_cuda:
        return R.hc_head(residual, fn, base, scale, rms_eps, hc_eps).to(cpu_act_dtype())
    dev = residual.device
    if t <= MHC_CLUSTER_MAX_T and hc in (4, 8) and h <= 16384:
        y = torch.empty(t, h, dtype=BF16, device=dev)
        _lib.call("stk_mhc_cluster", residual, fn, base, scale, None, None, None, y, t, h, hc, hc, rms_eps, hc_eps, 0, 2.0,
                  1, _lib.stream())
        return y
    splits = _lib.query("stk_mhc_pick_splits", t, hc * h)
    partial = scratch("mhc.partial", (splits * t * (hc + 1),), F32, dev)
    _lib.call("stk_mhc_dots", residual, fn, partial, t, h, hc, hc, splits, _lib.stream())
    y = torch.empty(t, h, dtype=BF16, device=dev)
    _lib.call("stk_mhc_finalize", residual, partial, splits, hc + 1, 1, base, scale, None, None, None, y, t, h, hc,
              rms_eps, hc_eps, 0, 2.0, 1, None, None, 0, _lib.stream())
    return y


# ----------------------------------------------------------------------------
# rope / KV cache
# ----------------------------------------------------------------------------
def inv_freq(rope_dim: int, theta: float, device) -> torch.Tensor:
    return (1.0 / (theta ** (torch.arange(0, rope_dim, 2, dtype=F32) / rope_dim))).to(device)


def q_norm_rope(q: torch.Tensor, positions: torch.Tensor, inv: torch.Tensor, rope_dim: int, eps: float,
                norm: bool = True, inverse: bool = False) -> torch.Tensor:
    """q [T, nh, D] bf16 (modified in place on GPU): weightless per-head RMSNorm then RoPE on the last dims."""
    t, nh, d = q.shape
    if not q.is_cuda:
        qf = R.rms_norm(q, None, eps) if norm else q.to(F32)
        ang = positions.to(F32)[:, None] * inv[None, :]
        cos, sin = torch.cos(ang), torch.sin(ang)
        qf = torch.cat([qf[..., :d - rope_dim], R.apply_rope_interleaved(qf[..., d - rope_dim:], cos, sin, inverse)], -1)
        return qf.to(cpu_act_dtype())
    assert q.stride(2) == 1 and q.stride(1) == d
    _lib.call("stk_q_norm_rope", q, q.stride(0), positions, inv, t, nh, d, rope_dim, eps, 1 if norm else 0,
              1 if inverse else 0, _lib.stream())
    return q
