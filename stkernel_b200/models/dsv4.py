"""The engine's DeepSeek-V4-style decoder: paged caches, batched ragged steps, tensor/expert
parallel shards, every hot op a kernel from :mod:`stkernel_b200.ops`.

Layer order and data flow follow overlay/nvidia_model.py:1509-1572,1713-1841 and
overlay/attention.py:541-670; semantics are pinned by :mod:`.dsv4_oracle`.

Parallel layout (one rank per GPU, `tp` ranks):
  * replicated: embedding, mHC parameters, fused wq_a|wkv, compressors, indexer, router gate
  * column-parallel: wq_b (heads), wo_a (o-groups), shared-expert w1|w3, LM head (vocab)
  * row-parallel + all-reduce: wo_b, shared-expert w2
  * routed experts: expert-parallel (E/tp experts per rank), summed by the same all-reduce; decode-sized steps use a
    second copy cut along the intermediate dimension (1/tp of every expert per rank: balanced whatever the routing)
"""
from __future__ import annotations

import hashlib
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..config import KV_SCALE_BYTES, ModelConfig
from ..ops import attention as A
from ..ops import cache as C
from ..ops.cache import PAGE, PagedCache
from ..ops import functional as Fn
from ..ops import moe as M
from ..utils.spans import span
from ..ops.functional import LinearWeight
from ..ops.scratch import side_branch
from ..runtime.planning import (dcp_global_row, dcp_local_index, dcp_local_rows, dcp_owner, pp_layer_range, sp_gather_sizes,
                                split_indexer_prefill_chunks)
from .dsv4_oracle import index_cache_computes
from .weights import compressor_slots

BF16 = torch.bfloat16
F32 = torch.float32


# ----------------------------------------------------------------------------
# weight sources
# ----------------------------------------------------------------------------
class WeightSource:
    """Hands out fp32 master tensors by checkpoint name."""

    def get(self, name: str, shape: Tuple[int, ...], device) -> torch.Tensor:
        raise NotImplementedError


class DictSource(WeightSource):
    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self.t = tensors

    def get(self, name, shape, device):
        t = self.t[name]
        assert tuple(t.shape) == tuple(shape), (name, t.shape, shape)
        return t.to(device)


class RandomSource(WeightSource):
    """Random-init weights: every tensor is a pure function of (seed, name), so replicated
    tensors agree across ranks without communication."""

    def __init__(self, seed: int = 0, std: float = 0.02):
        self.seed, self.std = seed, std

    def _gen(self, name: str, device) -> torch.Generator:
        h = int.from_bytes(hashlib.sha256(f"{self.seed}:{name}".encode()).digest()[:7], "little")
        g = torch.Generator(device=device)
        g.manual_seed(h)
        return g

    def get(self, name, shape, device):
        dev = torch.device(device)
        g = self._gen(name, dev)
        if name.endswith("tid2eid"):
            return torch.randint(0, 1 << 30, shape, generator=g, device=dev, dtype=torch.int64)
        if name.endswith("norm.weight") or name.endswith("_scale"):
            return torch.ones(shape, device=dev)
        if name.endswith("_base") or name.endswith("attn_sink"):
            return torch.zeros(shape, device=dev)
        if name.endswith("gate.bias"):
            return torch.rand(shape, generator=g, device=dev) * 0.2 - 0.1
        return torch.randn(shape, generator=g, device=dev) * self.std


# ----------------------------------------------------------------------------
# per-layer weights in storage format
# ----------------------------------------------------------------------------
@dataclass
class LayerWeights:
    kind: str
    ratio: int
    computes_topk: bool
    hc_attn: Tuple[torch.Tensor, torch.Tensor, torch.Tensor]
    hc_ffn: Tuple[torch.Tensor, torch.Tensor, torch.Tensor]
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor
    w_qa_kv: LinearWeight
    q_norm: torch.Tensor
    kv_norm: torch.Tensor
    w_qb: LinearWeight                     # [nh_local*D (+ ih*di on F-layers), q_lora]
    w_oa: List[LinearWeight]
    w_ob: LinearWeight
    sink: torch.Tensor
    sink_full: Optional[torch.Tensor] = None      # all heads' sinks (token-parallel attention under TP)
    w_oa_grouped: Optional[LinearWeight] = None   # the same groups stacked [G_l*o_lora, hpg*D] for one launch
    w_side: Optional[LinearWeight] = None  # bf16 [2cD (+ ih + 4di), H]: compressor | weights_proj | indexer compressor
    ape: Optional[torch.Tensor] = None
    comp_norm: Optional[torch.Tensor] = None
    iape: Optional[torch.Tensor] = None
    inorm: Optional[torch.Tensor] = None
    w_gate: Optional[LinearWeight] = None
    gate_bias: Optional[torch.Tensor] = None
    tid2eid: Optional[torch.Tensor] = None
    w_sh13: Optional[LinearWeight] = None
    w_sh2: Optional[LinearWeight] = None
    experts: Optional[M.ExpertWeights] = None
    experts_tp: Optional[M.ExpertWeights] = None          # all experts, 1/tp of each one's intermediate rows (decode steps)
    index: int = -1                        # layer number (load recording)
    eplb: Optional[Tuple[torch.Tensor, torch.Tensor]] = None   # (logical -> physical table, replica counts); None = identity


def _get(src: WeightSource, name: str, shape, device) -> torch.Tensor:
    return src.get(name, tuple(shape), device)


def build_experts(cfg: ModelConfig, src: WeightSource, prefix: str, device, tp_rank: int, tp_size: int,
                  placement=None) -> Tuple[M.ExpertWeights, Optional[Tuple[torch.Tensor, torch.Tensor]]]:
    """This rank's routed experts of one layer.  Without a placement rank r holds the logical experts
    [r*E/tp, (r+1)*E/tp); with one (parallel/eplb.py) it holds the logical experts of its physical slots, and the
    second result maps router ids to slot ids."""
    f = f"{prefix}.ffn"
    E, I, H = cfg.n_routed_experts, cfg.moe_intermediate_size, cfg.hidden_size
    if placement is None or placement.is_identity:
        e_l = E // tp_size
        logical = list(range(tp_rank * e_l, (tp_rank + 1) * e_l))
        start, tables = tp_rank * e_l, None
    else:
        logical = placement.local_logical(tp_rank)
        start, tables = tp_rank * placement.slots_per_rank, placement.tables(device)
    g = lambda n, s: _get(src, n, s, device)
    packs = []
    for e in logical:
        w13 = torch.cat([g(f"{f}.experts.{e}.w1.weight", (I, H)), g(f"{f}.experts.{e}.w3.weight", (I, H))], 0)
        w2 = g(f"{f}.experts.{e}.w2.weight", (H, I))
        packs.append(M.ExpertWeights.from_master(w13[None], w2[None], cfg.expert_dtype, device, 0))
    cat = lambda xs: torch.cat(xs, 0).contiguous() if xs[0] is not None else None
    ew = M.ExpertWeights(cat([p.w13 for p in packs]), cat([p.w2 for p in packs]), cat([p.s13 for p in packs]),
                         cat([p.s2 for p in packs]), cat([p.g13 for p in packs]), cat([p.g2 for p in packs]), start)
    return ew, tables


def build_experts_sliced(cfg: ModelConfig, src: WeightSource, prefix: str, device, tp_rank: int,
                         tp_size: int) -> M.ExpertWeights:
    """Every routed expert of one layer, cut along its intermediate dimension: rank r holds rows [r*I/tp, (r+1)*I/tp) of
    w1 / w3 and the matching columns of w2.  A decode step touches only top-k experts per token; with whole experts
    per rank the step waits for the rank that happens to hold most of them, with slices every rank streams the same
    bytes (1/tp of each selected expert) and the partial sums meet in the all-reduce that follows anyway."""
    f = f"{prefix}.ffn"
    E, I, H = cfg.n_routed_experts, cfg.moe_intermediate_size, cfg.hidden_size
    il = I // tp_size
    r0 = tp_rank * il
    g = lambda n, s: _get(src, n, s, device)
    packs = []
    for e in range(E):
        w13 = torch.cat([g(f"{f}.experts.{e}.w1.weight", (I, H))[r0:r0 + il], g(f"{f}.experts.{e}.w3.weight", (I, H))[r0:r0 + il]], 0)
        w2 = g(f"{f}.experts.{e}.w2.weight", (H, I))[:, r0:r0 + il].contiguous()
        packs.append(M.ExpertWeights.from_master(w13[None], w2[None], cfg.expert_dtype, device, 0))
    cat = lambda xs: torch.cat(xs, 0).contiguous() if xs[0] is not None else None
    return M.ExpertWeights(cat([p.w13 for p in packs]), cat([p.w2 for p in packs]), cat([p.s13 for p in packs]),
                           cat([p.s2 for p in packs]), cat([p.g13 for p in packs]), cat([p.g2 for p in packs]), 0)


def decode_expert_slices_wanted(cfg: ModelConfig, tp_size: int, device) -> bool:
    """Whether a second, sliced copy of the routed experts is kept for decode-sized steps (GPU, tensor parallel, NVFP4
    experts whose slices keep whole 32-value blocks; STK_MOE_DECODE_SLICED=0 switches it off)."""
    import os
    if os.environ.get("STK_MOE_DECODE_SLICED", "1") == "0" or tp_size <= 1 or torch.device(device).type != "cuda":
        return False
    return cfg.expert_dtype == "nvfp4" and cfg.moe_intermediate_size % (32 * tp_size) == 0


def build_layer(cfg: ModelConfig, src: WeightSource, prefix: str, li: int, device, tp_rank: int, tp_size: int,
                kind: Optional[str] = None, placement=None) -> LayerWeights:
    H, D, Rd, nh, hc = cfg.hidden_size, cfg.head_dim, cfg.qk_rope_head_dim, cfg.num_attention_heads, cfg.hc_mult
    dd = cfg.dense_dtype
    kind = kind or cfg.layer_kind(li)
    ratio = {"swa": 0, "c4a": 4, "c128a": 128}[kind]
    nh_l = nh // tp_size
    h0 = tp_rank * nh_l
    a = f"{prefix}.attn"
    # a checkpoint with power-of-two block scales is re-quantised with the same rule, which reproduces its codes
    ue8m0 = getattr(src, "fp8_scale_rule", "absmax") == "ue8m0"
    mk = lambda w: LinearWeight.from_master(w, dd, device, ue8m0)
    mkbf = lambda w: LinearWeight(w.to(device=device, dtype=BF16).contiguous())
    g = lambda n, s: _get(src, n, s, device)

    hc_attn = (g(f"{prefix}.hc_attn_fn", (cfg.mix_hc, hc * H)).to(F32).contiguous(),
               g(f"{prefix}.hc_attn_base", (cfg.mix_hc,)).to(F32), g(f"{prefix}.hc_attn_scale", (3,)).to(F32))
    hc_ffn = (g(f"{prefix}.hc_ffn_fn", (cfg.mix_hc, hc * H)).to(F32).contiguous(),
              g(f"{prefix}.hc_ffn_base", (cfg.mix_hc,)).to(F32), g(f"{prefix}.hc_ffn_scale", (3,)).to(F32))
    w_qa_kv = mk(torch.cat([g(f"{a}.wq_a.weight", (cfg.q_lora_rank, H)), g(f"{a}.wkv.weight", (D, H))], 0))
    wqb = g(f"{a}.wq_b.weight", (nh * D, cfg.q_lora_rank))[h0 * D:(h0 + nh_l) * D]
    computes = kind == "c4a" and index_cache_computes(cfg, li)
    if kind == "c4a" and computes:
        wqb = torch.cat([wqb, g(f"{a}.indexer.wq_b.weight", (cfg.index_n_heads * cfg.index_head_dim, cfg.q_lora_rank))], 0)
    G = cfg.o_groups
    hpg = nh // G
    woa_full = g(f"{a}.wo_a.weight", (G * cfg.o_lora_rank, hpg * D)).view(G, cfg.o_lora_rank, hpg * D)
    if tp_size <= G:
        g_l = G // tp_size
        groups = list(range(tp_rank * g_l, (tp_rank + 1) * g_l))
        w_oa = [mk(woa_full[gi]) for gi in groups]
        w_oa_grouped = None
        kbytes = hpg * D * (1 if dd == "fp8" else 2)
        if kbytes % 128 == 0 and cfg.o_lora_rank % 128 == 0:
            w_oa_grouped = LinearWeight(torch.cat([w.w for w in w_oa], 0).contiguous(),
                                        torch.cat([w.scale for w in w_oa], 0).contiguous() if dd == "fp8" else None)
        wob = g(f"{a}.wo_b.weight", (H, G * cfg.o_lora_rank))[:, groups[0] * cfg.o_lora_rank:(groups[-1] + 1) * cfg.o_lora_rank]
    else:
        raise NotImplementedError("tp_size > o_groups")
    lw = LayerWeights(
        kind=kind, ratio=ratio, computes_topk=computes, hc_attn=hc_attn, hc_ffn=hc_ffn,
        attn_norm=g(f"{prefix}.attn_norm.weight", (H,)).to(BF16), ffn_norm=g(f"{prefix}.ffn_norm.weight", (H,)).to(BF16),
        w_qa_kv=w_qa_kv, q_norm=g(f"{a}.q_norm.weight", (cfg.q_lora_rank,)).to(BF16),
        kv_norm=g(f"{a}.kv_norm.weight", (D,)).to(BF16), w_qb=mk(wqb), w_oa=w_oa, w_oa_grouped=w_oa_grouped, w_ob=mk(wob.contiguous()),
        sink=g(f"{a}.attn_sink", (nh,)).to(F32)[h0:h0 + nh_l].contiguous(),
        sink_full=g(f"{a}.attn_sink", (nh,)).to(F32).contiguous() if tp_size > 1 else None)
    if ratio:
        c = compressor_slots(ratio)
        side = [g(f"{a}.compressor.wkv.weight", (c * D, H)), g(f"{a}.compressor.wgate.weight", (c * D, H))]
        lw.ape = g(f"{a}.compressor.ape", (ratio, c * D)).to(F32).contiguous()
        lw.comp_norm = g(f"{a}.compressor.norm.weight", (D,)).to(BF16)
        if computes:
            di = cfg.index_head_dim
            side += [g(f"{a}.indexer.weights_proj.weight", (cfg.index_n_heads, H)),
                     g(f"{a}.indexer.compressor.wkv.weight", (2 * di, H)),
                     g(f"{a}.indexer.compressor.wgate.weight", (2 * di, H))]
            lw.iape = g(f"{a}.indexer.compressor.ape", (ratio, 2 * di)).to(F32).contiguous()
            lw.inorm = g(f"{a}.indexer.compressor.norm.weight", (di,)).to(BF16)
        lw.w_side = mkbf(torch.cat(side, 0))
    # ---- MoE ----
    f = f"{prefix}.ffn"
    E, I = cfg.n_routed_experts, cfg.moe_intermediate_size
    lw.w_gate = mkbf(g(f"{f}.gate.weight", (E, H)))
    if li < cfg.num_hash_layers:
        lw.tid2eid = (g(f"{f}.gate.tid2eid", (cfg.vocab_size, cfg.num_experts_per_tok)) % E).to(torch.int32).contiguous()
    else:
        lw.gate_bias = g(f"{f}.gate.bias", (E,)).to(F32)
    if cfg.n_shared_experts:
        Is = I * cfg.n_shared_experts
        isl = Is // tp_size
        r0 = tp_rank * isl
        w1 = g(f"{f}.shared_experts.w1.weight", (Is, H))[r0:r0 + isl]
        w3 = g(f"{f}.shared_experts.w3.weight", (Is, H))[r0:r0 + isl]
        lw.w_sh13 = mk(torch.cat([w1, w3], 0))
        lw.w_sh2 = mk(g(f"{f}.shared_experts.w2.weight", (H, Is))[:, r0:r0 + isl].contiguous())
    lw.experts, lw.eplb = build_experts(cfg, src, prefix, device, tp_rank, tp_size, placement)
    if decode_expert_slices_wanted(cfg, tp_size, device):
        lw.experts_tp = build_experts_sliced(cfg, src, prefix, device, tp_rank, tp_size)
    lw.index = li
    return lw


@dataclass
class ModelWeights:
    embed: torch.Tensor                 # bf16 [V, H] replicated
    head: LinearWeight                  # [V/tp, H]
    norm: torch.Tensor
    hc_head: Tuple[torch.Tensor, torch.Tensor, torch.Tensor]
    layers: List[LayerWeights]
    vocab_start: int = 0
    layer_offset: int = 0               # global index of layers[0] (a pipeline stage holds a contiguous range)


def build_model_weights(cfg: ModelConfig, src: WeightSource, device, tp_rank: int = 0, tp_size: int = 1,
                        head_fp8: bool = False, placements=None, layer_range: Optional[Tuple[int, int]] = None) -> ModelWeights:
    """placements: optional list of per-layer expert placements (parallel/eplb.py), None entries = identity.
    layer_range: (lo, hi) of a pipeline stage; only those layers are built (embedding, head and final norm are small
    next to them and are kept on every stage)."""
    H, V, hc = cfg.hidden_size, cfg.vocab_size, cfg.hc_mult
    g = lambda n, s: _get(src, n, s, device)
    vl = (V + tp_size - 1) // tp_size
    v0 = tp_rank * vl
    head = g("head.weight", (V, H))[v0:min(V, v0 + vl)]
    head_w = LinearWeight.from_master(head, "fp8", device) if head_fp8 else LinearWeight(head.to(BF16).contiguous())
    layers = [build_layer(cfg, src, f"layers.{li}", li, device, tp_rank, tp_size,
                          placement=placements[li] if placements is not None else None)
              for li in range(*(layer_range or (0, cfg.num_hidden_layers)))]
    return ModelWeights(
        embed=g("embed.weight", (V, H)).to(BF16).contiguous(), head=head_w, norm=g("norm.weight", (H,)).to(BF16),
        hc_head=(g("hc_head_fn", (hc, hc * H)).to(F32).contiguous(), g("hc_head_base", (hc,)).to(F32),
                 g("hc_head_scale", (1,)).to(F32)),
        layers=layers, vocab_start=v0, layer_offset=layer_range[0] if layer_range else 0)


# ----------------------------------------------------------------------------
# step inputs
# ----------------------------------------------------------------------------
@dataclass
class StepMeta:
    """Device-side description of one ragged step (decode rows and prefill chunks alike)."""
    token_ids: torch.Tensor        # [T] int64
    tok_req: torch.Tensor          # [T] int32 request row, -1 padding
    positions: torch.Tensor        # [T] int64, -1 padding
    first_pos: torch.Tensor        # [T] int32
    last_pos: torch.Tensor         # [T] int32
    swa_slot_mapping: torch.Tensor  # [T] int64 destination slot of each token's latent row
    swa_slots: torch.Tensor        # [T, W] int32 window rows
    swa_lens: torch.Tensor         # [T] int32
    max_comp_rows: int             # upper bound of compressed rows any request holds (c4 group)
    max_c128_rows: int = 0
    pure_decode: bool = False      # every request contributes exactly one token (no token attends to another new row)


def dcp_merge_candidates(gids: torch.Tensor, vals: torch.Tensor, k: int) -> torch.Tensor:
    """gids [T, n] int32 global row ids (-1 = no candidate), vals [T, n] fp32 scores (-inf for no candidate) -> the k best
    ids per row by (score descending, row ascending), -1 padded.  Two stable sorts, so equal scores resolve the same way
    on every rank and as on a rank that holds all rows (`runtime.planning.merge_topk_candidates` states the same rule)."""
    order = torch.sort(torch.where(gids >= 0, gids, torch.full_like(gids, 1 << 30)), dim=1, stable=True)[1]
    gids, vals = torch.gather(gids, 1, order), torch.gather(vals, 1, order)
    top, pos = torch.sort(vals, dim=1, descending=True, stable=True)
    ids = torch.gather(gids, 1, pos[:, :k])
    return torch.where(top[:, :k] > float("-inf"), ids, torch.full_like(ids, -1))


class DSV4Model:
    def __init__(self, cfg: ModelConfig, weights: ModelWeights, kv, comm=None, tp_rank: int = 0, tp_size: int = 1):
        self.cfg = cfg
        self.w = weights
        self.kv = kv
        self.comm = comm
        self.tp_rank, self.tp_size = tp_rank, tp_size
        dev = weights.embed.device
        self.device = dev
        self.inv = Fn.inv_freq(cfg.qk_rope_head_dim, cfg.rope_theta, dev)
        self.topk_buffer: Optional[torch.Tensor] = None     # IndexCache: shared by consecutive C4A layers
        self.pipe = None                                     # parallel.pipeline.PipeStage when the model is one stage of several
        self.pipe_defer = False                              # the engine exchanges a step's tokens when it finishes the step
        self.want_logprobs: Optional[int] = None             # set by the engine for a step that reports log-probabilities
        self.last_logprobs = None                            # (sampled token's, top values, top ids) of that step
        self.aux_layers: Tuple[int, ...] = ()
        self.aux_out: List[torch.Tensor] = []
        self.stats = {"sp_steps": 0, "mla_token_parallel_calls": 0, "dcp_topk_merges": 0}     # which paths ran (tests)
        # Decode context parallel (kv.dcp_size > 1): the ratio-4 caches hold every dcp_size-th page of each request.
        # A layer that computes top-k rows scores its own keys and the ranks merge their candidates; the selected
        # latent rows are then brought into a dense staging buffer on every rank (at most dcp_stage_bytes per call,
        # larger steps go in token blocks) and the attention kernels read that buffer like any paged cache.
        self._dcp_lt: Optional[torch.Tensor] = None
        self._dcp_stages: Dict[tuple, PagedCache] = {}
        self.dcp_stage_bytes = int(os.environ.get("STK_DCP_STAGE_MB", "64")) << 20
        self.load_recorder = None           # parallel.eplb.LoadRecorder when expert load is being recorded
        # Sequence-parallel indexer: with TP the indexer weights are replicated, so each rank scores only its
        # share of a large step's rows and the top-k rows are all-gathered (overlay/attention.py
        # `_indexer_sp_owned_ranges` in the reference; here every row of a step is split evenly, which is exact
        # because scoring and top-k are independent per row).
        self.indexer_sp = tp_size > 1 and comm is not None
        self.indexer_sp_min_rows = int(os.environ.get("STK_INDEXER_SP_MIN_ROWS", "8"))
        # fp32 indexer scores of one scoring call stay below this many bytes (query sub-chunks at long contexts)
        self.indexer_logits_bytes = int(os.environ.get("STK_INDEXER_MAX_LOGITS_MB", "512")) << 20
        # Token-parallel sparse attention: every rank holds the whole latent KV cache, and gathering a token's
        # top-k rows costs the same for 8 heads as for 64, so with heads split over the ranks the gather work is
        # replicated.  Large steps instead exchange q (all-to-all: heads -> tokens), attend with all heads for 1/tp of
        # the tokens, and exchange the output back (tokens -> heads).  Measured: with 32 heads per rank (2 GPUs) the
        # tensor-core kernel's time follows heads x tokens (its softmax warps set the pace) and the exchange buys
        # nothing; with 8 heads per rank (8 GPUs) a 4096-token chunk costs 2.06 ms against 2.93 ms for all 64 heads on
        # one GPU, i.e. the gather dominates and 1/8 of the tokens with all heads is ~5x less work.  Default: on for
        # steps of >= 1024 tokens when a rank holds at most 16 heads.
        # Sequence-parallel residual for large steps: the hyper-connection streams [T, hc, H] (and with them the mHC
        # mixing, norms and residual adds, which are per token) live on 1/tp of the tokens per rank; a sub-block's
        # input is all-gathered and its row-parallel output reduce-scattered (together the volume of the all-reduce
        # they replace), so that work is no longer repeated on every rank.
        self.sp_min_rows = int(os.environ.get("STK_SEQ_PARALLEL_MIN_ROWS", "1024")) if (tp_size > 1 and comm is not None) else 0
        nh_local = cfg.num_attention_heads // max(1, tp_size)
        self.mla_tp_min_rows = int(os.environ.get("STK_MLA_TP_MIN_ROWS", "1024" if nh_local <= 16 else "0"))
        # Decode-sized steps are a chain of launches that each fill a fraction of the GPU: independent branches of a
        # sub-block (compressor state update and KV insert beside the q / indexer chain, the shared expert beside the
        # router) run on a second stream, also inside captured graphs, so the chain gets shorter.
        self.fork_max_t = int(os.environ.get("STK_FORK_MAX_T", "64")) if dev.type == "cuda" else 0
        self.side_stream = torch.cuda.Stream(dev) if self.fork_max_t > 0 else None
        self.kv_stream = torch.cuda.Stream(dev) if self.fork_max_t > 0 else None     # latent-row insert, beside wq_b
        # Decode-sized steps fold neighbouring launches into the weight-streaming projections (q/kv norms into the
        # consumers, the router into the gate projection) and, under tensor parallelism, the two all-reduces of a layer
        # into the kernels on either side of them (`_ll`).  STK_DECODE_FUSE=0 restores the separate launches;
        # STK_LL_LOOPBACK=1 runs the folded all-reduce protocol on a single GPU (one rank, nothing to add).
        self.decode_fuse = dev.type == "cuda" and os.environ.get("STK_DECODE_FUSE", "1") == "1"
        self._ll_loop = None
        if dev.type == "cuda" and tp_size == 1 and os.environ.get("STK_LL_LOOPBACK", "0") == "1":
            from ..parallel.symm import LLExchange
            self._ll_loop = LLExchange.loopback(dev, 64 * cfg.hidden_size // 2)

    # ---- collectives ----------------------------------------------------------
    def _all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_size == 1 or self.comm is None:
            return x
        return self.comm.all_reduce(x)

    def _ll(self, t: int, h: int):
        """The folded all-reduce for a decode-sized [t, h] row-parallel output, or None (then the output is reduced by
        the GEMM epilogue / the all-reduce kernels)."""
        if not self.decode_fuse or t > Fn.SKINNY_MAX_T:
            return None
        if self._ll_loop is not None:
            return self._ll_loop if self._ll_loop.fits(t, h) else None
        if self.tp_size == 1 or self.comm is None or getattr(self.comm, "symm", None) is None or not self.comm.fuse_gemm:
            return None
        return self.comm.symm.ll_exchange(t, h)

    def _ll_any(self, words: int):
        """The folded exchange for `words` 8-byte words regardless of the step size, or None."""
        if not self.decode_fuse:
            return None
        if self.tp_size == 1 or self.comm is None or getattr(self.comm, "symm", None) is None or not self.comm.fuse_gemm:
            return None
        sy = self.comm.symm
        return sy.ll if (sy.enabled and words <= sy.ll.words) else None

    def _gemm_ar_ctx(self, t: int, n: int):
        """Symmetric context when the row-parallel GEMM can all-reduce in its own epilogue."""
        if self.tp_size == 1 or self.comm is None or getattr(self.comm, "symm", None) is None or not self.device.type == "cuda":
            return None
        if not self.comm.fuse_gemm:
            return None
        return self.comm.symm.gemm_ctx(t, n)

    # ---- attention sub-block ---------------------------------------------------
    def attention(self, li: int, lw: LayerWeights, y: torch.Tensor, yq, meta: StepMeta, causal_meta=None,
                  scatter: bool = False) -> torch.Tensor:
        """scatter: return this rank's 1/tp of the token rows of the reduced output (reduce-scatter) instead of all
        rows (all-reduce)."""
        cfg = self.cfg
        T = y.shape[0]
        D, Rd = cfg.head_dim, cfg.qk_rope_head_dim
        nh_l = cfg.num_attention_heads // self.tp_size
        ql = cfg.q_lora_rank
        fork = bool(lw.ratio) and self.side_stream is not None and 0 < T <= self.fork_max_t
        ev_in = torch.cuda.current_stream().record_event() if fork else None
        qkv = Fn.linear(yq if yq is not None else y, lw.w_qa_kv, tag="qa_kv")
        can_fork = self.side_stream is not None and 0 < T <= self.fork_max_t
        ev_qkv = torch.cuda.current_stream().record_event() if can_fork else None
        use_q = lw.w_qb.is_fp8 and Fn.wants_quant_act(T, y.device)
        fuse_norms = self.decode_fuse and T <= Fn.SKINNY_MAX_T and not use_q
        if fuse_norms:
            # no norm launch: the q_lora row is normalised inside the wq_b projection, the kv row inside the cache insert
            kvn, kv_norm_w = qkv[:, ql:], lw.kv_norm
            qb = Fn.linear(qkv[:, :ql], lw.w_qb, tag="qb", norm=(lw.q_norm, cfg.rms_norm_eps))
        else:
            res = Fn.rms_norm_pair(qkv[:, :ql], lw.q_norm, qkv[:, ql:], lw.kv_norm, cfg.rms_norm_eps, quant0=use_q, tag="qr")
            qr, kvn, kv_norm_w = res[0], res[1], None
            qb = Fn.linear(res[2] if use_q else qr, lw.w_qb, tag="qb")

        # decode-sized steps: the attention kernel norms and rotates q as it loads it, so only the latent row is written
        q_in_mla = (fuse_norms and A.USE_DECODE_MLA and T <= A.MLA_DECODE_MAX_T and nh_l % 8 == 0 and D == 512
                    and Rd == 64 and self.kv.swa_cache[li].fp8)

        # ... and on pure-decode steps it also builds and inserts the token's own latent row: no insert launch at all
        kv_in_mla = q_in_mla and meta.pure_decode and meta.swa_slot_mapping.dtype == torch.int64

        def kv_insert():
            qv = qb[:, :nh_l * D].view(T, nh_l, D)
            if kv_in_mla:
                return qv
            if q_in_mla:
                C.q_rope_kv_insert(None, kvn, meta.positions, meta.swa_slot_mapping, self.inv, self.kv.swa_cache[li],
                                   cfg.rms_norm_eps, kv_norm_w=kv_norm_w)
                return qv
            return C.q_rope_kv_insert(qv, kvn, meta.positions, meta.swa_slot_mapping,
                                      self.inv, self.kv.swa_cache[li], cfg.rms_norm_eps, kv_norm_w=kv_norm_w)

        topk_slots = topk_lens = None
        comp_cache = None
        ev_done = None
        if not lw.ratio:
            if kv_in_mla:
                q = kv_insert()
            elif q_in_mla and can_fork:
                # the latent row needs only the kv half of the projection: it is written beside the wq_b projection
                with side_branch(self.kv_stream, "kv"):
                    self.kv_stream.wait_event(ev_qkv)
                    q = kv_insert()
                    ev_done = self.kv_stream.record_event()
            else:
                q = kv_insert()
        else:
            c = compressor_slots(lw.ratio)
            ncomp = 2 * c * D
            grp = self.kv.c4 if lw.kind == "c4a" else self.kv.c128
            comp_cache = self.kv.comp_cache[li]
            computes = lw.kind == "c4a" and lw.computes_topk
            dcp = lw.kind == "c4a" and self.kv.dcp_size > 1
            ih = cfg.index_n_heads

            def compress_main(side):
                C.compress_windows(side[:, :ncomp], lw.ape, lw.comp_norm,
                                   self.inv, meta.positions, meta.tok_req, meta.first_pos, meta.last_pos,
                                   self.kv.comp_state[li], grp.table_dev, comp_cache, lw.ratio, c, cfg.rms_norm_eps)

            def compress_idx(side):
                C.compress_windows(side[:, ncomp + ih:], lw.iape, lw.inorm, self.inv, meta.positions,
                                   meta.tok_req, meta.first_pos, meta.last_pos, self.kv.idx_state[li],
                                   grp.table_dev, self.kv.idx_cache[li], lw.ratio, 2, cfg.rms_norm_eps)

            ev_side = ev_idx = ev_kv = None
            early_slots = None
            if fork:
                # side stream: side projection -> indexer-key compressor -> KV compressor -> q rope + SWA insert;
                # this stream keeps the q / indexer scoring chain and waits where it needs the other's results
                main, sd = torch.cuda.current_stream(), self.side_stream
                ev_qb = main.record_event()
                with side_branch(sd):
                    sd.wait_event(ev_in)       # y is ready: the branch starts beside the qa/kv projection
                    if (lw.kind == "c4a" and not computes and not dcp and self.topk_buffer is not None
                            and self.topk_buffer.shape[0] >= T):
                        # a layer that reuses the shared top-k rows only translates them to its own cache's slots:
                        # nothing of this layer is needed for that
                        early_slots = A.topk_to_slots(self.topk_buffer[:T], grp.table_dev, meta.tok_req,
                                                      grp.max_pages_per_req * C.PAGE, tag=f"topk")
                    side = Fn.linear(y, lw.w_side, out_dtype=F32, tag="side")
                    ev_side = sd.record_event()
                    if computes:
                        compress_idx(side)
                        ev_idx = sd.record_event()
                    compress_main(side)
                    if not q_in_mla:
                        sd.wait_event(ev_qb)
                        q = kv_insert()
                    ev_done = sd.record_event()
                if kv_in_mla:
                    q = kv_insert()
                elif q_in_mla:
                    # the latent row needs only the kv half of the first projection: its own branch, beside wq_b and
                    # not queued behind the compressors
                    with side_branch(self.kv_stream, "kv"):
                        self.kv_stream.wait_event(ev_qkv)
                        q = kv_insert()
                        ev_kv = self.kv_stream.record_event()
            else:
                q = kv_insert()
                side = Fn.linear(y, lw.w_side, out_dtype=F32, tag="side")
                compress_main(side)
            if lw.kind == "c4a":
                K = cfg.index_topk
                if self.topk_buffer is None or self.topk_buffer.shape[0] < T:
                    self.topk_buffer = torch.full((max(T, 16), K), -1, dtype=torch.int32, device=y.device)
                if computes:
                    di = cfg.index_head_dim
                    qi = qb[:, nh_l * D:].view(T, ih, di)
                    if fork:
                        torch.cuda.current_stream().wait_event(ev_side)
                    wi = side[:, ncomp:ncomp + ih]
                    quant = cfg.kv_cache_dtype == "fp8_ds_mla"
                    qq, wf = C.indexer_q_prep(qi, wi, meta.positions, self.inv, Rd, quant, fmt=cfg.indexer_dtype)
                    if fork:
                        torch.cuda.current_stream().wait_event(ev_idx)
                    else:
                        compress_idx(side)
                    nv = A.compressed_valid(meta.positions, lw.ratio)
                    n_rows = max(meta.max_comp_rows, 1)

                    def score_topk(a0: int, a1: int, out: torch.Tensor) -> None:
                        """Rows [a0, a1) of the step -> their top-k ids in out[: a1 - a0], in query sub-chunks that
                        keep the fp32 score matrix inside the logits budget (overlay/indexer.py:92-143,301-319: here
                        the scorer reads the paged K rows in place, so only the logits budget applies)."""
                        for _, qs in split_indexer_prefill_chunks([n_rows], [a1 - a0], 1 << 62, self.indexer_logits_bytes):
                            b0, b1 = a0 + qs.start, a0 + qs.stop
                            sc = A.indexer_scores(qq[b0:b1], wf[b0:b1], self.kv.idx_cache[li], grp.table_dev,
                                                  meta.tok_req[b0:b1], nv[b0:b1], n_rows)
                            A.topk_rows(sc, nv[b0:b1], K, out=out[qs.start:qs.stop])

                    if dcp:
                        self._dcp_score_topk(li, qq, wf, nv, n_rows, grp, meta, K)
                    elif self.indexer_sp and T >= self.indexer_sp_min_rows * self.tp_size:
                        sizes = sp_gather_sizes((0, T), self.tp_size)           # ceil split, the last ranks may be short
                        shard = sizes[0]
                        a0 = sum(sizes[:self.tp_rank])
                        part = torch.full((shard, K), -1, dtype=torch.int32, device=y.device)
                        if sizes[self.tp_rank] > 0:
                            score_topk(a0, a0 + sizes[self.tp_rank], part)
                        self.topk_buffer[:T] = self.comm.all_gather_dim0(part)[:T]
                    else:
                        score_topk(0, T, self.topk_buffer)
                if dcp:
                    topk_slots = topk_lens = None           # staged per token block below
                elif early_slots is not None:
                    topk_slots, topk_lens = early_slots
                else:
                    topk_slots, topk_lens = A.topk_to_slots(self.topk_buffer[:T], grp.table_dev, meta.tok_req,
                                                            grp.max_pages_per_req * C.PAGE, tag=f"topk")
            else:
                topk_slots, topk_lens = A.c128_indices(meta.positions, meta.tok_req, grp.table_dev, lw.ratio,
                                                       cfg.index_topk)
        if ev_done is not None:
            torch.cuda.current_stream().wait_event(ev_done)
        if lw.ratio and ev_kv is not None:
            torch.cuda.current_stream().wait_event(ev_kv)
        with span("sparse_mla", T):
            if lw.ratio and dcp:
                o = self._dcp_sparse_mla(li, lw, q, meta, grp, q_in_mla, kv_in_mla, kvn, kv_norm_w)
            elif (self.tp_size > 1 and self.comm is not None and lw.sink_full is not None and self.mla_tp_min_rows > 0
                    and T >= self.mla_tp_min_rows):
                o = self._mla_token_parallel(li, lw, q, meta, comp_cache, topk_slots, topk_lens)
            else:
                o = A.sparse_mla(q, self.kv.swa_cache[li], meta.swa_slots, meta.swa_lens, comp_cache, topk_slots,
                                 topk_lens, lw.sink, D ** -0.5, inv_rope=(meta.positions, self.inv),
                                 q_prep=(meta.positions, self.inv, cfg.rms_norm_eps) if q_in_mla else None,
                                 kv_insert=(kvn, kv_norm_w, meta.swa_slot_mapping) if kv_in_mla else None)
        # grouped low-rank output projection, then the row-parallel wo_b (+ all-reduce)
        G_l = len(lw.w_oa)
        hpg = cfg.num_attention_heads // cfg.o_groups
        og = o.view(T, G_l, hpg * D)
        if lw.w_oa_grouped is not None:
            z = Fn.linear(o.view(T, G_l * hpg * D), lw.w_oa_grouped, tag="oa", groups=G_l)
        else:
            z = torch.empty(T, G_l * cfg.o_lora_rank, dtype=o.dtype, device=y.device)
            for gi, wg in enumerate(lw.w_oa):
                Fn.linear(og[:, gi], wg, out=z[:, gi * cfg.o_lora_rank:(gi + 1) * cfg.o_lora_rank], tag=f"oa")
        with span("o_proj_b+allreduce", T):
            if scatter:
                return self.comm.reduce_scatter_dim0(Fn.linear(z, lw.w_ob, tag="ob"))
            ll = self._ll(T, cfg.hidden_size)
            if ll is not None:
                return Fn.linear(z, lw.w_ob, tag="ob", ll=ll)          # an LLPending: the next mHC kernel adds the ranks
            ar = self._gemm_ar_ctx(T, cfg.hidden_size)
            out = Fn.linear(z, lw.w_ob, tag="ob", ar_ctx=ar)
            return out if ar is not None else self._all_reduce(out)

    # ---- decode context parallel: ratio-4 rows dealt page by page over the ranks -----------------------------------
    def _dcp_local_table(self, grp) -> torch.Tensor:
        if self._dcp_lt is None:
            self._dcp_lt = grp.local_table()
        return self._dcp_lt

    def _dcp_score_topk(self, li: int, qq, wf, nv: torch.Tensor, n_rows: int, grp, meta: StepMeta, K: int) -> None:
        """Every rank scores the indexer keys it stores, keeps its K best (score, global row) pairs per token, and
        the ranks' lists are gathered and merged into the global top-k (overlay/ops_cache_utils.py:472-503,557-617
        interleaved KV; probes/sai_probe.py:1065-1146 cross-rank candidate merge).  Writes self.topk_buffer[:T]."""
        r, n = self.kv.dcp_rank, self.kv.dcp_size
        T = qq.shape[0]
        nv_l = dcp_local_rows(nv, n, r, PAGE).to(torch.int32)           # rows of each token's first nv that live here
        rows_l = (n_rows // (PAGE * n) + 1) * PAGE
        lt = self._dcp_local_table(grp)
        cand = torch.empty(T, 2, K, dtype=torch.int32, device=qq.device)
        ninf = float("-inf")
        for _, qs in split_indexer_prefill_chunks([rows_l], [T], 1 << 62, self.indexer_logits_bytes):
            b0, b1 = qs.start, qs.stop
            sc = A.indexer_scores(qq[b0:b1], wf[b0:b1], self.kv.idx_cache[li], lt, meta.tok_req[b0:b1], nv_l[b0:b1], rows_l)
            ids = A.topk_rows(sc, nv_l[b0:b1], K)
            ok = ids >= 0
            val = torch.gather(sc, 1, ids.clamp(min=0).long())
            cand[b0:b1, 1] = torch.where(ok, val, torch.full_like(val, ninf)).contiguous().view(torch.int32)
            gid = dcp_global_row(ids, n, r, PAGE)
            cand[b0:b1, 0] = torch.where(ok, gid, torch.full_like(gid, -1))
        allc = self.comm.all_gather_dim0(cand).view(n, T, 2, K)
        gids = allc[:, :, 0].permute(1, 0, 2).reshape(T, n * K)
        vals = allc[:, :, 1].permute(1, 0, 2).reshape(T, n * K).view(torch.float32)
        self.topk_buffer[:T] = dcp_merge_candidates(gids, vals, K)
        self.stats["dcp_topk_merges"] += 1

    def _dcp_stage(self, li: int, ids: torch.Tensor, tok_req: torch.Tensor, grp):
        """ids [t, K] global ratio-4 row ids (-1 padded) -> (cache, slots, lens): a dense paged buffer that holds
        row ids[i, j] at slot i * K + j.  Every rank fills in the rows it stores and the ranks' buffers are added
        (one writer per row), so each selected row crosses the links once and attention reads local memory."""
        r, n = self.kv.dcp_rank, self.kv.dcp_size
        cache = self.kv.comp_cache[li]
        t, K = ids.shape
        db = cache.data_bytes
        sb = KV_SCALE_BYTES if cache.fp8 else 0
        ok = ids >= 0
        idl = ids.clamp(min=0).long()
        mine = ok & (dcp_owner(idl, n, PAGE) == r)
        # this rank's own numbering of its rows: page = local index // PAGE of the local block table
        phys = self._dcp_local_table(grp)[tok_req.clamp(min=0).long()[:, None], dcp_local_index(idl, n, PAGE) // PAGE].long()
        phys = torch.where(mine, phys, torch.zeros_like(phys)).clamp(min=0)
        rr = idl % PAGE
        rows = t * K
        pages = -(-rows // PAGE)
        key = (pages, db, sb)
        stage = self._dcp_stages.get(key)
        if stage is None:
            stage = self._dcp_stages[key] = PagedCache.allocate(pages, cache.dim, cache.rope_dim, cache.fp8, cache.kind,
                                                                ids.device)
        flat = torch.arange(rows, device=ids.device)
        dst_pg, dst_r = flat // PAGE, flat % PAGE
        m = mine.view(rows, 1)
        for off, width in ((0, db), (PAGE * db, sb)):
            if width == 0:
                continue
            src = cache.buf[:, off:off + PAGE * width].view(cache.num_pages, PAGE, width)[phys, rr].view(rows, width)
            dst = stage.buf[:, off:off + PAGE * width].view(pages, PAGE, width)
            dst[dst_pg, dst_r] = torch.where(m, src, torch.zeros_like(src))
        self.comm.all_reduce(stage.buf.view(torch.int32))
        slots = torch.where(ok, flat.view(t, K), torch.full_like(idl, -1)).to(torch.int32)
        return stage, slots, ok.sum(1).to(torch.int32)

    def _dcp_sparse_mla(self, li: int, lw: LayerWeights, q, meta: StepMeta, grp, q_in_mla: bool, kv_in_mla: bool, kvn,
                        kv_norm_w) -> torch.Tensor:
        cfg = self.cfg
        T, D = q.shape[0], cfg.head_dim
        K = cfg.index_topk
        cache = self.kv.comp_cache[li]
        row_bytes = cache.data_bytes + (KV_SCALE_BYTES if cache.fp8 else 0)
        step = max(1, self.dcp_stage_bytes // (K * row_bytes))
        if T <= step:
            cc, ts, tl = self._dcp_stage(li, self.topk_buffer[:T], meta.tok_req, grp)
            return A.sparse_mla(q, self.kv.swa_cache[li], meta.swa_slots, meta.swa_lens, cc, ts, tl, lw.sink, D ** -0.5,
                                inv_rope=(meta.positions, self.inv),
                                q_prep=(meta.positions, self.inv, cfg.rms_norm_eps) if q_in_mla else None,
                                kv_insert=(kvn, kv_norm_w, meta.swa_slot_mapping) if kv_in_mla else None)
        # a prefill chunk: token blocks small enough for the staging budget
        o = torch.empty_like(q)
        for a in range(0, T, step):
            sl = slice(a, min(T, a + step))
            cc, ts, tl = self._dcp_stage(li, self.topk_buffer[sl], meta.tok_req[sl], grp)
            o[sl] = A.sparse_mla(q[sl], self.kv.swa_cache[li], meta.swa_slots[sl], meta.swa_lens[sl], cc, ts, tl, lw.sink,
                                 D ** -0.5, inv_rope=(meta.positions[sl], self.inv))
        return o

    def _mla_token_parallel(self, li: int, lw: LayerWeights, q: torch.Tensor, meta: StepMeta, comp_cache, topk_slots,
                            topk_lens) -> torch.Tensor:
        """q [T, nh_local, D] -> o [T, nh_local, D], computed as all heads of this rank's share of the tokens."""
        tp, r = self.tp_size, self.tp_rank
        self.stats["mla_token_parallel_calls"] += 1
        T, nh_l, D = q.shape
        share = -(-T // tp)
        sizes = [max(0, min(T, (s + 1) * share) - min(T, s * share)) for s in range(tp)]
        a0, mine = min(T, r * share), sizes[r]
        # heads -> tokens: block s of the result holds head block s of my tokens
        recv = self.comm.all_to_all_dim0(q, sizes, [mine] * tp)
        if mine > 0:
            q_seq = recv.view(tp, mine, nh_l, D).permute(1, 0, 2, 3).reshape(mine, tp * nh_l, D)
            sl = slice(a0, a0 + mine)
            o_seq = A.sparse_mla(q_seq, self.kv.swa_cache[li], meta.swa_slots[sl], meta.swa_lens[sl], comp_cache,
                                 topk_slots[sl] if topk_slots is not None else None,
                                 topk_lens[sl] if topk_lens is not None else None, lw.sink_full, D ** -0.5,
                                 inv_rope=(meta.positions[sl], self.inv))
            send = o_seq.view(mine, tp, nh_l, D).permute(1, 0, 2, 3).reshape(tp * mine, nh_l, D)
        else:
            send = q.new_zeros(0, nh_l, D)
        # tokens -> heads: block s of the result holds my head block of rank s's tokens
        return self.comm.all_to_all_dim0(send, [mine] * tp, sizes)

    # ---- MoE sub-block ----------------------------------------------------------
    def moe(self, lw: LayerWeights, y: torch.Tensor, yq, meta: StepMeta, scatter: bool = False) -> torch.Tensor:
        cfg = self.cfg
        T = y.shape[0]
        fork = self.side_stream is not None and 0 < T <= self.fork_max_t and lw.w_sh13 is not None
        if fork:
            # the shared expert (two launches) runs beside the gate projection, the router and the routed experts
            main, sd = torch.cuda.current_stream(), self.side_stream
            ev_in = main.record_event()
            with side_branch(sd):
                sd.wait_event(ev_in)
                shared = self._shared_expert(lw, y, yq)
                ev_sh = sd.record_event()
        routed = None
        if self.decode_fuse and T <= Fn.SKINNY_MAX_T:
            routed = Fn.gate_route(y, lw.w_gate, lw.gate_bias, cfg.num_experts_per_tok, cfg.scoring_func, cfg.norm_topk_prob,
                                   cfg.routed_scaling_factor, lw.tid2eid, meta.token_ids)
        if routed is None:
            logits = Fn.linear(y, lw.w_gate, out_dtype=F32, tag="gate")
            routed = M.router(logits, lw.gate_bias, cfg.num_experts_per_tok, cfg.scoring_func, cfg.norm_topk_prob,
                              cfg.routed_scaling_factor, lw.tid2eid, meta.token_ids)
        ids, wts = routed
        if self.load_recorder is not None and lw.index >= 0:
            self.load_recorder.record(lw.index, ids)                   # logical ids: what a rebalance needs
        # decode-sized steps: every rank computes its slice of every selected expert (balanced by construction);
        # larger steps: whole experts per rank
        experts = lw.experts
        if lw.experts_tp is not None and not scatter and T * ids.shape[1] <= M.DIRECT_MAX_PAIRS:
            experts = lw.experts_tp
        elif lw.eplb is not None:
            from ..parallel.eplb import to_physical
            ids = to_physical(ids, *lw.eplb)                           # one replica per pair, round-robin by token
        if not fork:
            shared = self._shared_expert(lw, y, yq)
        ll = None if scatter or not (y.is_cuda and experts.is_fp4) else self._ll(T, cfg.hidden_size)
        out = M.moe_experts(y, ids, wts, experts, cfg.swiglu_limit, shared, cfg.n_routed_experts,
                            shared_ready=ev_sh if fork else None, ll=ll)
        if ll is not None:
            return out                                                  # an LLPending
        return self.comm.reduce_scatter_dim0(out) if scatter else self._all_reduce(out)

    def _shared_expert(self, lw: LayerWeights, y: torch.Tensor, yq) -> Optional[torch.Tensor]:
        cfg = self.cfg
        if lw.w_sh13 is None:
            return None
        act = Fn.linear_swiglu(y, lw.w_sh13, cfg.swiglu_limit) if yq is None else None
        if act is not None:
            return Fn.linear(act, lw.w_sh2, tag="sh2")
        gu = Fn.linear(yq if (yq is not None and lw.w_sh13.is_fp8) else y, lw.w_sh13, tag="sh13")
        if lw.w_sh2.is_fp8 and Fn.wants_quant_act(y.shape[0], y.device):
            _, aq = Fn.swiglu_clamp(gu, cfg.swiglu_limit, quant=True, tag="shact")
            return Fn.linear(aq, lw.w_sh2, tag="sh2")
        return Fn.linear(Fn.swiglu_clamp(gu, cfg.swiglu_limit), lw.w_sh2, tag="sh2")

    def layer(self, li: int, lw: LayerWeights, X: torch.Tensor, meta: StepMeta, pend=None, defer: bool = False,
              sp: bool = False):
        """One decoder layer.  `pend` = (sub-block output, streams, post, comb) left unmixed by the previous layer: its
        post-mix runs inside this layer's first pre-mix.  With `defer` the layer returns such a tuple instead of the
        mixed streams.  With `sp` X holds this rank's 1/tp of the token rows (sequence-parallel residual)."""
        cfg = self.cfg
        n = X.shape[0]
        want_q = not sp and lw.w_qa_kv.is_fp8 and Fn.wants_quant_act(n, X.device)
        hc_args = (cfg.rms_norm_eps, cfg.hc_eps, cfg.hc_sinkhorn_iters)
        if pend is None:
            r = Fn.mhc_pre(X, *lw.hc_attn, lw.attn_norm, *hc_args, quant=want_q, tag="mhc_a")
        else:
            X, r = Fn.mhc_post_pre(*pend, *lw.hc_attn, lw.attn_norm, *hc_args, quant=want_q, tag="mhc_a")
        y, post, comb = r[0], r[1], r[2]
        if sp:
            y = self.comm.all_gather_dim0(y)
        with span("attention", n):
            a = self.attention(li, lw, y, r[3] if want_q else None, meta, scatter=sp)
        want_q = not sp and lw.w_sh13 is not None and lw.w_sh13.is_fp8 and Fn.wants_quant_act(n, X.device)
        X, r = Fn.mhc_post_pre(a, X, post, comb, *lw.hc_ffn, lw.ffn_norm, *hc_args, quant=want_q, tag="mhc_f")
        y, post, comb = r[0], r[1], r[2]
        if sp:
            y = self.comm.all_gather_dim0(y)
        with span("moe", n):
            f = self.moe(lw, y, r[3] if want_q else None, meta, scatter=sp)
        if defer:
            return f, X, post, comb
        return Fn.mhc_post(f, X, post, comb)

    # ---- whole model -------------------------------------------------------------
    def forward_hidden(self, meta: StepMeta) -> torch.Tensor:
        """-> final residual streams [T, hc, H]."""
        cfg = self.cfg
        T = meta.token_ids.shape[0]
        self._dcp_lt = None                  # the block tables may have changed since the last step
        sp = (self.sp_min_rows > 0 and T >= self.sp_min_rows and T % self.tp_size == 0 and not self.aux_layers)
        ids = meta.token_ids
        if sp:
            self.stats["sp_steps"] += 1
            share = T // self.tp_size
            ids = ids[self.tp_rank * share:(self.tp_rank + 1) * share]
        pipe = self.pipe
        lo = self.w.layer_offset
        hi = lo + len(self.w.layers)
        if pipe is None or pipe.first:
            X = Fn.embed_hc(ids, self.w.embed, cfg.hc_mult, cfg.vocab_size)
        else:
            # the streams of this step from the previous stage (its share of the rows when the residual is sharded),
            # and the shared top-k rows when this stage begins inside an IndexCache group
            from ..parallel.pipeline import stage_starts_inside_index_group
            X = pipe.recv_prev((ids.shape[0], cfg.hc_mult, cfg.hidden_size), Fn.cpu_act_dtype() if not ids.is_cuda else BF16,
                               ids.device)
            if stage_starts_inside_index_group(cfg, lo, hi):
                self.topk_buffer = pipe.recv_prev((max(T, 16), cfg.index_topk), torch.int32, ids.device)
        self.aux_out = []
        pend = None
        last = hi - 1
        for idx, lw in enumerate(self.w.layers):
            li = lo + idx
            defer = li != last and li not in self.aux_layers
            out = self.layer(li, lw, X, meta, pend, defer, sp)
            if defer:
                pend, X = out, out[1]
            else:
                pend, X = None, out
            if li in self.aux_layers:
                self.aux_out.append(X.float().mean(1).to(X.dtype))
        if pipe is not None and not pipe.last:
            from ..parallel.pipeline import stage_starts_inside_index_group
            pipe.send_next(X)
            nlo, nhi = pp_layer_range(cfg.num_hidden_layers, pipe.pp_size, pipe.pp_rank + 1)
            if stage_starts_inside_index_group(cfg, nlo, nhi):
                tb = self.topk_buffer
                if tb is None or tb.shape[0] < max(T, 16):
                    tb = torch.full((max(T, 16), cfg.index_topk), -1, dtype=torch.int32, device=X.device)
                pipe.send_next(tb[:max(T, 16)])
            return X
        if sp:
            X = self.comm.all_gather_dim0(X)
        return X

    def head_hidden(self, X: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        h = Fn.hc_head(X, *self.w.hc_head, cfg.rms_norm_eps, cfg.hc_eps)
        return Fn.rms_norm(h, self.w.norm, cfg.rms_norm_eps)

    def compute_logits(self, h: torch.Tensor) -> torch.Tensor:
        """h [n, H] -> logits [n, V] (vocab shards gathered across ranks)."""
        lg = Fn.linear(h, self.w.head, tag="head")
        if self.tp_size > 1 and self.comm is not None:
            lg = self.comm.all_gather_last_dim(lg)[:, :self.cfg.vocab_size]
        return lg

    def sample(self, h: torch.Tensor, temp: torch.Tensor, seed: torch.Tensor, pos: torch.Tensor,
               top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
               agreed_status: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Head hidden states [n, H] -> sampled tokens [n] (seeded Gumbel arg-max).  Under tensor parallelism the
        logits stay sharded: every rank takes the noisy arg-max of its vocabulary shard and the ranks exchange one
        candidate per row (no logits all-gather); truncated sampling (top-k / top-p) needs the whole row and gathers."""
        from ..ops import sampling as S
        n = h.shape[0]
        if self.want_logprobs is not None:
            # log-probabilities asked for: the whole rows are needed anyway (gathered across ranks); the token is the one
            # the sharded arg-max would pick (same noise, same logits)
            lg = self.compute_logits(h)
            toks, _ = S.gumbel_argmax(lg, temp, seed, pos, top_k=top_k, top_p=top_p)
            lp = torch.log_softmax(lg.float(), dim=-1)
            top_lp, top_ids = lp.topk(max(1, min(self.want_logprobs, lp.shape[1])), dim=-1)
            self.last_logprobs = (lp.gather(1, toks.view(-1, 1).long()).squeeze(1), top_lp, top_ids)
            return toks
        ll = None
        if self.tp_size > 1 and top_k is None and top_p is None and h.is_cuda and n <= 256:
            ll = self._ll_any(3 * n)
        if ll is not None:
            lg = Fn.linear(h, self.w.head, tag="head")
            toks, _ = S.gumbel_argmax(lg, temp, seed, pos, vocab_start=self.w.vocab_start, ll=ll, agreed_status=agreed_status)
            return toks
        toks, _ = S.gumbel_argmax(self.compute_logits(h), temp, seed, pos, top_k=top_k, top_p=top_p)
        return toks

    def forward_sample(self, meta: StepMeta, logit_rows: Optional[torch.Tensor], temp, seed, pos, top_k=None, top_p=None,
                       agreed_status=None) -> torch.Tensor:
        """Sampled tokens for the selected token rows (all rows when logit_rows is None)."""
        X = self.forward_hidden(meta)
        pipe = self.pipe
        if pipe is not None and not pipe.last:
            # an earlier stage: the step's tokens come back from the last one (now, or when the engine finishes the
            # step if the exchange is deferred)
            n = logit_rows.shape[0] if logit_rows is not None else meta.token_ids.shape[0]
            toks = torch.zeros(n, dtype=torch.int64, device=meta.token_ids.device)
            return toks if self.pipe_defer else pipe.broadcast_from_last(toks)
        if logit_rows is not None:
            X = X.index_select(0, logit_rows)
        toks = self.sample(self.head_hidden(X), temp, seed, pos, top_k, top_p, agreed_status)
        if pipe is None or self.pipe_defer:
            return toks.contiguous() if pipe is not None else toks
        return pipe.broadcast_from_last(toks.contiguous())

    def forward(self, meta: StepMeta, logit_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Logits for the selected token rows (all rows when logit_rows is None)."""
        X = self.forward_hidden(meta)
        if logit_rows is not None:
            X = X.index_select(0, logit_rows)
        return self.compute_logits(self.head_hidden(X))
