"""DSpark: semi-autoregressive block drafter with a Markov head, and its loader checks.

A draft step proposes N tokens per request in one parallel pass of a 3-layer decoder over a
query block (the anchor = last verified token, then N-1 mask tokens), then samples left to right,
adding to each position's base logits a first-order Markov bias ``W2 . W1[prev]`` and drawing with
the same seeded Gumbel noise, keyed by (seed, position), that the verifier will use.  The verifier
accepts position j iff its own argmax under that noise equals the draft's, and always emits its own
argmax, so the output distribution is the target's for any draft distribution.

Layout of the work (reference: overlay/dspark_v2.py:239-376 model, :379-443 context insert,
overlay/dspark_speculator_v2.py:233-298 sequential sampling, :66-111 knob parsers,
overlay/dspark_utils_v2.py:18-110 sideload contract):

* `combine`: main_x = RMSNorm(main_proj(concat of target aux hidden states));
* `insert_context`: per draft layer, the wkv half of the fused wq_a|wkv projection of main_x ->
  kv_norm -> RoPE + quantise + write at the token's slot of that layer's SWA cache;
* `draft`: block forward with non-causal window indices, hc_head, final norm, shared lm_head,
  optional top-k truncation (Markov bias gathered only at the base top-k), sequential sampling.

The Markov tensors are full [V, R] replicas on every rank: with identical seeds every rank samples
identical tokens and no per-position collective is needed.
"""
from __future__ import annotations

import dataclasses
import hashlib
from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..config import ConfigError, ModelConfig, SpecConfig
from ..models.dsv4 import DSV4Model, LayerWeights, ModelWeights, StepMeta, WeightSource, _get, build_layer
from ..ops import attention as A
from ..ops import cache as C
from ..ops import functional as Fn
from ..ops import sampling as S
from ..ops.cache import PAGE
from ..ops.functional import LinearWeight

BF16 = torch.bfloat16
F32 = torch.float32
_OFF = {"", "0", "false", "no", "off"}
_ON = {"1", "true", "yes", "on"}


# ---------------------------------------------------------------------------------------
# knob parsers and loader contracts (fail closed)
# ---------------------------------------------------------------------------------------
def parse_draft_topk(raw: str, vocab_size: int) -> Optional[int]:
    """"" / 0 / off -> None (dense Markov bias); otherwise an integer in [1, vocab]."""
    v = raw.strip().lower()
    if v in _OFF:
        return None
    try:
        k = int(v)
    except ValueError as e:
        raise ValueError(f"draft top-k must be an integer or 0, got {raw!r}") from e
    if not 1 <= k <= vocab_size:
        raise ValueError(f"draft top-k must be in [1, {vocab_size}], got {k}")
    return k


def parse_refine_pass(raw: str) -> bool:
    v = raw.strip().lower()
    if v in _OFF:
        return False
    if v in _ON:
        return True
    raise ValueError(f"refine pass must be a boolean value, got {raw!r}")


def refine_feedback_indices(max_reqs: int, n_query: int) -> List[int]:
    """Flat query-buffer indices of the mask slots: offset j >= 1 of every request receives the
    token drafted at offset j-1; anchors (offset 0) are never rewritten."""
    return [r * n_query + j for r in range(max_reqs) for j in range(1, n_query)]


def validate_markov_sideload(keys: Iterable[str], w1_shape: Sequence[int], w2_shape: Sequence[int], vocab_size: int,
                             rank: int, replicated_w1: bool, replicated_w2: bool) -> Optional[str]:
    """Error text, or None when the payload may overwrite the Markov tensors in place."""
    missing = {"markov_w1", "markov_w2"} - set(keys)
    if missing:
        return f"sideload payload missing keys: {sorted(missing)}"
    want = (vocab_size, rank)
    if tuple(w1_shape) != want:
        return f"markov_w1 shape {tuple(w1_shape)} != expected {want}"
    if tuple(w2_shape) != want:
        return f"markov_w2 shape {tuple(w2_shape)} != expected {want}"
    if not replicated_w1:
        return "sideload requires a replicated Markov W1"
    if not replicated_w2:
        return "sideload requires a replicated Markov W2"
    return None


def bf16_head_release_blockers(fp8_head: bool, fp8_draft_head: bool, release_requested: bool, tie_embeddings: bool,
                               head_shared_with_draft: bool, logprobs_need_bf16: bool) -> List[str]:
    """Reasons why the bf16 lm_head must stay resident although an fp8 copy exists.  The release is
    refused unless every consumer of the bf16 tensor has an fp8 replacement."""
    if not release_requested:
        return []
    out = []
    if not fp8_head:
        out.append("target lm_head has no fp8 copy")
    if head_shared_with_draft and not fp8_draft_head:
        out.append("draft shares the bf16 lm_head and has no fp8 draft head")
    if tie_embeddings:
        out.append("lm_head is tied to the embedding")
    if logprobs_need_bf16:
        out.append("logprob requests need the bf16 head")
    return out


# ---------------------------------------------------------------------------------------
# weights
# ---------------------------------------------------------------------------------------
@dataclass
class MarkovHead:
    w1: torch.Tensor            # [V, R] bf16, embedding of the previous token
    w2: torch.Tensor            # [V, R] bf16, bias[v] = w2[v] . w1[prev]
    fp8_built: bool = False     # set once a quantised copy exists; sideloading after that is refused

    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.w1.index_select(0, tokens)

    def apply(self, base: torch.Tensor, prev: torch.Tensor, topk: int) -> torch.Tensor:
        """base [B, V] -> fp32 proposal logits: base + bias on the base top-k (all of V when topk == 0),
        -inf elsewhere."""
        return S.markov_topk_bias(base, self.w2, self.embed(prev), topk)

    def sideload(self, path: str, vocab_size: int, rank: int) -> str:
        """Overwrite W1/W2 from a refit payload; returns the payload's SHA-256."""
        if self.fp8_built:
            raise RuntimeError("Markov sideload must run before the quantised W2 copy is built")
        payload = torch.load(path, map_location="cpu", weights_only=True)
        if not isinstance(payload, dict):
            raise RuntimeError(f"Markov sideload {path} must be a dict payload, got {type(payload)}")
        w1, w2 = payload.get("markov_w1"), payload.get("markov_w2")
        err = validate_markov_sideload(payload.keys(), tuple(w1.shape) if w1 is not None else (),
                                       tuple(w2.shape) if w2 is not None else (), vocab_size, rank, True, True)
        if err is None and not (bool(torch.isfinite(w1.float()).all()) and bool(torch.isfinite(w2.float()).all())):
            err = "sideload tensors contain non-finite values"
        if err is not None:
            raise RuntimeError(f"invalid Markov sideload ({path}): {err}")
        self.w1.copy_(w1.to(device=self.w1.device, dtype=self.w1.dtype))
        self.w2.copy_(w2.to(device=self.w2.device, dtype=self.w2.dtype))
        with open(path, "rb") as f:
            return hashlib.sha256(f.read()).hexdigest()


@dataclass
class DraftWeights:
    main_proj: LinearWeight      # [H, H * n_aux]
    main_norm: torch.Tensor
    model: ModelWeights          # draft layers + mtp norm/hc_head; embed and head alias the target's
    markov: MarkovHead


def build_draft_weights(cfg: ModelConfig, src: WeightSource, target: ModelWeights, device, tp_rank: int = 0,
                        tp_size: int = 1) -> DraftWeights:
    if not cfg.n_mtp_layers:
        raise ConfigError("the checkpoint config declares no draft (mtp) layers")
    H, V, hc, R = cfg.hidden_size, cfg.vocab_size, cfg.hc_mult, cfg.dspark_markov_rank
    n_aux = max(1, len(cfg.dspark_target_layer_ids))
    g = lambda n, s: _get(src, n, s, device)
    layers = [build_layer(cfg, src, f"mtp.{k}", cfg.num_hidden_layers + k, device, tp_rank, tp_size, kind="swa")
              for k in range(cfg.n_mtp_layers)]
    mw = ModelWeights(embed=target.embed, head=target.head, norm=g("mtp.norm.weight", (H,)).to(BF16),
                      hc_head=(g("mtp.hc_head_fn", (hc, hc * H)).to(F32).contiguous(), g("mtp.hc_head_base", (hc,)).to(F32),
                               g("mtp.hc_head_scale", (1,)).to(F32)),
                      layers=layers, vocab_start=target.vocab_start)
    return DraftWeights(
        main_proj=LinearWeight(g("mtp.main_proj.weight", (H, H * n_aux)).to(BF16).contiguous()),
        main_norm=g("mtp.main_norm.weight", (H,)).to(BF16), model=mw,
        markov=MarkovHead(g("mtp.markov_w1.weight", (V, R)).to(BF16).contiguous(),
                          g("mtp.markov_w2.weight", (V, R)).to(BF16).contiguous()))


class _DraftKV:
    """The draft layers' view of the KV manager: SWA caches only, indexed from 0."""

    def __init__(self, kv, first_layer: int, n: int):
        self.swa_cache = {k: kv.swa_cache[first_layer + k] for k in range(n)}
        self.swa = kv.swa
        self.dcp_rank, self.dcp_size = 0, 1
        self.comp_cache: Dict[int, Any] = {}
        self.idx_cache: Dict[int, Any] = {}
        self.comp_state: Dict[int, Any] = {}
        self.idx_state: Dict[int, Any] = {}


# ---------------------------------------------------------------------------------------
# the drafter
# ---------------------------------------------------------------------------------------
class DSparkDrafter:
    def __init__(self, cfg: ModelConfig, spec: SpecConfig, weights: DraftWeights, kv, comm=None, tp_rank: int = 0,
                 tp_size: int = 1, mask_token_id: int = 0):
        self.cfg, self.spec, self.w, self.kv = cfg, spec, weights, kv
        self.n = spec.num_speculative_tokens
        self.topk = min(spec.markov_topk, cfg.vocab_size)
        self.mask_token_id = mask_token_id
        n_l = cfg.n_mtp_layers
        dcfg = dataclasses.replace(cfg, num_hidden_layers=n_l, compress_ratios=(0,) * n_l, n_mtp_layers=0,
                                   num_hash_layers=0, dspark_target_layer_ids=())
        self.model = DSV4Model(dcfg, weights.model, _DraftKV(kv, cfg.num_hidden_layers, n_l), comm, tp_rank, tp_size)
        if spec.markov_sideload:
            self.sideload_sha = weights.markov.sideload(spec.markov_sideload, cfg.vocab_size, cfg.dspark_markov_rank)
        dev = weights.model.embed.device
        self.device = dev
        # non-causal window: the context rows [prefix-W, prefix) plus the N block rows, 64-row granules
        self.width = ((cfg.sliding_window + self.n + 63) // 64) * 64
        self._prefix = torch.zeros(kv.max_requests, dtype=torch.int32, device=dev)
        self._seqlen = torch.zeros(kv.max_requests, dtype=torch.int32, device=dev)
        self._steps = torch.arange(self.n, device=dev)

    # ---- context ---------------------------------------------------------------------
    def combine(self, aux: torch.Tensor) -> torch.Tensor:
        return Fn.rms_norm(Fn.linear(aux, self.w.main_proj, tag="main_proj"), self.w.main_norm, self.cfg.rms_norm_eps)

    def insert_context(self, aux: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor) -> None:
        """aux [T, H*n_aux] target hidden states of the tokens just verified (padding rows have slot -1)."""
        cfg = self.cfg
        main_x = self.combine(aux)
        ql = cfg.q_lora_rank
        for k, lw in enumerate(self.w.model.layers):
            kv = Fn.linear(main_x, lw.w_qa_kv, tag="ctx_kv")[:, ql:]
            kv = Fn.rms_norm(kv, lw.kv_norm, cfg.rms_norm_eps)
            C.kv_rope_quant_insert(kv, positions, slot_mapping, self.model.inv, self.model.kv.swa_cache[k])

    # ---- one draft block ---------------------------------------------------------------
    def block_meta(self, anchors: torch.Tensor, anchor_pos: torch.Tensor, rows: torch.Tensor) -> StepMeta:
        """Device-side metadata of the query block: request b holds positions anchor_pos[b] + [0, N)."""
        n, b = self.n, anchors.shape[0]
        tokens = torch.full((b, n), self.mask_token_id, dtype=torch.int64, device=self.device)
        tokens[:, 0] = anchors
        pos = anchor_pos.to(torch.int64)[:, None] + self._steps[None, :]
        tok_req = rows.to(torch.int32)[:, None].expand(b, n).reshape(-1).contiguous()
        table = self.kv.swa.table_dev
        page = table[rows.long()[:, None], (pos // PAGE)]
        slot = torch.where(page >= 0, page.to(torch.int64) * PAGE + pos % PAGE, torch.full_like(pos, -1))
        self._prefix.index_copy_(0, rows.long(), anchor_pos.to(torch.int32))
        self._seqlen.index_copy_(0, rows.long(), (anchor_pos + n).to(torch.int32))
        slots, lens = A.swa_indices_noncausal(tok_req, self._prefix, self._seqlen, table, self.cfg.sliding_window,
                                              self.width)
        first = anchor_pos.to(torch.int32)[:, None].expand(b, n).reshape(-1)
        last = (anchor_pos.to(torch.int32) + n - 1)[:, None].expand(b, n).reshape(-1)
        return StepMeta(tokens.view(-1), tok_req, pos.view(-1), first.contiguous(), last.contiguous(), slot.view(-1),
                        slots, lens, 1)

    def draft(self, anchors: torch.Tensor, anchor_pos: torch.Tensor, rows: torch.Tensor, temperature: torch.Tensor,
              seed: torch.Tensor, want_logits: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """anchors [B] int64 (last verified token), anchor_pos [B] its position, rows [B] request rows.
        Returns draft tokens [B, N] (token j is proposed for position anchor_pos + 1 + j) and, on request,
        the proposal logits [B, N, V] that were sampled from."""
        n, b = self.n, anchors.shape[0]
        meta = self.block_meta(anchors, anchor_pos, rows)
        X = self.model.forward_hidden(meta)
        base = self.model.compute_logits(self.model.head_hidden(X)).view(b, n, -1)
        if self.topk > 0 and not want_logits:
            # the candidate sets (top-k of the base logits) do not depend on the sampled tokens: select them for all
            # positions at once, then run the dependent part -- W1 row, gathered W2 rows, noisy arg-max -- in one kernel
            ci, cv = S.topk_candidates(base.reshape(b * n, -1), self.topk)
            toks = S.markov_chain(ci.view(b, n, -1), cv.view(b, n, -1), anchors, self.w.markov.w1, self.w.markov.w2,
                                  temperature, seed, anchor_pos.to(torch.int64) + 1)
            return toks, None
        out = torch.empty(b, n, dtype=torch.int64, device=self.device)
        rec = torch.empty(b, n, base.shape[-1], dtype=F32, device=self.device) if want_logits else None
        prev = anchors
        pos = anchor_pos.to(torch.int64)
        for i in range(n):
            logits_i = self.w.markov.apply(base[:, i], prev, self.topk)
            # the verifier draws the token of position Q with the key of its predecessor row's sample slot,
            # i.e. "position being sampled" = anchor_pos + 1 + i
            tok, proc = S.gumbel_argmax(logits_i, temperature, seed, pos + 1 + i, want_processed=want_logits)
            out[:, i] = tok
            if rec is not None:
                rec[:, i] = proc
            prev = tok
        return out, rec
