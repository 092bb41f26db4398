"""Typed, frozen configuration for the whole engine.

One ``EngineConfig`` (model / parallel / cache / scheduler / speculative / kernel
sections) is built once from CLI + JSON, validated, printed resolved and never
re-read on a hot path.  This replaces the reference's three tiers of shell knobs,
``VLLM_*`` environment switches and ``vllm serve`` flags
(launchers/start-hy4-tp4.sh:16-155,370-391; overlay/attention.py:98-117).

Validation is fail-closed: an invalid knob raises ``ConfigError`` (the launcher
maps it to exit status 2, as launchers/start-hy4-tp4.sh:59-118 does).
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple


class ConfigError(ValueError):
    """Raised for any knob that fails validation (fail-closed)."""


KV_QUANT_BLOCK = 64          # elements per UE8M0 scale in an fp8_ds_mla row
KV_SCALE_BYTES = 8           # scale bytes per row (nope/64 used, rest padding)
FP8_BLOCK = 128              # block edge of dense FP8 weight scales / act groups
NVFP4_GROUP = 16             # elements per e4m3 scale (NVFP4)
MXFP4_GROUP = 32             # elements per ue8m0 scale (MXFP4 checkpoint layout)
FP8_MAX = 448.0


def _check_field_types(cfg) -> None:
    """Every field holds a value of its declared kind (a `config.json` with a string where a number belongs must fail as
    a configuration error that names the field, not as a TypeError somewhere in the arithmetic)."""
    for f in dataclasses.fields(cfg):
        v, d = getattr(cfg, f.name), f.default
        if isinstance(d, bool):
            ok = isinstance(v, bool)
        elif isinstance(d, int):
            ok = isinstance(v, int) and not isinstance(v, bool)
        elif isinstance(d, float):
            ok = isinstance(v, (int, float)) and not isinstance(v, bool) and v == v and abs(v) != float("inf")
        elif isinstance(d, str):
            ok = isinstance(v, str)
        elif isinstance(d, tuple):
            ok = isinstance(v, tuple) and all(isinstance(x, int) and not isinstance(x, bool) for x in v)
        else:
            ok = True
        if not ok:
            raise ConfigError(f"{f.name}: {v!r} is not a valid {type(d).__name__}")


@dataclass(frozen=True)
class ModelConfig:
    """Architecture of a DeepSeek-V4-style decoder.

    Field names follow the HF config consumed by the reference
    (overlay/attention.py:276-298, overlay/nvidia_model.py:775-808,1076-1078).
    """

    vocab_size: int = 129280
    hidden_size: int = 4096
    num_hidden_layers: int = 48
    num_attention_heads: int = 64
    head_dim: int = 512                     # latent KV width = nope + rope
    qk_rope_head_dim: int = 64
    q_lora_rank: int = 1536
    o_lora_rank: int = 1024
    o_groups: int = 8
    sliding_window: int = 128
    compress_ratios: Tuple[int, ...] = ()   # per layer: <=1 SWA-only, 4 C4A, 128 C128A
    index_n_heads: int = 64
    index_head_dim: int = 128
    index_topk: int = 2048
    index_topk_freq: int = 4
    use_index_cache: bool = True
    # Indexer operand format: "fp8" = e4m3 q with the scale folded into the head weights and e4m3 keys with one scale
    # per row (when the KV cache is fp8_ds_mla, else bf16); "mxfp4" = e2m1 q and keys with one ue8m0 scale per 32
    # values (overlay/ops_fused_indexer_q.py:175-282): half the indexer-K bytes.  Reference (CPU) path only.
    indexer_dtype: str = "fp8"
    hc_mult: int = 4
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    n_routed_experts: int = 256
    num_experts_per_tok: int = 6
    moe_intermediate_size: int = 2048
    n_shared_experts: int = 1
    swiglu_limit: float = 10.0
    norm_topk_prob: bool = True
    scoring_func: str = "sigmoid"           # "sigmoid" | "sqrtsoftplus"
    topk_method: str = "noaux_tc"           # bias-corrected selection
    routed_scaling_factor: float = 1.0
    num_hash_layers: int = 0
    expert_dtype: str = "nvfp4"             # "nvfp4" | "mxfp4" | "bf16"
    dense_dtype: str = "fp8"                # "fp8" (128x128 block) | "bf16"
    kv_cache_dtype: str = "fp8_ds_mla"      # "fp8_ds_mla" | "bf16"
    n_mtp_layers: int = 0
    dspark_target_layer_ids: Tuple[int, ...] = ()
    dspark_markov_rank: int = 256
    dspark_block_size: int = 8
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 430000

    # ---- derived -----------------------------------------------------
    @property
    def nope_dim(self) -> int:
        return self.head_dim - self.qk_rope_head_dim

    @property
    def kv_row_data_bytes(self) -> int:
        """fp8 nope bytes + bf16 rope bytes (576 for the production shape)."""
        return self.nope_dim + 2 * self.qk_rope_head_dim

    @property
    def kv_row_bytes(self) -> int:
        """Bytes per cached token row incl. scales (584 for the production shape)."""
        return self.kv_row_data_bytes + KV_SCALE_BYTES

    @property
    def mix_hc(self) -> int:
        return (2 + self.hc_mult) * self.hc_mult

    def layer_kind(self, layer: int) -> str:
        r = self.compress_ratios[layer] if layer < len(self.compress_ratios) else 0
        if r <= 1:
            return "swa"
        if r == 4:
            return "c4a"
        if r == 128:
            return "c128a"
        raise ConfigError(f"unsupported compress ratio {r} at layer {layer}")

    def compress_ratio(self, layer: int) -> int:
        r = self.compress_ratios[layer] if layer < len(self.compress_ratios) else 0
        return r if r > 1 else 0

    def validate(self) -> None:
        _check_field_types(self)
        for name in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "head_dim", "q_lora_rank",
                     "o_lora_rank", "o_groups", "index_n_heads", "index_head_dim", "index_topk", "hc_mult",
                     "n_routed_experts", "num_experts_per_tok", "moe_intermediate_size", "sliding_window"):
            if getattr(self, name) < 1:
                raise ConfigError(f"{name} must be positive")
        if self.qk_rope_head_dim < 0 or self.n_mtp_layers < 0 or self.n_shared_experts < 0 or self.num_hash_layers < 0:
            raise ConfigError("qk_rope_head_dim, n_mtp_layers, n_shared_experts and num_hash_layers must not be negative")
        if self.head_dim <= self.qk_rope_head_dim:
            raise ConfigError("head_dim must exceed qk_rope_head_dim")
        if self.nope_dim % KV_QUANT_BLOCK:
            raise ConfigError(f"nope dim {self.nope_dim} must be a multiple of {KV_QUANT_BLOCK}")
        if self.nope_dim // KV_QUANT_BLOCK > KV_SCALE_BYTES:
            raise ConfigError("nope dim too large for 8 scale bytes per row")
        if self.qk_rope_head_dim % 2:
            raise ConfigError("rope dim must be even")
        if self.num_attention_heads % self.o_groups:
            raise ConfigError("o_groups must divide num_attention_heads")
        if len(self.compress_ratios) not in (0, self.num_hidden_layers,
                                             self.num_hidden_layers + self.n_mtp_layers):
            raise ConfigError("compress_ratios must have one entry per layer")
        for i in range(self.num_hidden_layers):
            self.layer_kind(i)
        if self.scoring_func not in ("sigmoid", "sqrtsoftplus"):
            raise ConfigError(f"unknown scoring_func {self.scoring_func!r}")
        if self.expert_dtype not in ("nvfp4", "mxfp4", "bf16"):
            raise ConfigError(f"unknown expert_dtype {self.expert_dtype!r}")
        if self.dense_dtype not in ("fp8", "bf16"):
            raise ConfigError(f"unknown dense_dtype {self.dense_dtype!r}")
        if self.kv_cache_dtype not in ("fp8_ds_mla", "bf16"):
            raise ConfigError(f"unknown kv_cache_dtype {self.kv_cache_dtype!r}")
        if self.num_experts_per_tok > self.n_routed_experts:
            raise ConfigError("top-k exceeds expert count")
        if self.index_topk_freq < 1:
            raise ConfigError("index_topk_freq must be >= 1")
        if self.index_head_dim < self.qk_rope_head_dim:
            raise ConfigError("index_head_dim must be >= rope dim")
        if self.indexer_dtype not in ("fp8", "mxfp4"):
            raise ConfigError(f"unknown indexer_dtype {self.indexer_dtype!r}")
        if self.indexer_dtype == "mxfp4" and (self.qk_rope_head_dim % 32 or (self.index_head_dim - self.qk_rope_head_dim) % 32):
            raise ConfigError("mxfp4 indexer operands need the rope and non-rope parts of index_head_dim in blocks of 32")


def alternating_ratios(n_layers: int, first: int = 4, second: int = 0) -> Tuple[int, ...]:
    """Layers alternate compressed-sparse attention with sliding-window-only."""
    return tuple(first if i % 2 == 0 else second for i in range(n_layers))


def flash_config(num_layers: int = 48, **over: Any) -> ModelConfig:
    """The DeepSeek-V4-Flash-shaped architecture used by the headline benchmark."""
    kw: Dict[str, Any] = dict(num_hidden_layers=num_layers,
                              compress_ratios=alternating_ratios(num_layers))
    kw.update(over)
    cfg = ModelConfig(**kw)
    cfg.validate()
    return cfg


def tiny_config(**over: Any) -> ModelConfig:
    """2-layer CPU-sized decoder: one C4A layer + one SWA layer, 8 experts top-2."""
    kw: Dict[str, Any] = dict(
        vocab_size=1024, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
        head_dim=80, qk_rope_head_dim=16, q_lora_rank=96, o_lora_rank=64, o_groups=2,
        sliding_window=32, compress_ratios=(4, 0), index_n_heads=2, index_head_dim=32,
        index_topk=16, index_topk_freq=4, hc_mult=4, hc_sinkhorn_iters=20,
        n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
        n_shared_experts=1, scoring_func="sigmoid", expert_dtype="bf16", dense_dtype="bf16",
        kv_cache_dtype="bf16", max_position_embeddings=4096,
    )
    kw.update(over)
    cfg = ModelConfig(**kw)
    cfg.validate()
    return cfg


@dataclass(frozen=True)
class ParallelConfig:
    tp_size: int = 1
    ep_size: int = 1             # experts partitioned over ep ranks (== tp group)
    pp_size: int = 1
    dcp_size: int = 1            # decode context parallel (KV interleave)
    indexer_sp: bool = True      # sequence-parallel indexer scoring for prefill chunks
    indexer_sp_min_rows: int = 256
    fused_collectives: bool = True   # False => NCCL-after-GEMM baseline paths
    eplb_redundant: int = 0          # spare physical expert slots per layer for replicas of hot experts (EPLB)
    eplb_record: bool = False        # count routed tokens per logical expert and layer (input of a rebalance)
    use_multimem: bool = False       # NVLS multimem loads/stores in the all-reduce

    def validate(self) -> None:
        for name in ("tp_size", "ep_size", "pp_size", "dcp_size"):
            if getattr(self, name) < 1:
                raise ConfigError(f"{name} must be >= 1")
        if self.ep_size not in (1, self.tp_size):
            raise ConfigError("ep_size must be 1 or equal tp_size")
        if self.eplb_redundant < 0 or self.eplb_redundant % self.tp_size:
            raise ConfigError("eplb_redundant must be a non-negative multiple of tp_size")


@dataclass(frozen=True)
class CacheConfig:
    page_tokens: int = 64            # rows per page in every cache group
    engine_block_tokens: int = 256   # scheduler-visible block (4 SWA pages, 1 C4A page)
    gpu_memory_utilization: float = 0.60
    num_pages: Optional[int] = None  # explicit pool size (tests / bench)
    enable_prefix_caching: bool = True
    # Context tokens the compressed-KV pools hold over all requests together.  None: room for max_num_seqs requests of
    # max_model_len each (nothing ever waits for pages).  With `size_by_memory` the engine derives it on a GPU from
    # gpu_memory_utilization x device memory minus what is allocated when it starts (the weights).
    kv_pool_tokens: Optional[int] = None
    size_by_memory: bool = False

    def validate(self) -> None:
        if self.page_tokens != 64:
            raise ConfigError("page_tokens must be 64")
        if self.engine_block_tokens % self.page_tokens:
            raise ConfigError("engine block must be a whole number of pages")
        if not (0.0 < self.gpu_memory_utilization <= 0.98):
            raise ConfigError("gpu_memory_utilization out of range")


@dataclass(frozen=True)
class SchedulerConfig:
    max_model_len: int = 430000
    max_num_seqs: int = 32
    max_num_batched_tokens: int = 4096
    graph_cap: int = 256             # largest decode batch captured as a CUDA graph
    decode_first: bool = True
    # Schedule and launch step k+1 before the tokens of step k are read: a decode row's input token is copied on the
    # device from the previous step's samples, the host reads them while the next step runs, and a request that turns
    # out to have ended (EOS) has one surplus row computed and dropped.  Off by default; not with speculative decoding.
    async_scheduling: bool = False

    def validate(self) -> None:
        if self.max_num_seqs < 1 or self.max_num_batched_tokens < 1:
            raise ConfigError("scheduler limits must be positive")
        if self.graph_cap < 0:
            raise ConfigError("graph_cap must be >= 0")


@dataclass(frozen=True)
class SpecConfig:
    method: str = "none"             # "none" | "dspark"
    num_speculative_tokens: int = 5
    markov_topk: int = 512           # 0 => dense Markov bias over the whole vocab
    temperature: float = 0.6
    markov_sideload: str = ""
    replicate_markov: bool = True

    def validate(self) -> None:
        if self.method not in ("none", "dspark"):
            raise ConfigError(f"unknown speculative method {self.method!r}")
        if self.method == "dspark" and not (1 <= self.num_speculative_tokens <= 15):
            raise ConfigError("num_speculative_tokens must be in [1, 15]")
        if self.markov_topk < 0:
            raise ConfigError("markov_topk must be >= 0")


@dataclass(frozen=True)
class KernelConfig:
    compressor_fp8: bool = True
    target_lm_head_fp8: bool = True
    fused_gate: bool = True
    oneshot_max_bytes: int = 512 * 1024   # one-shot all-reduce up to here, two-shot above
    wait_budget_iters: int = 4_000_000    # bound of every device-side spin
    multi_stream: bool = True

    def validate(self) -> None:
        if self.oneshot_max_bytes < 0 or self.wait_budget_iters < 1:
            raise ConfigError("kernel limits must be positive")


@dataclass(frozen=True)
class EngineConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    cache: CacheConfig = field(default_factory=CacheConfig)
    sched: SchedulerConfig = field(default_factory=SchedulerConfig)
    spec: SpecConfig = field(default_factory=SpecConfig)
    kernels: KernelConfig = field(default_factory=KernelConfig)
    seed: int = 0

    def validate(self) -> "EngineConfig":
        for part in (self.model, self.parallel, self.cache, self.sched, self.spec, self.kernels):
            part.validate()
        if self.model.num_attention_heads % self.parallel.tp_size:
            raise ConfigError("tp_size must divide num_attention_heads")
        if self.model.o_groups % self.parallel.tp_size and self.parallel.tp_size % self.model.o_groups:
            raise ConfigError("tp_size and o_groups must divide one another")
        if self.spec.method == "dspark" and self.parallel.pp_size > 1:
            # The reference refuses DSpark under pipeline parallelism
            # (overlay/dspark_utils_v2.py:158-159).
            raise ConfigError("dspark speculative decoding does not support pp_size > 1")
        return self

    # ---- (de)serialisation --------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    def resolved(self) -> str:
        """The resolved configuration as printed at start-up."""
        return json.dumps(self.to_dict(), indent=1, sort_keys=True)

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "EngineConfig":
        def build(cls, sub):
            sub = dict(sub or {})
            names = {f.name for f in dataclasses.fields(cls)}
            unknown = set(sub) - names
            if unknown:
                raise ConfigError(f"unknown {cls.__name__} keys: {sorted(unknown)}")
            for k, v in list(sub.items()):
                if isinstance(v, list):
                    sub[k] = tuple(v)
            return cls(**sub)

        known = {"model", "parallel", "cache", "sched", "spec", "kernels", "seed"}
        unknown = set(d) - known
        if unknown:
            raise ConfigError(f"unknown EngineConfig sections: {sorted(unknown)}")
        return EngineConfig(
            model=build(ModelConfig, d.get("model")),
            parallel=build(ParallelConfig, d.get("parallel")),
            cache=build(CacheConfig, d.get("cache")),
            sched=build(SchedulerConfig, d.get("sched")),
            spec=build(SpecConfig, d.get("spec")),
            kernels=build(KernelConfig, d.get("kernels")),
            seed=int(d.get("seed", 0)),
        ).validate()


def model_config_from_hf(hf: Dict[str, Any]) -> ModelConfig:
    """Build a ModelConfig from a DeepSeek-V4 ``config.json`` dictionary."""
    names = {f.name for f in dataclasses.fields(ModelConfig)}
    kw = {k: (tuple(v) if isinstance(v, list) else v) for k, v in hf.items() if k in names}
    if "expert_dtype" in hf and hf["expert_dtype"] == "fp4":
        kw["expert_dtype"] = "mxfp4"    # checkpoint layout: e2m1 + ue8m0 per 32
    cfg = ModelConfig(**kw)
    cfg.validate()
    return cfg
