"""Operator knobs: environment -> validated launch settings, failing closed with exit code 2.

Every knob is checked before anything is started (no process, no GPU context), so a typo costs
nothing.  The set mirrors the shell knobs of the reference launcher
(launchers/start-hy4-tp4.sh:16-118: GPU_MEM, MAX_MODEL_LEN, MAX_NUM_SEQS, MAX_NUM_BATCHED, SPEC_TOKENS,
FP8HEAD, MARKOV_TOPK, REFINE, MARKOV_SIDELOAD, and the env block :123-147), restated for one 8-GPU
NVSwitch node: TP_SIZE picks the GPUs, ONESHOT arms the symmetric-memory all-reduce, FUSED the
GEMM+collective kernels, DCP deals the ratio-4 KV pages over the ranks (capacity for long contexts).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional

MODEL_VOCAB_SIZE = 129280
EXIT_BAD_KNOB = 2
_SAFE_PATH = re.compile(r"^[A-Za-z0-9_./-]+$")
_UINT = re.compile(r"^(0|[1-9][0-9]*)$")


class KnobError(ValueError):
    """A knob failed validation; `str(e)` is the operator-facing ABORT line."""


def _flag(env: Mapping[str, str], name: str, default: str) -> int:
    v = env.get(name, default)
    if v not in ("0", "1"):
        raise KnobError(f"ABORT: {name} must be 0 or 1 (got {v})")
    return int(v)


def _uint(env: Mapping[str, str], name: str, default: str, lo: int, hi: int) -> int:
    v = env.get(name, default)
    if not _UINT.match(v) or len(v) > len(str(hi)) + 1:
        raise KnobError(f"ABORT: {name} must be an integer in [{lo},{hi}] (got {v})")
    n = int(v, 10)
    if not lo <= n <= hi:
        raise KnobError(f"ABORT: {name} must be an integer in [{lo},{hi}] (got {v})")
    return n


def _ratio(env: Mapping[str, str], name: str, default: str, lo: float, hi: float) -> float:
    v = env.get(name, default)
    try:
        f = float(v)
    except ValueError:
        raise KnobError(f"ABORT: {name} must be a number in ({lo},{hi}] (got {v})") from None
    if not (lo < f <= hi):
        raise KnobError(f"ABORT: {name} must be a number in ({lo},{hi}] (got {v})")
    return f


@dataclass
class Knobs:
    tp_size: int = 8
    gpu_mem: float = 0.60
    max_model_len: int = 430000
    max_num_seqs: int = 32
    max_num_batched: int = 4096
    graph_cap: int = 256
    spec_tokens: int = 5
    fp8_head: int = 0
    markov_topk: int = 512
    refine: int = 0
    markov_sideload: str = ""
    temperature: float = 0.8
    effort: str = ""
    oneshot: int = 1
    fused: int = 1
    multimem: int = 0
    pp_size: int = 1              # pipeline stages; ranks = TP_SIZE x PP_SIZE
    async_sched: int = 0          # 1: schedule and launch the next step before this step's tokens are read
    dcp: int = 0                  # 1: ratio-4 KV pages dealt over the tensor-parallel ranks (decode context parallel)
    idx_freq: int = 4
    idx_sp: int = 1
    compressor_fp8: int = 1
    target_head_fp8: int = 1
    gate_fused: int = 1
    dev_mode: int = 1
    port: int = 8000
    model_path: str = ""
    model_root: str = "/models"
    served_name: str = "deepseek-v4-flash"
    warnings: List[str] = field(default_factory=list)

    def to_env(self) -> Dict[str, str]:
        """The env block handed to every rank (the engine reads STK_* names only)."""
        return {
            "STK_TP_SIZE": str(self.tp_size), "STK_GPU_MEM": str(self.gpu_mem), "STK_MAX_MODEL_LEN": str(self.max_model_len),
            "STK_MAX_NUM_SEQS": str(self.max_num_seqs), "STK_MAX_NUM_BATCHED_TOKENS": str(self.max_num_batched),
            "STK_GRAPH_CAP": str(self.graph_cap), "STK_SPEC_TOKENS": str(self.spec_tokens),
            "STK_FP8_DRAFT_HEAD": str(self.fp8_head), "STK_DRAFT_TOPK": str(self.markov_topk),
            "STK_REFINE_PASS": str(self.refine), "STK_MARKOV_SIDELOAD": self.markov_sideload,
            "STK_TEMPERATURE": str(self.temperature), "STK_REASONING_EFFORT": self.effort,
            "STK_ONESHOT_AR": str(self.oneshot), "STK_FUSED_COLLECTIVES": str(self.fused), "STK_MULTIMEM": str(self.multimem),
            "STK_INDEX_TOPK_FREQ": str(self.idx_freq), "STK_INDEXER_SP": str(self.idx_sp),
            "STK_COMPRESSOR_FP8": str(self.compressor_fp8), "STK_TARGET_LM_HEAD_FP8": str(self.target_head_fp8),
            "STK_GATE_FUSED": str(self.gate_fused), "STK_DEV_MODE": str(self.dev_mode), "STK_PORT": str(self.port),
            "STK_MODEL_PATH": self.model_path, "STK_SERVED_MODEL_NAME": self.served_name,
            # rendezvous stays on loopback: one node, one process per GPU
            "MASTER_ADDR": "127.0.0.1", "NCCL_DEBUG": "WARN",
        }


def parse_knobs(env: Mapping[str, str]) -> Knobs:
    k = Knobs()
    k.model_root = env.get("MODEL_ROOT", k.model_root).rstrip("/") or "/"
    k.model_path = env.get("MODEL_PATH", "")
    k.served_name = env.get("SERVED_NAME", k.served_name)
    tp = env.get("TP_SIZE", "8")
    if tp not in ("1", "2", "4", "8"):
        raise KnobError(f"ABORT: TP_SIZE must be 1, 2, 4 or 8 (got {tp})")
    k.tp_size = int(tp)
    k.gpu_mem = _ratio(env, "GPU_MEM", "0.60", 0.0, 0.95)
    k.max_model_len = _uint(env, "MAX_MODEL_LEN", "430000", 256, 1 << 20)
    k.max_num_seqs = _uint(env, "MAX_NUM_SEQS", "32", 1, 1024)
    k.max_num_batched = _uint(env, "MAX_NUM_BATCHED", "4096", 64, 65536)
    k.graph_cap = _uint(env, "GRAPH_CAP", "256", 0, 4096)
    k.spec_tokens = _uint(env, "SPEC_TOKENS", "5", 0, 15)
    k.fp8_head = _flag(env, "FP8HEAD", "0")
    k.refine = _flag(env, "REFINE", "0")
    topk = env.get("MARKOV_TOPK", "512")
    if not _UINT.match(topk) or len(topk) > len(str(MODEL_VOCAB_SIZE)):
        raise KnobError(f"ABORT: MARKOV_TOPK must be 0 or an integer in [1,{MODEL_VOCAB_SIZE}] (got {topk})")
    k.markov_topk = int(topk, 10)
    if k.markov_topk > MODEL_VOCAB_SIZE:
        raise KnobError(f"ABORT: MARKOV_TOPK exceeds model vocab ({k.markov_topk} > {MODEL_VOCAB_SIZE})")
    side = env.get("MARKOV_SIDELOAD", "")
    if side:
        if not side.startswith(k.model_root + "/"):
            raise KnobError(f"ABORT: MARKOV_SIDELOAD must be an absolute path under {k.model_root} (got {side})")
        if not _SAFE_PATH.match(side) or ".." in side:
            raise KnobError(f"ABORT: unsafe character in MARKOV_SIDELOAD: {side}")
    k.markov_sideload = side
    temp = env.get("TEMP", "0.8")
    try:
        k.temperature = float(temp)
    except ValueError:
        raise KnobError(f"ABORT: TEMP must be a number in [0,2] (got {temp})") from None
    if not 0.0 <= k.temperature <= 2.0:
        raise KnobError(f"ABORT: TEMP must be a number in [0,2] (got {temp})")
    k.effort = env.get("EFFORT", "")
    if k.effort not in ("", "none", "low", "medium", "high", "max", "xhigh"):
        raise KnobError(f"ABORT: EFFORT must be one of none/low/medium/high/max (got {k.effort})")
    k.oneshot = _flag(env, "ONESHOT", "1")
    k.fused = _flag(env, "FUSED", "1")
    k.multimem = _flag(env, "MULTIMEM", "0")
    k.dcp = _flag(env, "DCP", "0")
    k.pp_size = _uint(env, "PP_SIZE", "1", 1, 8)
    k.async_sched = _flag(env, "ASYNC_SCHED", "0")
    k.idx_freq = _uint(env, "IDXFREQ", "4", 1, 64)
    k.idx_sp = _flag(env, "IDXSP", "1")
    k.compressor_fp8 = _flag(env, "COMPRESSOR_FP8", "1")
    k.target_head_fp8 = _flag(env, "TGT_HEAD_FP8", "1")
    k.gate_fused = _flag(env, "GATEFUSE", "1")
    k.dev_mode = _flag(env, "DEVMODE", "1")
    k.port = _uint(env, "PORT", "8000", 1, 65535)
    if k.model_path and (not _SAFE_PATH.match(k.model_path) or ".." in k.model_path):
        raise KnobError(f"ABORT: unsafe character in MODEL_PATH: {k.model_path}")
    # cross-knob rules
    draft_knobs = k.fp8_head == 1 or k.refine == 1 or bool(k.markov_sideload)
    if draft_knobs and k.spec_tokens == 0:
        raise KnobError("ABORT: FP8HEAD/REFINE/MARKOV_SIDELOAD require speculative decoding (SPEC_TOKENS >= 1)")
    if k.refine == 1 and k.spec_tokens < 2:
        raise KnobError("ABORT: REFINE=1 requires SPEC_TOKENS >= 2 (there are no noise slots to refine)")
    if k.fused == 1 and k.oneshot == 0 and k.tp_size > 1:
        raise KnobError("ABORT: FUSED=1 needs the symmetric-memory path (ONESHOT=1)")
    if k.tp_size * k.pp_size > 8:
        raise KnobError(f"ABORT: TP_SIZE x PP_SIZE must fit one 8-GPU node (got {k.tp_size} x {k.pp_size})")
    if k.pp_size > 1 and k.spec_tokens:
        raise KnobError("ABORT: PP_SIZE > 1 is not available with speculative decoding (SPEC_TOKENS=0)")
    if k.pp_size > 1:
        k.warnings.append("PP_SIZE > 1: steps run without CUDA graphs and the stages' tensor-parallel groups use NCCL")
    if k.async_sched == 1 and (k.spec_tokens or k.pp_size > 1):
        raise KnobError("ABORT: ASYNC_SCHED=1 is not available with speculative decoding or pipeline stages "
                        "(SPEC_TOKENS=0, PP_SIZE=1)")
    if k.dcp == 1 and k.tp_size == 1:
        raise KnobError("ABORT: DCP=1 deals the ratio-4 KV pages over the tensor-parallel ranks (TP_SIZE >= 2)")
    if k.dcp == 1:
        k.warnings.append("DCP=1: steps run without CUDA graphs (a capacity setting for long contexts, not a speed-up)")
    if k.multimem == 1 and k.oneshot == 0:
        raise KnobError("ABORT: MULTIMEM=1 needs the symmetric-memory path (ONESHOT=1)")
    if k.max_num_batched < k.max_num_seqs * (1 + k.spec_tokens):
        raise KnobError("ABORT: MAX_NUM_BATCHED must hold one verify row block per sequence "
                        f"({k.max_num_seqs} x {1 + k.spec_tokens})")
    rows = k.max_num_seqs * (1 + k.spec_tokens)
    if k.graph_cap and rows > k.graph_cap:
        k.warnings.append(f"decode batches above {k.graph_cap // (1 + k.spec_tokens)} sequences run outside CUDA graphs "
                          f"({rows} rows > GRAPH_CAP {k.graph_cap})")
    return k
