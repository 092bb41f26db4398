"""Checkpoint access: DeepSeek-V4 safetensors layout -> the tensors `build_model_weights` asks for.

* `SafetensorsIndex`: memory-maps every shard, reads the JSON headers itself (8-byte length + JSON +
  raw little-endian data) and hands out zero-copy views, including the dtypes torch's own loader does
  not name (F8_E8M0 scale bytes, packed FP4 as U8);
* `CheckpointSource`: a `WeightSource` over the index.  Quantised tensors come with a sibling
  ``.scale``: FP8 e4m3 weights with 128x128 block scales (fp32, or ue8m0 exponent bytes), MXFP4
  experts as packed e2m1 + ue8m0 per 32.  They are expanded to the master value they encode; the
  builder's block quantiser reproduces the stored codes exactly when it uses the checkpoint's scale
  rule (`fp8_scale_rule`), because the largest code of every block then maps back to the same scale;
* `shard_plan`: which slice of which tensor a TP rank owns (column-parallel rows, row-parallel
  columns, head ranges of attn_sink, expert ranges), always on 128-element block boundaries;
* `write_checkpoint`: the inverse, used by tests and by the random-weight tooling.

Name map and stacking rules: overlay/nvidia_model.py:1843-1953,2002-2036 (``.scale`` siblings,
``ffn.gate.bias``, e8m0 scales kept as raw bytes, w1/w3 and wq_a/wkv stacked after loading, attn_sink
sliced by head range); overlay/dspark_v2.py:616-764 for the ``mtp.*`` family.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch

from ..config import FP8_BLOCK, ModelConfig, model_config_from_hf
from ..ops import reference as R
from .dsv4 import WeightSource
from .weights import weight_shapes

_DTYPES = {"F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8),
           "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
           "BOOL": (torch.bool, 1), "F8_E4M3": (torch.float8_e4m3fn, 1), "F8_E5M2": (torch.float8_e5m2, 1),
           "F8_E8M0": (torch.uint8, 1), "F4": (torch.uint8, 1)}
_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int64: "I64", torch.int32: "I32",
          torch.uint8: "U8", torch.float8_e4m3fn: "F8_E4M3", torch.int8: "I8", torch.bool: "BOOL"}


@dataclass(frozen=True)
class TensorInfo:
    file: str
    dtype: str
    shape: Tuple[int, ...]
    start: int
    end: int


class SafetensorsIndex:
    def __init__(self, path: str):
        self.path = path
        self.tensors: Dict[str, TensorInfo] = {}
        self._maps: Dict[str, mmap.mmap] = {}
        self._data0: Dict[str, int] = {}
        files = self._shards(path)
        if not files:
            raise FileNotFoundError(f"no .safetensors files under {path}")
        for f in files:
            self._read_header(f)

    @staticmethod
    def _shards(path: str) -> List[str]:
        if os.path.isfile(path):
            return [path]
        idx = os.path.join(path, "model.safetensors.index.json")
        if os.path.isfile(idx):
            with open(idx) as f:
                names = sorted(set(json.load(f)["weight_map"].values()))
            return [os.path.join(path, n) for n in names]
        return sorted(os.path.join(path, n) for n in os.listdir(path) if n.endswith(".safetensors"))

    def _read_header(self, file: str) -> None:
        size = os.path.getsize(file)
        with open(file, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise ValueError(f"{file}: shorter than a safetensors header")
            (n,) = struct.unpack("<Q", head)
            if n > 256 << 20 or n > size - 8:
                raise ValueError(f"{file}: implausible header length {n} (file of {size} bytes)")
            header = json.loads(f.read(n))
        if not isinstance(header, dict):
            raise ValueError(f"{file}: the header is not a JSON object")
        self._data0[file] = 8 + n
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            # a damaged or truncated shard fails here, by tensor name, not later inside a view of too few bytes
            if not (isinstance(meta, dict) and isinstance(meta.get("dtype"), str) and isinstance(meta.get("shape"), list)
                    and isinstance(meta.get("data_offsets"), list) and len(meta["data_offsets"]) == 2
                    and all(isinstance(x, int) and not isinstance(x, bool) and x >= 0
                            for x in meta["shape"] + meta["data_offsets"])):
                raise ValueError(f"{file}: malformed entry for tensor {name}")
            if meta["dtype"] not in _DTYPES:
                raise ValueError(f"{file}: tensor {name} has unsupported dtype {meta['dtype']}")
            a, b = meta["data_offsets"]
            if a > b or 8 + n + b > size:
                raise ValueError(f"{file}: tensor {name} claims bytes [{a}, {b}) of a data region of {size - 8 - n}")
            self.tensors[name] = TensorInfo(file, meta["dtype"], tuple(meta["shape"]), a, b)

    def __contains__(self, name: str) -> bool:
        return name in self.tensors

    def keys(self) -> Iterable[str]:
        return self.tensors.keys()

    def _map(self, file: str) -> mmap.mmap:
        m = self._maps.get(file)
        if m is None:
            with open(file, "rb") as f:
                m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps[file] = m
        return m

    def get(self, name: str) -> torch.Tensor:
        """Zero-copy view (read-only memory: clone or move before writing)."""
        info = self.tensors[name]
        dt, size = _DTYPES[info.dtype]
        numel = 1
        for s in info.shape:
            numel *= s
        packed = info.dtype == "F4"
        nbytes = (numel + 1) // 2 if packed else numel * size
        if info.end - info.start != nbytes:
            raise ValueError(f"{name}: {info.end - info.start} bytes on disk, shape {info.shape} needs {nbytes}")
        if nbytes == 0:
            return torch.empty(info.shape, dtype=dt)
        buf = memoryview(self._map(info.file))[self._data0[info.file] + info.start:self._data0[info.file] + info.end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)       # read-only mapping: callers copy before writing
            t = torch.frombuffer(buf, dtype=torch.uint8)
        if packed:
            return t.view(*info.shape[:-1], info.shape[-1] // 2)
        return t.view(dt).view(info.shape)

    def dtype_name(self, name: str) -> str:
        return self.tensors[name].dtype

    def close(self) -> None:
        for m in self._maps.values():
            try:
                m.close()
            except BufferError:          # views still alive; the map goes with them
                pass
        self._maps.clear()


def _e8m0(scale: torch.Tensor) -> torch.Tensor:
    return torch.exp2(scale.to(torch.float32) - 127.0)


class CheckpointSource(WeightSource):
    """Master-valued tensors by checkpoint name, with shape checks."""

    def __init__(self, path: str):
        self.index = SafetensorsIndex(path)
        self.fp8_scale_rule = "absmax"           # becomes "ue8m0" when the checkpoint stores exponent bytes
        for name in self.index.keys():
            if name.endswith(".scale") and self.index.dtype_name(name) == "F8_E8M0":
                base = name[:-6] + ".weight"
                if base in self.index and self.index.dtype_name(base) == "F8_E4M3":
                    self.fp8_scale_rule = "ue8m0"
                    break

    def has(self, name: str) -> bool:
        return name in self.index

    def raw(self, name: str) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        scale_name = name[:-len(".weight")] + ".scale" if name.endswith(".weight") else None
        scale = self.index.get(scale_name) if scale_name and scale_name in self.index else None
        return self.index.get(name), scale

    def get(self, name: str, shape: Tuple[int, ...], device) -> torch.Tensor:
        if name not in self.index:
            raise KeyError(f"checkpoint has no tensor {name}")
        w, scale = self.raw(name)
        kind = self.index.dtype_name(name)
        if kind == "F8_E4M3":
            if scale is None:
                raise KeyError(f"{name} is fp8 but has no .scale sibling")
            s = _e8m0(scale) if self.index.dtype_name(name[:-7] + ".scale") == "F8_E8M0" else scale.to(torch.float32)
            out = R.dequant_fp8_block128_weight(w.to(device), s.to(device))
        elif kind in ("U8", "F4") and scale is not None:
            out = R.dequant_mxfp4(w.to(device), scale.to(device))       # packed e2m1 + ue8m0 per 32
        elif kind == "I8" and scale is not None:
            out = R.dequant_mxfp4(w.view(torch.uint8).to(device), scale.view(torch.uint8).to(device))
        else:
            out = w.to(device)
        if tuple(out.shape) != tuple(shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(out.shape)} != expected {tuple(shape)}")
        return out

    def missing(self, cfg: ModelConfig) -> List[str]:
        return [n for n in weight_shapes(cfg) if n not in self.index]

    def unexpected(self, cfg: ModelConfig) -> List[str]:
        want = set(weight_shapes(cfg))
        return [n for n in self.index.keys() if n not in want and not n.endswith(".scale")]


def load_model_config(path: str) -> ModelConfig:
    with open(os.path.join(path, "config.json")) as f:
        return model_config_from_hf(json.load(f))


# ---------------------------------------------------------------------------------------
# TP shard plan
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Shard:
    name: str
    dim: Optional[int]           # None = replicated
    start: int = 0
    stop: int = 0


def _block_range(total: int, tp: int, rank: int, block: int = FP8_BLOCK) -> Tuple[int, int]:
    """Contiguous share of `total` on whole blocks; trailing ranks may hold less (or nothing)."""
    blocks = -(-total // block)
    per = -(-blocks // tp)
    a = min(total, rank * per * block)
    return a, min(total, a + per * block)


def shard_plan(cfg: ModelConfig, tp_size: int, rank: int) -> Dict[str, Shard]:
    """name -> slice owned by `rank`.  Column-parallel: wq_b, indexer wq_b (head ranges), wo_a (groups),
    shared w1/w3, head (vocab rows); row-parallel: wo_b, shared w2 (input columns); experts by range;
    attn_sink by head range; everything else replicated."""
    out: Dict[str, Shard] = {}
    nh, D = cfg.num_attention_heads, cfg.head_dim
    if nh % tp_size or cfg.o_groups % tp_size and tp_size % cfg.o_groups:
        raise ValueError(f"tp_size {tp_size} does not divide heads {nh} / o_groups {cfg.o_groups}")
    h0, h1 = rank * nh // tp_size, (rank + 1) * nh // tp_size
    e_per = cfg.n_routed_experts // tp_size
    for name, (shape, kind) in weight_shapes(cfg).items():
        leaf = name.split(".")
        s = Shard(name, None)
        if name.endswith("attn.wq_b.weight"):
            s = Shard(name, 0, h0 * D, h1 * D)
        elif name.endswith("attn.attn_sink"):
            s = Shard(name, 0, h0, h1)
        elif name.endswith("attn.wo_a.weight"):
            g = cfg.o_groups
            s = Shard(name, 0, rank * g // tp_size * cfg.o_lora_rank, (rank + 1) * g // tp_size * cfg.o_lora_rank)
        elif name.endswith("attn.wo_b.weight"):
            s = Shard(name, 1, *_block_range(shape[1], tp_size, rank))
        elif "shared_experts" in name and leaf[-2] in ("w1", "w3"):
            s = Shard(name, 0, *_block_range(shape[0], tp_size, rank))
        elif "shared_experts" in name and leaf[-2] == "w2":
            s = Shard(name, 1, *_block_range(shape[1], tp_size, rank))
        elif ".experts." in name:
            e = int(leaf[leaf.index("experts") + 1])
            mine = rank * e_per <= e < (rank + 1) * e_per
            s = Shard(name, None) if mine else Shard(name, 0, 0, 0)
        elif name == "head.weight":
            per = -(-shape[0] // tp_size)
            s = Shard(name, 0, min(shape[0], rank * per), min(shape[0], (rank + 1) * per))
        out[name] = s
    return out


def plan_bytes(cfg: ModelConfig, tp_size: int, rank: int) -> int:
    """Bytes of weights a rank holds in the storage formats (fp8 dense, 4.5-bit experts, bf16/fp32 rest)."""
    total = 0.0
    shapes = weight_shapes(cfg)
    for name, sh in shard_plan(cfg, tp_size, rank).items():
        shape, kind = shapes[name]
        n = 1
        for i, d in enumerate(shape):
            n *= (sh.stop - sh.start) if sh.dim == i else d
        per = {"dense": 1.0 + 4.0 / (FP8_BLOCK * FP8_BLOCK) if cfg.dense_dtype == "fp8" else 2.0,
               "expert": 0.5 + 1.0 / 16 if cfg.expert_dtype != "bf16" else 2.0,
               "fp32": 4.0, "bf16": 2.0, "int": 4.0}[kind]
        total += n * per
    return int(total)


# ---------------------------------------------------------------------------------------
# writer
# ---------------------------------------------------------------------------------------
def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], dtype_names: Optional[Dict[str, str]] = None) -> None:
    header: Dict[str, Any] = {}
    blobs: List[bytes] = []
    off = 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        dn = (dtype_names or {}).get(name) or _NAMES[t.dtype]
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": dn, "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def write_checkpoint(path: str, cfg: ModelConfig, masters: Dict[str, torch.Tensor], shards: int = 2,
                     scale_rule: str = "ue8m0") -> None:
    """Write `masters` in the checkpoint's storage formats: dense -> fp8 + block scales, experts -> MXFP4."""
    import dataclasses
    os.makedirs(path, exist_ok=True)
    shapes = weight_shapes(cfg)
    out: Dict[str, torch.Tensor] = {}
    names: Dict[str, str] = {}
    for name, t in masters.items():
        kind = shapes[name][1]
        if kind == "dense" and cfg.dense_dtype == "fp8":
            q, s = R.quant_fp8_block128_weight(t.float(), ue8m0=(scale_rule == "ue8m0"))
            out[name] = q
            sn = name[:-7] + ".scale"
            if scale_rule == "ue8m0":
                out[sn] = (torch.log2(s).round() + 127).clamp(0, 255).to(torch.uint8)
                names[sn] = "F8_E8M0"
            else:
                out[sn] = s
        elif kind == "expert" and cfg.expert_dtype != "bf16":
            p, sb = R.quant_mxfp4(t.float())
            out[name], out[name[:-7] + ".scale"] = p, sb
            names[name[:-7] + ".scale"] = "F8_E8M0"
        elif kind == "fp32":
            out[name] = t.float()
        elif kind == "int":
            out[name] = t.to(torch.int32)
        else:
            out[name] = t.to(torch.bfloat16)
    keys = sorted(out)
    per = -(-len(keys) // shards)
    weight_map = {}
    for i in range(shards):
        part = keys[i * per:(i + 1) * per]
        fn = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        write_safetensors(os.path.join(path, fn), {k: out[k] for k in part}, names)
        weight_map.update({k: fn for k in part})
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    hf = {k: (list(v) if isinstance(v, tuple) else v) for k, v in dataclasses.asdict(cfg).items()}
    hf["expert_dtype"] = "fp4" if cfg.expert_dtype == "mxfp4" else cfg.expert_dtype
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(hf, f)
