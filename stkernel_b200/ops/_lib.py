"""ctypes binding of ``libstk_b200.so`` (the sm_100a kernels).

``call(name, *args)`` passes tensors as raw device pointers and appends nothing
implicitly; the caller supplies the CUDA stream through :func:`stream`.  On a
machine with a GPU a missing library is an error (ops never fall back silently
to PyTorch there); on a CPU-only machine the ops use the reference statements.
"""
from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path
from typing import Any, Dict, Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "libstk_b200.so"
_lib: Optional[ctypes.CDLL] = None

_CSRC = Path(__file__).resolve().parent.parent / "csrc"
_DECL = re.compile(r"STK_API\s+(int|long long)\s+(stk_\w+)\s*\(([^)]*)\)", re.S)


def _parse_signatures() -> Dict[str, tuple]:
    """Read every `STK_API` declaration from the .cu sources: name -> (restype, [argtypes])."""
    out: Dict[str, tuple] = {}
    for src in sorted(_CSRC.glob("*.cu")):
        for ret, name, args in _DECL.findall(src.read_text()):
            types = []
            for a in [x.strip() for x in args.split(",") if x.strip()]:
                if "*" in a:
                    types.append(ctypes.c_void_p)
                elif a.startswith("long long"):
                    types.append(ctypes.c_longlong)
                elif a.startswith("float"):
                    types.append(ctypes.c_float)
                elif a.startswith("int"):
                    types.append(ctypes.c_int)
                else:
                    raise RuntimeError(f"unhandled parameter {a!r} in {name}")
            out[name] = (ctypes.c_longlong if ret == "long long" else ctypes.c_int, types)
    return out


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: run `python -m stkernel_b200.csrc.build` (the CUDA ops have no fallback "
                "on a GPU machine)")
        _lib = ctypes.CDLL(str(_LIB_PATH), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else ctypes.DEFAULT_MODE)
        for name, (ret, types) in _parse_signatures().items():
            fn = getattr(_lib, name)
            fn.argtypes = types
            fn.restype = ret
    return _lib


def use_cuda(t: torch.Tensor) -> bool:
    """True when `t` lives on a GPU, in which case the CUDA library must be used."""
    return t.is_cuda


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class KernelError(RuntimeError):
    pass


launch_count = 0


def call(name: str, *args: Any) -> int:
    """Launch `name`; tensors become pointers.  Raises on a rejected launch."""
    global launch_count
    fn = getattr(lib(), name)
    conv = [a.data_ptr() if isinstance(a, torch.Tensor) else a for a in args]
    rc = fn(*conv)
    if rc != 0:
        raise KernelError(f"{name} returned {rc}")
    launch_count += 1
    return rc


def query(name: str, *args: int) -> int:
    return getattr(lib(), name)(*args)


_sm_count: Dict[int, int] = {}


def sm_count() -> int:
    d = torch.cuda.current_device()
    if d not in _sm_count:
        _sm_count[d] = torch.cuda.get_device_properties(d).multi_processor_count
    return _sm_count[d]


_status: Dict[int, torch.Tensor] = {}


def status_buffer() -> torch.Tensor:
    """Per-device int32[2] status word shared by all kernels (0 = ok)."""
    d = torch.cuda.current_device()
    if d not in _status:
        _status[d] = torch.zeros(2, dtype=torch.int32, device=f"cuda:{d}")
    return _status[d]


def check_status() -> None:
    """Host-side check (synchronises): raises if any kernel recorded a bounded-wait timeout or a bad index."""
    st = status_buffer().tolist()
    if st[0] != 0:
        status_buffer().zero_()
        names = {1: "mbarrier wait timed out", 2: "peer flag wait timed out", 3: "index out of range",
                 4: "local flag wait timed out"}
        raise KernelError(f"device status {st[0]} ({names.get(st[0], '?')}), detail {st[1]}")
