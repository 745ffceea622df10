"""ctypes binding of the C ABI in ``include/acache_b200.h``.

The shared library is built in-tree by ``python -m acache_b200.build`` and loaded
from ``acache_b200/csrc``.  There is no fallback: if the library is missing or a
call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "csrc" / "libacache_b200.so"

F32, F16, BF16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

_SIGNATURES = {
    "acache_status_string": (c_char_p, [c_int]),
    "acache_last_cuda_error": (c_char_p, []),
    "acache_abi_version": (c_int, []),
    "acache_store_kvcache": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                     c_int64, c_int, c_void_p, c_void_p]),
    "acache_relocate_affix": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int64, c_int, c_int, c_int, c_void_p,
                                      c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                      c_int, c_int, c_void_p, c_void_p]),
    "acache_rope_store": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                                  c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p,
                                  c_void_p, c_int64, c_void_p, c_void_p]),
    "acache_anchor_topk": (c_int, [c_void_p, c_int, c_int, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "acache_anchor_importance_scratch_bytes": (c_int64, [c_int, c_int, c_int]),
    "acache_anchor_importance": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                         c_int64, c_int, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_float,
                                         c_void_p, c_void_p, c_int64, c_void_p]),
    "acache_attention": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int,
                                 c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_float, c_int,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "acache_paged_attention": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int,
                                       c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                                       c_int, c_float, c_void_p, c_void_p]),
    "acache_rmsnorm": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_int, c_void_p]),
    "acache_act_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "acache_transfer_tokens": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_int, c_int64, c_float,
                                       c_void_p, c_void_p, c_void_p]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


class AcacheError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Loads the library (once) and installs argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise AcacheError(
            f"{LIB_PATH} is missing: build it with `python -m acache_b200.build` (needs nvcc); "
            "there is no CPU or PyTorch fallback for these operators")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}") from None


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(status: int, what: str):
    if status == 0:
        return
    lib = load()
    msg = lib.acache_status_string(status).decode()
    if status == -3:
        msg += ": " + lib.acache_last_cuda_error().decode()
    if status == -1:
        raise ValueError(f"{what}: {msg}")
    if status == -2:
        raise NotImplementedError(f"{what}: {msg}")
    raise AcacheError(f"{what}: {msg}")


# ---- device-side error flag ---------------------------------------------------------
_err_flags: dict[int, torch.Tensor] = {}


def err_flag(device: torch.device) -> torch.Tensor:
    """One int32 per device that kernels raise when they meet an out-of-range slot,
    block id or table row (they skip the access instead of faulting)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    flag = _err_flags.get(idx)
    if flag is None:
        flag = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _err_flags[idx] = flag
    return flag


_ERR_TEXT = {1: "slot outside the cache", 2: "position outside the RoPE table", 3: "read slot outside the cache",
             4: "relocation shift outside the RoPE table"}


def check_device_errors(device: torch.device | None = None):
    """Synchronises and raises if any kernel flagged a bad index since the last check."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    flag = err_flag(device)
    code = int(flag.item())
    if code:
        flag.zero_()
        raise AcacheError(f"device-side index check failed: {_ERR_TEXT.get(code, code)}")
