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
    "acache_qkv_rope_scatter": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_int64,
                                        c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "acache_linear": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int64, c_int,
                              c_int, c_void_p, c_void_p]),
    "acache_linear_partials_splits": (c_int, [c_int, c_int, c_int]),
    "acache_linear_partials": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                                       c_int, c_void_p, c_void_p]),
    "acache_linear_swiglu": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int64,
                                     c_int, c_int, c_void_p, c_void_p]),
    "acache_linear_qkv_rope_scatter": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                               c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                                               c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                                               c_void_p]),
    "acache_linear_argmax_scratch_bytes": (c_int64, [c_int, c_int]),
    "acache_linear_argmax": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "acache_diag_mma_rate": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "acache_anchor_topk": (c_int, [c_void_p, c_int, c_int, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "acache_anchor_importance_scratch_bytes": (c_int64, [c_int, c_int, c_int]),
    "acache_anchor_importance": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                         c_int64, c_int, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_float,
                                         c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "acache_anchor_importance_batched_scratch_bytes": (c_int64, [c_int, c_int, c_int, c_int]),
    "acache_anchor_importance_batched": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                 c_int, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p,
                                                 c_int64, c_int, c_int, c_float, c_void_p, c_int64, c_void_p, c_int64,
                                                 c_void_p, c_void_p]),
    "acache_anchor_importance_static_scratch_bytes": (c_int64, []),
    "acache_anchor_importance_static": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int64, c_int,
                                                c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "acache_attention": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int,
                                 c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_float, c_int,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "acache_attention_grouped_scratch_bytes": (c_int64, [c_int, c_int, c_int, c_int, c_int]),
    "acache_attention_grouped": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int,
                                         c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                         c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                         c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "acache_paged_attention": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int,
                                       c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                                       c_int, c_float, c_void_p, c_void_p]),
    "acache_rmsnorm": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_int, c_void_p]),
    "acache_add_rmsnorm": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int,
                                   c_float, c_int, c_void_p]),
    "acache_add_rmsnorm_partials": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p,
                                            c_int64, c_int, c_int, c_float, c_int, c_void_p]),
    "acache_act_mul_halves": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "acache_act_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "acache_apply_transfer": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_float, c_void_p]),
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


# kernels launched through this binding since import (the benchmark reads the difference)
LAUNCHES = 0

# optional per-operator device timing: name -> {"events": [(start, end), ...] of eager calls,
# "ms"/"n": time and count harvested from graph replays, "work": work units of all of them}
_TIMERS: dict | None = None
# while a CUDA graph is being captured: the (name, start, end) event pairs recorded inside it
_GRAPH_EVENTS: list | None = None


def enable_kernel_timers(on: bool = True):
    """Brackets every call of a timed operator with CUDA events on the launching stream.
    Off by default; the benchmark turns it on to measure the dominant kernel live."""
    global _TIMERS
    _TIMERS = {} if on else None


def kernel_timers_enabled() -> bool:
    return _TIMERS is not None


def _timer_record(name: str) -> dict:
    return _TIMERS.setdefault(name, {"events": [], "work": 0.0, "ms": 0.0, "n": 0})


def kernel_timers() -> dict:
    """name -> (total_ms, launches, work) resolved from the recorded events."""
    out = {}
    if _TIMERS:
        torch.cuda.synchronize()
        for name, rec in _TIMERS.items():
            out[name] = (sum(a.elapsed_time(b) for a, b in rec["events"]) + rec["ms"], len(rec["events"]) + rec["n"],
                         rec["work"])
    return out


def begin_graph_capture() -> list:
    """Timed operators called until ``end_graph_capture`` record EXTERNAL events (event-record
    nodes of the graph being captured) and list them in the returned list."""
    global _GRAPH_EVENTS
    _GRAPH_EVENTS = []
    return _GRAPH_EVENTS


def end_graph_capture():
    global _GRAPH_EVENTS
    _GRAPH_EVENTS = None


def harvest_graph_timers(events: list, work: float):
    """Adds the times between the event pairs of a graph whose last replay HAS COMPLETED."""
    if _TIMERS is None:
        return
    for name, a, b in events:
        rec = _timer_record(name)
        rec["ms"] += a.elapsed_time(b)
        rec["n"] += 1
        rec["work"] += work


class timed:
    """``with timed(name, work): launch`` - a no-op unless timers are enabled."""

    __slots__ = ("name", "work", "start")

    def __init__(self, name: str, work: float = 0.0):
        self.name, self.work, self.start = name, work, None

    def __enter__(self):
        if _TIMERS is not None:
            self.start = torch.cuda.Event(enable_timing=True, external=_GRAPH_EVENTS is not None)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if self.start is not None:
            end = torch.cuda.Event(enable_timing=True, external=_GRAPH_EVENTS is not None)
            end.record()
            if _GRAPH_EVENTS is not None:
                _GRAPH_EVENTS.append((self.name, self.start, end))
            else:
                rec = _timer_record(self.name)
                rec["events"].append((self.start, end))
                rec["work"] += self.work
        return False


def check(status: int, what: str, launches: int = 1):
    global LAUNCHES
    if status == 0:
        LAUNCHES += launches
        return
    lib = load()
    msg = lib.acache_status_string(status).decode()
    if status == -3:
        msg += ": " + lib.acache_last_cuda_error().decode()
    if status == -1:
        raise ValueError(f"{what}: {msg}")
    if status == -4:
        raise OverflowError(f"{what}: {msg}")
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
        # made (and later cleared) under inference mode so that it can be reset no matter
        # whether the caller runs inside or outside of torch.inference_mode()
        with torch.inference_mode():
            flag = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _err_flags[idx] = flag
    return flag


def existing_err_flag(device: torch.device):
    """The device's error flag if some earlier call already made it, else None; for callers
    that must not cause an allocation themselves."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return _err_flags.get(idx)


_ERR_TEXT = {1: "slot outside the cache", 2: "position outside the RoPE table", 3: "read slot outside the cache",
             4: "relocation shift outside the RoPE table", 5: "a bounded wait inside a kernel ran out",
             6: "shared memory of a tensor-core kernel is not 1024-byte aligned",
             7: "requests of a group do not name the same shared span"}
ACACHE_EUNSUPPORTED = -2


def check_device_errors(device: torch.device | None = None):
    """Synchronises and raises if any kernel flagged a bad index since the last check."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    flag = err_flag(device)
    code = int(flag.item())
    if code:
        with torch.inference_mode():
            flag.zero_()
        from .model.acache_attention import reset_grouped_scratch

        reset_grouped_scratch()  # its tickets may have been left odd by the failed call
        raise AcacheError(f"device-side index check failed: {_ERR_TEXT.get(code, code)}")
