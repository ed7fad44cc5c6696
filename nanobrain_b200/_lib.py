"""ctypes binding of the C ABI declared in ``include/nb_attn.h``.

The structures below mirror the header field by field. There is deliberately no fallback: if
the shared library is missing or cannot be loaded, importing an entry point raises.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libnb_attn.so"
ABI_VERSION = 2

# Every symbol include/nb_attn.h declares.
EXPORTED_SYMBOLS = (
    "nb_attn_fwd",
    "nb_attn_bwd",
    "nb_attn_bwd_workspace_bytes",
    "nb_attn_strerror",
    "nb_attn_abi_version",
    "nb_attn_selftest_mma",
    "nb_attn_bwd_builtin_scratch",
    "nb_attn_fwd_workspace_bytes",
    "nb_attn_selftest_wait",
    "nb_attn_schedule_capacity",
    "nb_attn_schedule_build",
    "nb_attn_schedule_host",
)
BUILTIN_SCRATCH_ROWS = 65536
BUILTIN_SCRATCH_ITEMS = 16384
SCHED_ITEM_INTS = 8   # an nb_attn_sched_item is eight int32: seq, tile, own begin/len, other begin/len, 2 reserved

# Codes a kernel may write to the status word (enum nb_attn_status).
STATUS_OK, STATUS_WAIT_TIMEOUT, STATUS_BAD_SEQLENS = 0, 1, 2
STATUS_TEXT = {
    STATUS_WAIT_TIMEOUT: "a bounded wait inside a kernel gave up; results are garbage",
    STATUS_BAD_SEQLENS: "cu_seqlens is not a valid packing (offsets decreasing, a sequence longer than "
                        "max_seqlen, or the last offset beyond the token count); outputs were not written",
}


class Tensor(C.Structure):
    _fields_ = [
        ("ptr", C.c_void_p),
        ("stride_batch", C.c_int64),
        ("stride_token", C.c_int64),
        ("stride_head", C.c_int64),
    ]


class Shape(C.Structure):
    _fields_ = [
        ("batch", C.c_int32),
        ("heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("max_seqlen_q", C.c_int32),
        ("max_seqlen_k", C.c_int32),
        ("total_q", C.c_int64),
        ("total_k", C.c_int64),
        ("cu_seqlens_q", C.c_void_p),
        ("cu_seqlens_k", C.c_void_p),
        ("scale", C.c_float),
    ]


class FwdArgs(C.Structure):
    _fields_ = [
        ("shape", Shape),
        ("q", Tensor),
        ("k", Tensor),
        ("v", Tensor),
        ("o", Tensor),
        ("lse", C.c_void_p),
        ("status", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("shape", Shape),
        ("q", Tensor),
        ("k", Tensor),
        ("v", Tensor),
        ("o", Tensor),
        ("d_o", Tensor),
        ("dq", Tensor),
        ("dk", Tensor),
        ("dv", Tensor),
        ("lse", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
        ("event_main_begin", C.c_void_p),
        ("event_main_end", C.c_void_p),
    ]


_lib = None


def load() -> C.CDLL:
    """Load ``libnb_attn.so`` (once) and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m nanobrain_b200.build` "
            "(there is no CPU or PyTorch fallback for this operator)"
        )
    lib = C.CDLL(str(LIB_PATH))
    lib.nb_attn_abi_version.restype = C.c_int
    lib.nb_attn_abi_version.argtypes = []
    lib.nb_attn_strerror.restype = C.c_char_p
    lib.nb_attn_strerror.argtypes = [C.c_int]
    lib.nb_attn_bwd_workspace_bytes.restype = C.c_size_t
    lib.nb_attn_bwd_workspace_bytes.argtypes = [C.POINTER(Shape)]
    lib.nb_attn_fwd_workspace_bytes.restype = C.c_size_t
    lib.nb_attn_fwd_workspace_bytes.argtypes = [C.POINTER(Shape)]
    lib.nb_attn_selftest_wait.restype = C.c_int
    lib.nb_attn_selftest_wait.argtypes = [C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.nb_attn_schedule_capacity.restype = C.c_int64
    lib.nb_attn_schedule_capacity.argtypes = [C.c_int64, C.c_int32]
    lib.nb_attn_schedule_build.restype = C.c_int
    lib.nb_attn_schedule_build.argtypes = [C.POINTER(Shape), C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
    lib.nb_attn_schedule_host.restype = C.c_int
    lib.nb_attn_schedule_host.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int64,
                                          C.c_int64, C.c_int, C.c_void_p, C.c_int64]
    lib.nb_attn_fwd.restype = C.c_int
    lib.nb_attn_fwd.argtypes = [C.POINTER(FwdArgs), C.c_void_p]
    lib.nb_attn_bwd.restype = C.c_int
    lib.nb_attn_bwd.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
    lib.nb_attn_bwd_builtin_scratch.restype = C.c_int
    lib.nb_attn_bwd_builtin_scratch.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
    lib.nb_attn_selftest_mma.restype = C.c_int
    lib.nb_attn_selftest_mma.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    got = lib.nb_attn_abi_version()
    if got != ABI_VERSION:
        raise RuntimeError(f"libnb_attn.so has ABI version {got}, this package expects {ABI_VERSION}")
    _lib = lib
    return lib


def fwd_workspace_bytes(shape: Shape) -> int:
    """Scratch bytes ``nb_attn_fwd`` needs for this shape (0 in dense mode)."""
    return int(load().nb_attn_fwd_workspace_bytes(C.byref(shape)))


def bwd_workspace_bytes(shape: Shape) -> int:
    """Scratch bytes ``nb_attn_bwd`` needs for this shape."""
    return int(load().nb_attn_bwd_workspace_bytes(C.byref(shape)))


def check(code: int, what: str) -> None:
    """Raise RuntimeError for a non-zero return code of the library."""
    if code != 0:
        msg = load().nb_attn_strerror(code).decode()
        raise RuntimeError(f"{what} failed: {msg} (code {code})")
