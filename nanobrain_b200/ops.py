"""``torch.library`` custom ops over the C-ABI attention library.

Two public entry points:

``sdpa(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False)``
    Same signature as ``F.scaled_dot_product_attention`` and a drop-in for the call at
    ``src/nanobrain/modules.py:62`` of the reference (``F.scaled_dot_product_attention(q, k, v,
    is_causal=self.causal)`` with ``causal=False``): logical ``[B, H, L, 64]`` bf16 CUDA tensors,
    no mask, no dropout, non-causal. The result is logical ``[B, H, L, 64]`` backed by
    ``[B, L, H, 64]`` memory so the head merge at ``modules.py:63`` stays a view.

``sdpa_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale=None)``
    Packed variable-length form: ``[T, H, 64]`` tokens, sequence ``i`` owns rows
    ``[cu_seqlens[i], cu_seqlens[i+1])``. ``max_seqlen_*`` are host integers, so the call never
    synchronises with the device.

Anything outside that subset raises; there is no fallback and no backend dispatch. Both ops
carry fake (meta) kernels and autograd formulas, so they trace under ``torch.compile`` and
``loss.backward()`` reaches the CUDA backward (``src/nanobrain/misc.py:368-371``).
"""

from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional

import torch
from torch import Tensor

from . import _lib

HEAD_DIM = 64
_DEBUG = os.environ.get("NB_ATTN_DEBUG", "0") == "1"

_status_words: dict[int, Tensor] = {}


def _status_word(device: torch.device) -> Tensor:
    """One int32 per device that kernels write to when something went wrong on the device.

    The word lives in pinned host memory, which the GPU addresses directly: a kernel's rare write
    goes over the bus, and the host can look at the word at any time without synchronising."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32).pin_memory()
        _status_words[idx] = t
    return t


def _raise_for_status(word: Tensor) -> None:
    code = int(word[0])
    if code != 0:
        word.zero_()
        text = _lib.STATUS_TEXT.get(code, "unknown code")
        raise RuntimeError(f"nanobrain_b200 attention kernel reported device status {code}: {text}")


def poll_status(device: Optional[torch.device] = None) -> None:
    """Raise if a kernel that has already finished reported a problem. Never synchronises: every
    op calls this before it launches, so a failed step surfaces at the next attention call."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _raise_for_status(_status_word(device))


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise with ``device`` and raise if any kernel launched so far reported a problem.
    Call it where the training step synchronises anyway (for example where the loss is read)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    torch.cuda.synchronize(device)
    _raise_for_status(_status_word(device))


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError("nanobrain_b200.sdpa: " + msg)


def _check_qkv(q: Tensor, k: Tensor, v: Tensor, ndim: int) -> None:
    for name, t in (("query", q), ("key", k), ("value", v)):
        _require(t.is_cuda, f"{name} must be a CUDA tensor (there is no CPU path)")
        _require(t.dtype == torch.bfloat16, f"{name} must be bfloat16, got {t.dtype}")
        _require(t.dim() == ndim, f"{name} must have {ndim} dimensions, got {t.dim()}")
        _require(t.shape[-1] == HEAD_DIM, f"head_dim must be {HEAD_DIM}, got {t.shape[-1]}")
    _require(q.device == k.device == v.device, "query, key and value must be on the same device")
    _require(k.shape == v.shape, "key and value must have the same shape")


def _strides_ok(t: Tensor) -> bool:
    if t.stride(-1) != 1 or t.data_ptr() % 16 != 0:
        return False
    for size, stride in zip(t.shape[:-1], t.stride()[:-1]):
        if size > 1 and (stride <= 0 or stride % 8 != 0):
            return False
    return True


def _dense_layout(t: Tensor) -> Tensor:
    """Return ``t`` (logical [B,H,L,64]) if the kernels can address it, else a [B,L,H,64]-memory copy."""
    if _strides_ok(t):
        return t
    return t.transpose(1, 2).contiguous().transpose(1, 2)


def _packed_layout(t: Tensor) -> Tensor:
    return t if _strides_ok(t) else t.contiguous()


def _dense_desc(t: Tensor) -> _lib.Tensor:
    b, h, l, d = t.shape
    sb = t.stride(0) if b > 1 else h * l * d
    sh = t.stride(1) if h > 1 else d
    st = t.stride(2) if l > 1 else h * d
    return _lib.Tensor(t.data_ptr(), sb, st, sh)


def _packed_desc(t: Tensor) -> _lib.Tensor:
    n, h, d = t.shape
    st = t.stride(0) if n > 1 else h * d
    sh = t.stride(1) if h > 1 else d
    return _lib.Tensor(t.data_ptr(), 0, st, sh)


def _new_dense(like: Tensor) -> Tensor:
    b, h, l, d = like.shape
    return like.new_empty((b, l, h, d)).transpose(1, 2)


def _stream_ptr() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _before_launch(device: torch.device) -> None:
    poll_status(device)


def _after_launch(device: torch.device) -> None:
    if _DEBUG:
        check_status(device)


# ------------------------------------------------------------------------------------------
# Dense ops
# ------------------------------------------------------------------------------------------
@torch.library.custom_op("nanobrain_b200::sdpa_fwd", mutates_args=(), device_types="cuda")
def sdpa_fwd(q: Tensor, k: Tensor, v: Tensor, scale: float) -> tuple[Tensor, Tensor]:
    _check_qkv(q, k, v, 4)
    b, h, lq, d = q.shape
    _require(k.shape[0] == b and k.shape[1] == h, "query and key must agree on batch and heads (no GQA)")
    lk = k.shape[2]
    _require(b > 0 and h > 0 and lq > 0 and lk > 0, "empty tensors are not supported")
    q, k, v = _dense_layout(q), _dense_layout(k), _dense_layout(v)
    out = _new_dense(q)
    lse = torch.empty((b, h, lq), dtype=torch.float32, device=q.device)
    lib = _lib.load()
    _before_launch(q.device)
    with torch.cuda.device(q.device):
        args = _lib.FwdArgs(
            _lib.Shape(b, h, d, lq, lk, b * lq, b * lk, None, None, scale),
            _dense_desc(q), _dense_desc(k), _dense_desc(v), _dense_desc(out),
            lse.data_ptr(), _status_word(q.device).data_ptr(), None, 0,
        )
        _lib.check(lib.nb_attn_fwd(C.byref(args), _stream_ptr()), "nb_attn_fwd")
    _after_launch(q.device)
    return out, lse


@sdpa_fwd.register_fake
def _(q, k, v, scale):
    b, h, lq, d = q.shape
    return _new_dense(q), q.new_empty((b, h, lq), dtype=torch.float32)


@torch.library.custom_op("nanobrain_b200::sdpa_bwd", mutates_args=(), device_types="cuda")
def sdpa_bwd(
    d_out: Tensor, q: Tensor, k: Tensor, v: Tensor, out: Tensor, lse: Tensor, scale: float
) -> tuple[Tensor, Tensor, Tensor]:
    _check_qkv(q, k, v, 4)
    b, h, lq, d = q.shape
    lk = k.shape[2]
    q, k, v = _dense_layout(q), _dense_layout(k), _dense_layout(v)
    out, d_out = _dense_layout(out), _dense_layout(d_out)
    _require(d_out.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "out and d_out must be bfloat16")
    lse = lse.contiguous()
    dq, dk, dv = _new_dense(q), _new_dense(k), _new_dense(v)
    lib = _lib.load()
    _before_launch(q.device)
    shape = _lib.Shape(b, h, d, lq, lk, b * lq, b * lk, None, None, scale)
    ws_bytes = _lib.bwd_workspace_bytes(shape)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        args = _lib.BwdArgs(
            shape,
            _dense_desc(q), _dense_desc(k), _dense_desc(v), _dense_desc(out), _dense_desc(d_out),
            _dense_desc(dq), _dense_desc(dk), _dense_desc(dv),
            lse.data_ptr(), workspace.data_ptr(), ws_bytes, _status_word(q.device).data_ptr(),
        )
        _lib.check(lib.nb_attn_bwd(C.byref(args), _stream_ptr()), "nb_attn_bwd")
    _after_launch(q.device)
    return dq, dk, dv


@sdpa_bwd.register_fake
def _(d_out, q, k, v, out, lse, scale):
    return _new_dense(q), _new_dense(k), _new_dense(v)


def _sdpa_setup(ctx, inputs, output):
    q, k, v, scale = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse)
    ctx.scale = scale


def _sdpa_backward(ctx, d_out, d_lse):
    q, k, v, out, lse = ctx.saved_tensors
    dq, dk, dv = sdpa_bwd(d_out, q, k, v, out, lse, ctx.scale)
    return dq, dk, dv, None


sdpa_fwd.register_autograd(_sdpa_backward, setup_context=_sdpa_setup)


# ------------------------------------------------------------------------------------------
# Varlen ops
# ------------------------------------------------------------------------------------------
def _check_cu(cu: Tensor, name: str, device: torch.device) -> None:
    _require(cu.dtype == torch.int32 and cu.dim() == 1 and cu.numel() >= 2, f"{name} must be int32 [B+1]")
    _require(cu.device == device, f"{name} must live on the same device as the tokens")
    _require(cu.is_contiguous(), f"{name} must be contiguous")


@torch.library.custom_op("nanobrain_b200::sdpa_varlen_fwd", mutates_args=(), device_types="cuda")
def sdpa_varlen_fwd(
    q: Tensor, k: Tensor, v: Tensor, cu_seqlens_q: Tensor, cu_seqlens_k: Tensor,
    max_seqlen_q: int, max_seqlen_k: int, scale: float,
) -> tuple[Tensor, Tensor]:
    _check_qkv(q, k, v, 3)
    _check_cu(cu_seqlens_q, "cu_seqlens_q", q.device)
    _check_cu(cu_seqlens_k, "cu_seqlens_k", q.device)
    _require(cu_seqlens_q.numel() == cu_seqlens_k.numel(), "cu_seqlens_q and cu_seqlens_k must have the same length")
    tq, h, d = q.shape
    tk = k.shape[0]
    _require(k.shape[1] == h, "query and key must agree on heads (no GQA)")
    _require(tq > 0 and tk > 0 and max_seqlen_q > 0 and max_seqlen_k > 0, "empty tensors are not supported")
    nseq = cu_seqlens_q.numel() - 1
    q, k, v = _packed_layout(q), _packed_layout(k), _packed_layout(v)
    out = torch.empty((tq, h, d), dtype=q.dtype, device=q.device)
    lse = torch.empty((h, tq), dtype=torch.float32, device=q.device)
    lib = _lib.load()
    _before_launch(q.device)
    shape = _lib.Shape(nseq, h, d, max_seqlen_q, max_seqlen_k, tq, tk,
                       cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), scale)
    ws_bytes = _lib.fwd_workspace_bytes(shape)  # the scheduler's work list
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        args = _lib.FwdArgs(
            shape, _packed_desc(q), _packed_desc(k), _packed_desc(v), _packed_desc(out),
            lse.data_ptr(), _status_word(q.device).data_ptr(), workspace.data_ptr(), ws_bytes,
        )
        _lib.check(lib.nb_attn_fwd(C.byref(args), _stream_ptr()), "nb_attn_fwd")
    _after_launch(q.device)
    return out, lse


@sdpa_varlen_fwd.register_fake
def _(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale):
    tq, h, d = q.shape
    return q.new_empty((tq, h, d)), q.new_empty((h, tq), dtype=torch.float32)


@torch.library.custom_op("nanobrain_b200::sdpa_varlen_bwd", mutates_args=(), device_types="cuda")
def sdpa_varlen_bwd(
    d_out: Tensor, q: Tensor, k: Tensor, v: Tensor, out: Tensor, lse: Tensor,
    cu_seqlens_q: Tensor, cu_seqlens_k: Tensor, max_seqlen_q: int, max_seqlen_k: int, scale: float,
) -> tuple[Tensor, Tensor, Tensor]:
    _check_qkv(q, k, v, 3)
    tq, h, d = q.shape
    tk = k.shape[0]
    nseq = cu_seqlens_q.numel() - 1
    q, k, v = _packed_layout(q), _packed_layout(k), _packed_layout(v)
    out, d_out = _packed_layout(out), _packed_layout(d_out)
    _require(d_out.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "out and d_out must be bfloat16")
    lse = lse.contiguous()
    dq = torch.empty((tq, h, d), dtype=q.dtype, device=q.device)
    dk = torch.empty((tk, h, d), dtype=q.dtype, device=q.device)
    dv = torch.empty((tk, h, d), dtype=q.dtype, device=q.device)
    lib = _lib.load()
    _before_launch(q.device)
    shape = _lib.Shape(nseq, h, d, max_seqlen_q, max_seqlen_k, tq, tk,
                       cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), scale)
    ws_bytes = _lib.bwd_workspace_bytes(shape)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        args = _lib.BwdArgs(
            shape,
            _packed_desc(q), _packed_desc(k), _packed_desc(v), _packed_desc(out), _packed_desc(d_out),
            _packed_desc(dq), _packed_desc(dk), _packed_desc(dv),
            lse.data_ptr(), workspace.data_ptr(), ws_bytes, _status_word(q.device).data_ptr(),
        )
        _lib.check(lib.nb_attn_bwd(C.byref(args), _stream_ptr()), "nb_attn_bwd")
    _after_launch(q.device)
    return dq, dk, dv


@sdpa_varlen_bwd.register_fake
def _(d_out, q, k, v, out, lse, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, scale):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _varlen_setup(ctx, inputs, output):
    q, k, v, cu_q, cu_k, max_q, max_k, scale = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse, cu_q, cu_k)
    ctx.max_q, ctx.max_k, ctx.scale = max_q, max_k, scale


def _varlen_backward(ctx, d_out, d_lse):
    q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
    dq, dk, dv = sdpa_varlen_bwd(d_out, q, k, v, out, lse, cu_q, cu_k, ctx.max_q, ctx.max_k, ctx.scale)
    return dq, dk, dv, None, None, None, None, None


sdpa_varlen_fwd.register_autograd(_varlen_backward, setup_context=_varlen_setup)


# ------------------------------------------------------------------------------------------
# FLOP formulas: the reference measures TFLOP/s with ``FlopCounterMode`` over one forward +
# backward (``src/nanobrain/train.py:414-432``); a custom op is invisible to it unless a formula
# is registered. Same convention as torch's own SDPA formulas: 2 GEMMs forward, 5 backward.
# ------------------------------------------------------------------------------------------
def _pair_sum(cu_q: Tensor, cu_k: Tensor) -> int:
    lq = (cu_q[1:] - cu_q[:-1]).to(torch.int64)
    lk = (cu_k[1:] - cu_k[:-1]).to(torch.int64)
    return int((lq * lk).sum().item())


def _register_flop_formulas() -> None:
    from torch.utils.flop_counter import register_flop_formula

    @register_flop_formula(torch.ops.nanobrain_b200.sdpa_fwd)
    def _(q_shape, k_shape, v_shape, scale, *args, out_shape=None, **kwargs) -> int:
        b, h, lq, d = q_shape
        return 4 * b * h * lq * k_shape[2] * d

    @register_flop_formula(torch.ops.nanobrain_b200.sdpa_bwd)
    def _(d_out_shape, q_shape, k_shape, *args, out_shape=None, **kwargs) -> int:
        b, h, lq, d = q_shape
        return 10 * b * h * lq * k_shape[2] * d

    # The varlen formulas need the lengths, i.e. tensor values: get_raw=True hands over the tensors.
    @register_flop_formula(torch.ops.nanobrain_b200.sdpa_varlen_fwd, get_raw=True)
    def _(q, k, v, cu_q, cu_k, *args, out_val=None, **kwargs) -> int:
        return 4 * q.shape[1] * q.shape[2] * _pair_sum(cu_q, cu_k)

    @register_flop_formula(torch.ops.nanobrain_b200.sdpa_varlen_bwd, get_raw=True)
    def _(d_out, q, k, v, out, lse, cu_q, cu_k, *args, out_val=None, **kwargs) -> int:
        return 10 * q.shape[1] * q.shape[2] * _pair_sum(cu_q, cu_k)


_register_flop_formulas()


# ------------------------------------------------------------------------------------------
# Public functions
# ------------------------------------------------------------------------------------------
def sdpa(
    query: Tensor,
    key: Tensor,
    value: Tensor,
    attn_mask: Optional[Tensor] = None,
    dropout_p: float = 0.0,
    is_causal: bool = False,
    scale: Optional[float] = None,
    enable_gqa: bool = False,
) -> Tensor:
    """Drop-in for ``F.scaled_dot_product_attention`` as called at ``src/nanobrain/modules.py:62``."""
    _require(attn_mask is None, "attn_mask is not supported (the reference passes none)")
    _require(dropout_p == 0.0, "dropout_p must be 0.0")
    _require(not is_causal, "is_causal=True is not supported (the reference's blocks are bidirectional)")
    _require(not enable_gqa, "enable_gqa is not supported")
    scale = 1.0 / math.sqrt(query.shape[-1]) if scale is None else float(scale)
    out, _ = sdpa_fwd(query, key, value, scale)
    return out


def sdpa_varlen(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    cu_seqlens_q: Tensor,
    cu_seqlens_k: Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    scale: Optional[float] = None,
) -> Tensor:
    """Bidirectional attention over packed ``[T, H, 64]`` tokens addressed by ``cu_seqlens``."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)
    out, _ = sdpa_varlen_fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q), int(max_seqlen_k), scale)
    return out


def selftest_mma(mode: int, a: Tensor, b: Tensor) -> Tensor:
    """Run one tensor-core operand form on a [128,128] bf16 pair; see ``nb_attn_selftest_mma``."""
    _require(a.is_cuda and b.is_cuda and a.dtype == b.dtype == torch.bfloat16, "a and b must be CUDA bfloat16")
    _require(a.shape == (128, 128) and b.shape == (128, 128), "a and b must be [128, 128]")
    a, b = a.contiguous(), b.contiguous()
    d = torch.empty((128, 128 if mode == 0 else 64), dtype=torch.float32, device=a.device)
    lib = _lib.load()
    with torch.cuda.device(a.device):
        _lib.check(
            lib.nb_attn_selftest_mma(mode, a.data_ptr(), b.data_ptr(), d.data_ptr(),
                                     _status_word(a.device).data_ptr(), _stream_ptr()),
            "nb_attn_selftest_mma",
        )
    return d
