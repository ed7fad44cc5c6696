"""The varlen tile scheduler's work list, seen from Python.

In packed mode every attention call turns ``cu_seqlens`` into a list of (sequence, 128-row tile)
items on the device -- most expensive items first, ragged last tiles at the end -- and works through
it in that order (the forward with one CTA per item and head, the backward with one persistent CTA
per SM), so that ragged per-sample visible-token counts (the reference's
``src/nanobrain/model.py:186-199`` and its per-image eval loop at ``model.py:254-270``) do not
leave SMs idle. The calls build the list themselves; the functions here expose the same builder
for inspection and tests, on the host (no GPU needed) and on the device.
"""

from __future__ import annotations

import ctypes as C
from typing import List, Tuple

import torch
from torch import Tensor

from . import _lib

TILE = 128


def capacity(total_tokens: int, batch: int) -> int:
    """Entries a work list needs for ``batch`` sequences with ``total_tokens`` tokens in all."""
    return int(_lib.load().nb_attn_schedule_capacity(int(total_tokens), int(batch)))


def decode(items: Tensor) -> List[Tuple[int, int]]:
    """``[(sequence, tile), ...]`` of the used entries of a list (``[n, 8]`` int32 records), in list
    order. Unused entries have sequence -1."""
    rows = items.cpu().reshape(-1, _lib.SCHED_ITEM_INTS).tolist()
    return [(r[0], r[1]) for r in rows if r[0] >= 0]


def work_list_host(cu_seqlens_q: Tensor, cu_seqlens_k: Tensor, max_seqlen_q: int, max_seqlen_k: int,
                   total_q: int, total_k: int, side: int) -> Tensor:
    """The list the device kernel builds, computed on the host from CPU ``cu_seqlens`` (int32):
    ``[capacity, 8]`` int32 records (sequence, tile, own begin, own length, other begin, other
    length, two reserved).

    ``side`` 0: query tiles are the items (forward); 1: key tiles are (backward). Raises
    ``RuntimeError`` where the device would report ``STATUS_BAD_SEQLENS``."""
    cu_q = cu_seqlens_q.to(torch.int32).contiguous()
    cu_k = cu_seqlens_k.to(torch.int32).contiguous()
    batch = cu_q.numel() - 1
    n = capacity(total_q if side == 0 else total_k, batch)
    items = torch.empty((max(n, 1), _lib.SCHED_ITEM_INTS), dtype=torch.int32)
    rc = _lib.load().nb_attn_schedule_host(cu_q.data_ptr(), cu_k.data_ptr(), batch, int(max_seqlen_q),
                                          int(max_seqlen_k), int(total_q), int(total_k), int(side),
                                          items.data_ptr(), n)
    _lib.check(rc, "nb_attn_schedule_host")
    return items[:n]


def work_list_device(cu_seqlens_q: Tensor, cu_seqlens_k: Tensor, max_seqlen_q: int, max_seqlen_k: int,
                     total_q: int, total_k: int, heads: int, side: int) -> Tuple[Tensor, Tensor]:
    """Build the list on the device. Returns ``(items, status)``; ``status`` is a pinned int32 word
    that holds ``_lib.STATUS_BAD_SEQLENS`` afterwards if ``cu_seqlens`` failed the device check."""
    dev = cu_seqlens_q.device
    batch = cu_seqlens_q.numel() - 1
    n = capacity(total_q if side == 0 else total_k, batch)
    items = torch.empty((max(n, 1), _lib.SCHED_ITEM_INTS), dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32).pin_memory()
    shape = _lib.Shape(batch, heads, 64, int(max_seqlen_q), int(max_seqlen_k), int(total_q), int(total_k),
                       cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), 0.125)
    with torch.cuda.device(dev):
        rc = _lib.load().nb_attn_schedule_build(C.byref(shape), int(side), items.data_ptr(), n, status.data_ptr(),
                                               C.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(rc, "nb_attn_schedule_build")
    return items[:n], status


def selftest_wait(limit_ns: int, device: torch.device) -> Tuple[int, Tensor]:
    """Run the bounded-wait self-test (``nb_attn_selftest_wait``): one CTA waits ``limit_ns`` for a
    barrier nobody arrives on. Returns ``(status code, out)`` after synchronising; the expected
    result is ``(_lib.STATUS_WAIT_TIMEOUT, [1, 1])``."""
    status = torch.zeros(1, dtype=torch.int32).pin_memory()
    out = torch.zeros(2, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        rc = _lib.load().nb_attn_selftest_wait(int(limit_ns), status.data_ptr(), out.data_ptr(),
                                              C.c_void_p(torch.cuda.current_stream().cuda_stream))
        _lib.check(rc, "nb_attn_selftest_wait")
        torch.cuda.synchronize(device)
    return int(status[0]), out.cpu()
