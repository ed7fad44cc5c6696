"""Packed-token preparation for the varlen attention path.

The reference encodes a FIXED number of visible patches per sequence (``num_visible``, padded
with background patches when a volume has too few in-mask patches:
``src/nanobrain/model.py:186-199`` and ``sample_sequences`` at ``model.py:347-363``). With a varlen
attention operator every sequence can instead keep its own number of visible patches; this module
builds that packed layout: one ``[T, ...]`` token axis holding all sequences back to back plus
``cu_seqlens`` (int32 ``[B+1]``), which is exactly what ``nanobrain_b200.sdpa_varlen`` and the
packed path of ``nanobrain_b200.modules.Attention`` consume.

Everything here is plain torch index arithmetic and runs on any device.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor


def visible_counts(mask_frac: Tensor, visible_ratio: float, min_mask_frac: float = 0.25, min_visible: int = 1) -> Tensor:
    """Per-sample number of visible patches: ``visible_ratio`` of the patches whose mask fraction
    reaches ``min_mask_frac`` (the in-mask test of ``sample_sequences``, ``model.py:354,361``)."""
    in_mask = (mask_frac >= min_mask_frac).sum(dim=1)
    return torch.clamp((in_mask.to(torch.float32) * visible_ratio).floor().to(torch.int64), min=min_visible)


def sample_order(mask_frac: Tensor, num_samples: int = 1, min_mask_frac: float = 0.25,
                 generator: Optional[torch.Generator] = None) -> Tensor:
    """Random patch order per (image, sample) with out-of-mask patches sorted last -- the rule of
    ``sample_sequences`` (``model.py:347-363``): uniform scores, 2.0 for patches outside the mask,
    argsort. Returns int64 ``[B, S, P]``."""
    b, p = mask_frac.shape
    scores = torch.rand(b, num_samples, p, device=mask_frac.device, generator=generator)
    scores = torch.where(mask_frac[:, None, :] >= min_mask_frac, scores, torch.full_like(scores, 2.0))
    return scores.argsort(dim=2)


def cu_seqlens_from_counts(counts: Tensor) -> Tensor:
    """int32 ``[N+1]`` exclusive prefix sums of per-sequence token counts (stays on ``counts.device``)."""
    cu = torch.zeros(counts.numel() + 1, dtype=torch.int32, device=counts.device)
    cu[1:] = torch.cumsum(counts.reshape(-1), 0).to(torch.int32)
    return cu


def packed_gather_index(order: Tensor, counts: Tensor, capacity: Optional[int] = None):
    """Flat gather index for packing the first ``counts[i]`` entries of every row of ``order``.

    ``order``: int64 ``[N, P]`` (patch ids per sequence, most wanted first); ``counts``: int64 ``[N]``.
    Returns ``(seq_id [T], patch_id [T], cu_seqlens [N+1] int32, valid [T] bool)``.

    With ``capacity=None`` the packed length is the exact total, which costs ONE device-to-host
    sync (the reference pays the same sync at ``model.py:359-361``). With an integer ``capacity``
    (a host-known upper bound, e.g. ``N * max_visible``) nothing synchronises: the outputs have
    ``capacity`` rows, rows past ``cu_seqlens[-1]`` are padding (``valid`` False, indices clamped
    to a real patch) and are never attended to because no sequence owns them."""
    n, p = order.shape
    cu = cu_seqlens_from_counts(counts)
    total = int(cu[-1].item()) if capacity is None else int(capacity)
    pos = torch.arange(total, device=order.device, dtype=torch.int64)
    # sequence owning each packed row: number of sequence ends that are <= row
    seq_id = torch.searchsorted(cu[1:].to(torch.int64), pos, right=True)
    valid = seq_id < n
    seq_id = torch.clamp(seq_id, max=n - 1)
    within = pos - cu[:-1].to(torch.int64)[seq_id]
    within = torch.clamp(within, min=0, max=p - 1)
    patch_id = order[seq_id, within]
    return seq_id, patch_id, cu, valid


def pack_visible_tokens(patches: Tensor, coords: Tensor, order: Tensor, counts: Tensor,
                        capacity: Optional[int] = None):
    """Gather the visible patches of every sequence into the packed layout.

    ``patches``: ``[B, P, patch_dim]``; ``coords``: ``[B, P, 3]`` (or ``[1, P, 3]`` broadcast);
    ``order``: ``[B, S, P]`` from :func:`sample_order`; ``counts``: ``[B]`` or ``[B, S]`` visible
    patches per sequence. Replaces the fixed-length gather + split of ``model.py:188-197``.

    Returns ``(tokens [T, patch_dim], token_coords [T, 3], cu_seqlens int32 [B*S+1], seq_id [T],
    patch_id [T], valid [T])``; the (image, sample) pairs are flattened image-major like
    ``.flatten(0, 1)`` at ``model.py:189``."""
    b, s, p = order.shape
    counts = counts.reshape(b, -1).expand(b, s).reshape(-1)
    flat_order = order.reshape(b * s, p)
    seq_id, patch_id, cu, valid = packed_gather_index(flat_order, counts, capacity)
    image_id = seq_id // s
    tokens = patches[image_id, patch_id]
    token_coords = coords.expand(b, -1, -1)[image_id, patch_id]
    return tokens, token_coords, cu, seq_id, patch_id, valid


def unpack_to_padded(x: Tensor, cu_seqlens: Tensor, max_len: int, seq_id: Tensor, fill: float = 0.0):
    """Scatter packed rows ``[T, D]`` into a dense ``[N, max_len, D]`` tensor (what the dense decoder
    of ``model.py:143-165`` consumes) and the matching ``[N, max_len]`` validity mask."""
    n = cu_seqlens.numel() - 1
    pos = torch.arange(x.shape[0], device=x.device, dtype=torch.int64)
    within = pos - cu_seqlens[:-1].to(torch.int64)[seq_id]
    keep = (within >= 0) & (within < max_len) & (pos < cu_seqlens[-1].to(torch.int64))
    within = torch.clamp(within, 0, max_len - 1)
    dense = x.new_full((n, max_len, x.shape[1]), fill)
    mask = torch.zeros((n, max_len), dtype=torch.bool, device=x.device)
    dense[seq_id[keep], within[keep]] = x[keep]
    mask[seq_id[keep], within[keep]] = True
    return dense, mask


def segment_mean(x: Tensor, cu_seqlens: Tensor, seq_id: Tensor, valid: Optional[Tensor] = None) -> Tensor:
    """Mean over each sequence's rows of a packed ``[T, D]`` tensor -> ``[N, D]``: the global
    embedding of ``forward_embeddings`` (``tokens.mean(dim=0)``, ``model.py:273-276``) for a whole
    batch of ragged images in one call instead of one forward per image."""
    n = cu_seqlens.numel() - 1
    w = torch.ones(x.shape[0], device=x.device, dtype=x.dtype) if valid is None else valid.to(x.dtype)
    sums = torch.zeros((n, x.shape[1]), device=x.device, dtype=x.dtype).index_add_(0, seq_id, x * w[:, None])
    lengths = (cu_seqlens[1:] - cu_seqlens[:-1]).to(x.dtype).clamp(min=1)
    return sums / lengths[:, None]
