"""Host-side mirror of the attention-facing part of the reference's ``ViTMAE3D``
(``src/nanobrain/model.py:21-286``) with a packed-token (varlen) path.

The reference encodes a FIXED number of visible patches per sequence and evaluates images one at
a time because their in-mask patch counts differ (``model.py:186-199`` and ``254-270``). With the
varlen attention operator every sequence keeps its own length:

* ``forward_encoder`` / ``forward_decoder`` / ``forward``: same signatures and arithmetic as the
  reference's (``model.py:124-141``, ``143-165``, ``167-233``), on the dense operator. Parameter
  names are the reference's, so its checkpoints load with ``load_state_dict``.
* ``forward_encoder_packed``: patch-embed, position-embed, class tokens and the block loop over
  ``[T, dim]`` packed tokens addressed by ``cu_seqlens``; class tokens are inserted per sequence,
  which shifts sequence ``i`` by ``R * i`` rows (the packed form of the ``torch.cat`` at
  ``model.py:135-136``).
* ``forward_packed``: one MAE step in which sample ``i`` encodes its own ``counts[i]`` visible
  patches (packed encoder) and the decoder runs dense over ``R + S`` tokens per sample.
* ``embed_packed``: ``forward_embeddings`` for a list of ragged images in ONE packed encoder pass
  instead of one forward per image.

The data pipeline around the model (NIfTI loading, resampling, normalisation), checkpoint
registration and visualisation are not mirrored; the functions below take patches or volumes that
are already on the grid.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from . import token_prep as T
from .modules import Block, LayerNorm, SeparablePosEmbed3D


def patchify3d(x: Tensor, patch_size: int = 8) -> Tensor:
    """``[B, X, Y, Z]`` -> ``[B, gx*gy*gz, p^3]`` (``src/nanobrain/model.py:297-301``)."""
    b, sx, sy, sz = x.shape
    p = patch_size
    gx, gy, gz = sx // p, sy // p, sz // p
    x = x.reshape(b, gx, p, gy, p, gz, p).permute(0, 1, 3, 5, 2, 4, 6)
    return x.reshape(b, gx * gy * gz, p * p * p)


def make_coord_grid(grid_size: Sequence[int], patch_size: int = 8, device=None) -> Tensor:
    """Integer patch coordinates ``[1, P, 3]`` in patch-grid order (``model.py:334-344``)."""
    ids = [torch.arange(size // patch_size, device=device) for size in grid_size]
    return torch.stack(torch.meshgrid(*ids, indexing="ij"), dim=-1).reshape(1, -1, 3)


def sample_sequences(mask_patches: Tensor, num_samples: int, seq_length: Optional[int] = None,
                     min_mask_frac: float = 0.25) -> Tensor:
    """Mirror of ``sample_sequences`` (``model.py:347-363``): one shuffle per (image, sample) with
    out-of-mask patches last, cut to ``seq_length`` (default: the largest in-mask count, one sync).
    Draws from the global RNG exactly like the reference (one ``torch.rand(B, S, P)``)."""
    mask_frac = mask_patches.mean(dim=2)
    order = T.sample_order(mask_frac, num_samples, min_mask_frac)
    if seq_length is None:
        seq_length = int((mask_frac >= min_mask_frac).sum(dim=1).max().item())
    return order[:, :, :seq_length]


def _init_weights(m: nn.Module) -> None:
    # the reference's initialisation (model.py:366-376): xavier-uniform Linears, unit LayerNorms
    if isinstance(m, nn.Linear):
        nn.init.xavier_uniform_(m.weight)
        if m.bias is not None:
            nn.init.constant_(m.bias, 0)
    elif isinstance(m, nn.LayerNorm) and m.elementwise_affine:
        nn.init.constant_(m.weight, 1.0)
        if m.bias is not None:
            nn.init.constant_(m.bias, 0)


class ViTMAE3D(nn.Module):
    """3D ViT masked autoencoder with the reference's parameters and a packed-token path."""

    def __init__(
        self,
        grid_size: Tuple[int, int, int] = (192, 240, 192),
        patch_size: int = 8,
        depth: int = 12,
        embed_dim: int = 768,
        num_heads: int = 12,
        decoder_depth: int = 4,
        decoder_embed_dim: int = 512,
        decoder_num_heads: int = 8,
        qkv_bias: bool = True,
        proj_bias: bool = True,
        mlp_ratio: float = 4,
        class_tokens: int = 1,
        drop_path_rate: float = 0.0,
    ) -> None:
        super().__init__()
        self.grid_size = tuple(grid_size)
        self.patch_size = (patch_size, patch_size, patch_size)
        self.embed_dim = embed_dim
        self.class_tokens = class_tokens
        patch_grid = tuple(size // patch_size for size in grid_size)
        patch_dim = patch_size ** 3
        self.register_buffer("coord_grid", make_coord_grid(grid_size, patch_size), persistent=False)

        self.patch_embed = nn.Linear(patch_dim, embed_dim)
        self.pos_embed = SeparablePosEmbed3D(patch_grid, embed_dim)
        self.cls_token = nn.Parameter(torch.empty(1, class_tokens, embed_dim)) if class_tokens else None
        dpr = [x.item() for x in torch.linspace(0, drop_path_rate, depth)]
        self.blocks = nn.ModuleList([
            Block(dim=embed_dim, num_heads=num_heads, qkv_bias=qkv_bias, proj_bias=proj_bias, mlp_ratio=mlp_ratio,
                  drop_path=dpr[i])
            for i in range(depth)
        ])
        self.norm = LayerNorm(embed_dim)

        self.decoder_proj = nn.Linear(embed_dim, decoder_embed_dim)
        self.decoder_pos_embed = SeparablePosEmbed3D(patch_grid, decoder_embed_dim)
        self.mask_token = nn.Parameter(torch.empty(1, 1, decoder_embed_dim))
        self.decoder_blocks = nn.ModuleList([
            Block(dim=decoder_embed_dim, num_heads=decoder_num_heads, qkv_bias=qkv_bias, proj_bias=proj_bias,
                  mlp_ratio=mlp_ratio)
            for _ in range(decoder_depth)
        ])
        self.decoder_norm = LayerNorm(decoder_embed_dim)
        self.decoder_head = nn.Linear(decoder_embed_dim, patch_dim)
        self.init_weights()

    def init_weights(self) -> None:
        self.apply(_init_weights)
        if self.class_tokens:
            nn.init.normal_(self.cls_token, std=0.02)
        nn.init.normal_(self.mask_token, std=0.02)
        self.decoder_head.weight.data.mul_(0.0)

    # ------------------------------------------------------------------ dense (reference) path
    def forward_encoder(self, patches: Tensor, coord: Tensor) -> Tensor:
        """``[B, N, P]`` patches + ``[B, N, 3]`` coordinates -> ``[B, R+N, D]`` (``model.py:124-141``)."""
        b = patches.shape[0]
        x = self.pos_embed(self.patch_embed(patches), coord)
        if self.class_tokens:
            x = torch.cat([self.cls_token.expand(b, -1, -1), x], dim=1)
        for block in self.blocks:
            x = block(x)
        return self.norm(x)

    def forward_decoder(self, embeds: Tensor, target_coord: Tensor) -> Tensor:
        """``[B, R+N, D]`` encoder tokens + ``[B, M, 3]`` target coordinates -> ``[B, M, P]``
        predicted patches (``model.py:143-165``): dense attention over all ``R+N+M`` tokens."""
        b, m = embeds.shape[0], target_coord.shape[1]
        embeds = self.decoder_proj(embeds)
        mask_tokens = self.decoder_pos_embed(self.mask_token.expand(b, m, -1), target_coord)
        x = torch.cat([embeds, mask_tokens], dim=1)
        for block in self.decoder_blocks:
            x = block(x)
        return self.decoder_head(self.decoder_norm(x[:, -m:]))

    def forward(self, images: Tensor, mask: Tensor, num_visible: int, num_predict: Optional[int] = None,
                num_samples: int = 1, with_state: bool = True):
        """The reference's training forward (``model.py:167-233``): fixed ``num_visible`` per sequence."""
        b = images.shape[0]
        p = self.patch_size[0]
        patches, mask_patches = patchify3d(images, p), patchify3d(mask, p)
        coord = self.coord_grid.expand(b, -1, -1)
        seq_length = None if num_predict is None else num_visible + num_predict
        order = sample_sequences(mask_patches, num_samples, seq_length)
        num_predict = order.shape[2] - num_visible
        bid = torch.arange(b, device=images.device)[:, None, None]
        patches = patches[bid, order].flatten(0, 1)
        mask_patches = mask_patches[bid, order].flatten(0, 1)
        coord = coord[bid, order].flatten(0, 1)
        vis_patches, target_patches = torch.split(patches, [num_visible, num_predict], dim=1)
        vis_mask, target_mask = torch.split(mask_patches, [num_visible, num_predict], dim=1)
        vis_coord, target_coord = torch.split(coord, [num_visible, num_predict], dim=1)
        embeds = self.forward_encoder(vis_patches, vis_coord)
        pred = self.forward_decoder(embeds, target_coord)
        loss = F.mse_loss(pred, target_patches, reduction="none")
        loss = (target_mask * loss).sum() / target_mask.sum()
        if not with_state:
            return loss
        patch_ids = order.flatten(0, 1)
        vis_ids, target_ids = torch.split(patch_ids, [num_visible, num_predict], dim=1)
        return loss, {
            "vis_patches": vis_patches, "target_patches": target_patches, "vis_mask_patches": vis_mask,
            "target_mask_patches": target_mask, "embeds": embeds, "pred_patches": pred, "vis_ids": vis_ids,
            "target_ids": target_ids,
            "image_ids": torch.arange(b, device=images.device).repeat_interleave(num_samples),
        }

    # ------------------------------------------------------------------ packed path
    def forward_encoder_packed(self, tokens: Tensor, coord: Tensor, cu_seqlens: Tensor, max_seqlen: int,
                               seq_id: Optional[Tensor] = None):
        """Encoder over packed tokens.

        ``tokens``: ``[T, P]`` patches of all sequences back to back, ``coord``: ``[T, 3]``,
        ``cu_seqlens``: int32 ``[N+1]`` (rows past ``cu_seqlens[-1]`` are padding and stay padding),
        ``max_seqlen``: host upper bound of the sequence lengths, ``seq_id``: int64 ``[T]`` owner of
        each row (computed if omitted).

        Returns ``(x [T + R*N, D], cu_seqlens', max_seqlen + R, seq_id', is_cls [T + R*N])`` where
        sequence ``i`` now owns rows ``[cu[i] + R*i, cu[i+1] + R*(i+1))`` and starts with its ``R``
        class tokens, like the dense ``torch.cat([cls, x], dim=1)`` of ``model.py:135-136``."""
        t = tokens.shape[0]
        n = cu_seqlens.numel() - 1
        r = self.class_tokens
        if seq_id is None:
            pos = torch.arange(t, device=tokens.device)
            seq_id = torch.clamp(torch.searchsorted(cu_seqlens[1:].to(torch.int64), pos, right=True), max=n - 1)
        x = self.pos_embed(self.patch_embed(tokens), coord)
        is_cls = torch.zeros(t + r * n, dtype=torch.bool, device=tokens.device)
        if r:
            # Row t of sequence i moves to t + R*(i+1); the R rows before a sequence's first token
            # hold its class tokens. Padding rows (past the last sequence) move behind everything.
            starts = cu_seqlens[:-1].to(torch.int64) + r * torch.arange(n, device=tokens.device)
            cls_rows = (starts[:, None] + torch.arange(r, device=tokens.device)[None, :]).reshape(-1)
            is_cls[cls_rows] = True
            pos = torch.arange(t, device=tokens.device)
            pad = pos >= cu_seqlens[-1].to(torch.int64)
            dest = pos + r * (seq_id + 1)
            dest = torch.where(pad, pos + r * n, dest)
            full = x.new_empty((t + r * n, x.shape[1]))
            full[dest] = x
            full[cls_rows] = self.cls_token[0].to(x.dtype).repeat(n, 1)
            x = full
            new_seq = torch.empty(t + r * n, dtype=torch.int64, device=tokens.device)
            new_seq[dest] = seq_id
            new_seq[cls_rows] = torch.arange(n, device=tokens.device).repeat_interleave(r)
            seq_id = new_seq
            cu_seqlens = (cu_seqlens.to(torch.int64) + r * torch.arange(n + 1, device=tokens.device)).to(torch.int32)
            max_seqlen = max_seqlen + r
        for block in self.blocks:
            x = block(x, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen, seq_id=seq_id)
        return self.norm(x), cu_seqlens, max_seqlen, seq_id, is_cls

    def forward_packed(self, images: Tensor, mask: Tensor, counts: Tensor, max_visible: int,
                       seq_length: int, num_samples: int = 1, order: Optional[Tensor] = None):
        """One MAE step in which every sequence encodes its own number of visible patches.

        ``counts``: int64 ``[B]`` or ``[B, S]`` visible patches per sequence (e.g. from
        :func:`nanobrain_b200.token_prep.visible_counts`), ``max_visible``: a host upper bound of
        them (sizes the packed buffer: nothing synchronises), ``seq_length``: patches per sequence
        that take part (visible + predicted), ``order``: optional precomputed ``[B, S, seq_length]``
        patch order (default: :func:`sample_sequences`).

        The encoder runs packed over ``sum(counts)`` tokens; the decoder runs dense over ``R +
        seq_length`` tokens per sequence -- the encoder's tokens of the sequence first, mask tokens
        with the position embedding of the remaining patches after them -- and the loss is the
        reference's mask-weighted MSE (``model.py:201-203``) over each sequence's own targets.
        Returns ``(loss, state)``."""
        b = images.shape[0]
        p = self.patch_size[0]
        r = self.class_tokens
        patches, mask_patches = patchify3d(images, p), patchify3d(mask, p)
        if order is None:
            order = sample_sequences(mask_patches, num_samples, seq_length)
        s = order.shape[1]
        n = b * s
        counts = counts.reshape(b, -1).expand(b, s).reshape(-1).to(torch.int64)
        coord = self.coord_grid.expand(b, -1, -1)

        # visible tokens, packed (replaces the fixed-length gather + split of model.py:186-199)
        tokens, tok_coord, cu, seq_id, _, valid = T.pack_visible_tokens(patches, coord, order, counts.reshape(b, s),
                                                                        capacity=n * max_visible)
        x, cu_r, _, seq_r, _ = self.forward_encoder_packed(tokens, tok_coord, cu, max_visible, seq_id=seq_id)

        # dense decoder input [N, R + seq_length, D']: encoder rows of the sequence, then mask tokens
        x = self.decoder_proj(x)
        dense_enc, from_enc = T.unpack_to_padded(x, cu_r, r + seq_length, seq_r)
        bid = torch.arange(b, device=images.device)[:, None, None]
        seq_coord = coord[bid, order].flatten(0, 1)                       # [N, seq_length, 3]
        mask_tokens = self.decoder_pos_embed(self.mask_token.expand(n, seq_length, -1), seq_coord)
        mask_tokens = torch.cat([mask_tokens.new_zeros(n, r, mask_tokens.shape[2]), mask_tokens], dim=1)
        y = torch.where(from_enc[:, :, None], dense_enc.to(mask_tokens.dtype), mask_tokens)
        for block in self.decoder_blocks:
            y = block(y)
        pred = self.decoder_head(self.decoder_norm(y[:, r:]))            # [N, seq_length, P]

        target = patches[bid, order].flatten(0, 1)
        target_mask = mask_patches[bid, order].flatten(0, 1)
        is_target = torch.arange(seq_length, device=images.device)[None, :] >= counts[:, None]
        weight = target_mask * is_target[:, :, None]
        loss = (weight * F.mse_loss(pred, target, reduction="none")).sum() / weight.sum()
        return loss, {"pred_patches": pred, "order": order, "counts": counts, "cu_seqlens": cu_r,
                      "tokens_valid": valid, "is_target": is_target}

    @torch.inference_mode()
    def embed_packed(self, samples: Sequence[Tuple[Tensor, Tensor]], return_dense: bool = False) -> List[dict]:
        """Global (and optionally dense) embeddings of a list of images in ONE packed encoder pass.

        ``samples``: per image ``(patches [P, patch_dim], in_mask [P] bool)``, i.e. what the
        reference's ``forward_embeddings`` has after ``patchify3d`` (``model.py:262-263``). The
        reference runs one encoder forward per image because the in-mask counts differ
        (``model.py:254-270``); here all images' in-mask patches are packed and every block makes a
        single varlen attention call. Outputs follow ``model.py:271-285``: the mean of the patch
        tokens (class tokens dropped) and, on request, the tokens scattered back on the patch grid."""
        device = self.coord_grid.device
        lengths = [int(m.sum()) for _, m in samples]
        if min(lengths) <= 0:
            raise ValueError("every image needs at least one in-mask patch")
        tokens = torch.cat([pt.to(device)[m.to(device)] for pt, m in samples])
        coord = torch.cat([self.coord_grid[0][m.to(device)] for _, m in samples])
        cu = T.cu_seqlens_from_counts(torch.tensor(lengths, device=device))
        with torch.autocast(device.type, dtype=torch.bfloat16, enabled=device.type == "cuda"):
            x, cu_r, _, seq_r, is_cls = self.forward_encoder_packed(tokens, coord, cu, max(lengths))
        x = x.float()
        keep = ~is_cls
        means = T.segment_mean(x[keep], cu, seq_r[keep])
        outputs = []
        grid = [size // self.patch_size[0] for size in self.grid_size]
        starts = [0]
        for length in lengths:
            starts.append(starts[-1] + length)
        patch_tokens = x[keep]
        for i, (_, m) in enumerate(samples):
            out = {"global_embedding": means[i], "dense_embedding": None, "dense_mask": None}
            if return_dense:
                m = m.to(device)
                dense = patch_tokens.new_zeros(m.numel(), self.embed_dim)
                dense[m] = patch_tokens[starts[i]:starts[i + 1]]
                out["dense_embedding"] = dense.reshape(*grid, self.embed_dim)
                out["dense_mask"] = m.reshape(grid)
            outputs.append(out)
        return outputs
