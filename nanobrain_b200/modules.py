"""Host-side mirror of the reference's ``Attention``, ``Mlp``, ``Block`` and
``SeparablePosEmbed3D`` with the SDPA call swapped for the B200 operator.

``Attention`` keeps the reference's constructor arguments, parameter names (``q``, ``k``, ``v``,
``proj``: checkpoints load unchanged, cf. ``src/nanobrain/misc.py:343``) and dense behaviour
(``src/nanobrain/modules.py:21-65``). It adds a packed path: given ``[T, dim]`` tokens of several
sequences and their ``cu_seqlens`` it views the Linear outputs as ``[T, H, 64]`` -- already the
varlen layout, no copy -- and calls the varlen operator.
"""

from __future__ import annotations

from functools import partial
from typing import Callable, Optional, Tuple

import torch
import torch.nn as nn
from torch import Tensor

from .ops import sdpa, sdpa_varlen

# The reference's norm layer: LayerNorm with timm's eps (``src/nanobrain/modules.py:88-89``).
LayerNorm = partial(nn.LayerNorm, eps=1e-6)


class DropPath(nn.Module):
    """Stochastic depth per sample, as ``timm.layers.DropPath`` which the reference uses at
    ``src/nanobrain/modules.py:112,120``: in training each sample's residual branch is dropped with
    probability ``drop_prob`` and the kept ones are scaled by ``1 / (1 - drop_prob)``.

    For packed ``[T, dim]`` tokens a "sample" is a sequence: pass ``seq_id`` (int64 ``[T]``, the
    sequence owning each row) and ``num_seqs`` so that all rows of one sequence share one draw."""

    def __init__(self, drop_prob: float = 0.0, scale_by_keep: bool = True) -> None:
        super().__init__()
        self.drop_prob = float(drop_prob)
        self.scale_by_keep = scale_by_keep

    def extra_repr(self) -> str:
        return f"drop_prob={self.drop_prob:0.3f}"

    def forward(self, x: Tensor, seq_id: Optional[Tensor] = None, num_seqs: Optional[int] = None) -> Tensor:
        if self.drop_prob == 0.0 or not self.training:
            return x
        keep = 1.0 - self.drop_prob
        if seq_id is None:
            mask = x.new_empty((x.shape[0],) + (1,) * (x.dim() - 1)).bernoulli_(keep)
        else:
            mask = x.new_empty(int(num_seqs)).bernoulli_(keep)[seq_id][:, None]
        if keep > 0.0 and self.scale_by_keep:
            mask = mask / keep
        return x * mask


class Attention(nn.Module):
    """Multi-head bidirectional attention; drop-in for ``nanobrain.modules.Attention``."""

    def __init__(
        self,
        dim: int,
        num_heads: int,
        qkv_bias: bool = False,
        proj_bias: bool = False,
        context_dim: Optional[int] = None,
        causal: bool = False,
    ) -> None:
        super().__init__()
        if causal:
            raise ValueError("the B200 attention operator is bidirectional only (the reference never sets causal)")
        if dim % num_heads != 0 or dim // num_heads != 64:
            raise ValueError(f"head_dim must be 64, got dim={dim}, num_heads={num_heads}")
        self.num_heads = num_heads
        self.head_dim = dim // num_heads
        self.causal = False
        kv_in = dim if context_dim is None else context_dim
        self.q = nn.Linear(dim, dim, bias=qkv_bias)
        self.k = nn.Linear(kv_in, dim, bias=qkv_bias)
        self.v = nn.Linear(kv_in, dim, bias=qkv_bias)
        self.proj = nn.Linear(dim, dim, bias=proj_bias)

    def extra_repr(self) -> str:
        return f"num_heads={self.num_heads}, causal={self.causal}"

    def forward(
        self,
        x: Tensor,
        context: Optional[Tensor] = None,
        cu_seqlens: Optional[Tensor] = None,
        max_seqlen: Optional[int] = None,
        cu_seqlens_k: Optional[Tensor] = None,
        max_seqlen_k: Optional[int] = None,
    ) -> Tensor:
        src = x if context is None else context
        heads, hd = self.num_heads, self.head_dim
        if cu_seqlens is None:
            # Dense: x [B, N, dim]; views of the Linear outputs, logical [B, H, N, 64].
            bsz, n, dim = x.shape
            m = src.shape[1]
            q = self.q(x).view(bsz, n, heads, hd).transpose(1, 2)
            k = self.k(src).view(bsz, m, heads, hd).transpose(1, 2)
            v = self.v(src).view(bsz, m, heads, hd).transpose(1, 2)
            y = sdpa(q, k, v, is_causal=False)
            y = y.transpose(1, 2).reshape(bsz, n, dim)
        else:
            # Packed: x [T, dim]; sequence i owns rows [cu_seqlens[i], cu_seqlens[i+1]).
            if max_seqlen is None:
                raise ValueError("max_seqlen is required with cu_seqlens (a host integer; avoids a device sync)")
            t, dim = x.shape
            cu_k = cu_seqlens if cu_seqlens_k is None else cu_seqlens_k
            max_k = max_seqlen if max_seqlen_k is None else max_seqlen_k
            q = self.q(x).view(t, heads, hd)
            k = self.k(src).view(src.shape[0], heads, hd)
            v = self.v(src).view(src.shape[0], heads, hd)
            y = sdpa_varlen(q, k, v, cu_seqlens, cu_k, max_seqlen, max_k).reshape(t, dim)
        return self.proj(y)


class Mlp(nn.Module):
    """Token-wise MLP; same parameters as ``nanobrain.modules.Mlp`` (``modules.py:68-85``)."""

    def __init__(self, dim: int, mlp_ratio: float = 4, bias: bool = False) -> None:
        super().__init__()
        hidden = int(dim * mlp_ratio)
        self.fc1 = nn.Linear(dim, hidden, bias=bias)
        self.act = nn.GELU()
        self.fc2 = nn.Linear(hidden, dim, bias=bias)

    def forward(self, x: Tensor) -> Tensor:
        return self.fc2(self.act(self.fc1(x)))


class Block(nn.Module):
    """Pre-norm residual block, drop-in for ``nanobrain.modules.Block``
    (``src/nanobrain/modules.py:92-131``): same constructor arguments -- the reference builds its
    encoder with ``Block(..., drop_path=dpr[ii])`` at ``src/nanobrain/model.py:68-75`` -- and the
    same parameter names. ``cu_seqlens`` / ``max_seqlen`` are passed through to the attention, so
    one block serves dense ``[B, N, dim]`` and packed ``[T, dim]`` tokens (LayerNorm and the MLP
    are token-wise); with stochastic depth on packed tokens also pass ``seq_id``."""

    def __init__(self, dim: int, num_heads: int, qkv_bias: bool = False, proj_bias: bool = False,
                 context_dim: Optional[int] = None, mlp_ratio: float = 4, drop_path: float = 0.0,
                 norm_layer: Callable[[int], nn.Module] = LayerNorm) -> None:
        super().__init__()
        self.norm1 = norm_layer(dim)
        self.attn = Attention(dim, num_heads, qkv_bias=qkv_bias, proj_bias=proj_bias, context_dim=context_dim)
        self.drop_path1 = DropPath(drop_path) if drop_path > 0 else nn.Identity()
        self.norm2 = norm_layer(dim)
        self.mlp = Mlp(dim, mlp_ratio=mlp_ratio, bias=proj_bias)
        self.drop_path2 = DropPath(drop_path) if drop_path > 0 else nn.Identity()

    def _drop(self, layer: nn.Module, y: Tensor, seq_id: Optional[Tensor], num_seqs: Optional[int]) -> Tensor:
        if isinstance(layer, DropPath) and seq_id is not None:
            return layer(y, seq_id=seq_id, num_seqs=num_seqs)
        return layer(y)

    def forward(self, x: Tensor, context: Optional[Tensor] = None, cu_seqlens: Optional[Tensor] = None,
                max_seqlen: Optional[int] = None, seq_id: Optional[Tensor] = None) -> Tensor:
        num_seqs = None if cu_seqlens is None else cu_seqlens.numel() - 1
        y = self.attn(self.norm1(x), context=context, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
        x = x + self._drop(self.drop_path1, y, seq_id, num_seqs)
        return x + self._drop(self.drop_path2, self.mlp(self.norm2(x)), seq_id, num_seqs)


class SeparablePosEmbed3D(nn.Module):
    """Sum of three learned per-axis tables indexed by a token's grid coordinate; same parameters
    (``weight_x``, ``weight_y``, ``weight_z``) and initialisation as the reference's module at
    ``src/nanobrain/modules.py:137-173``. It is token-wise, so it takes dense ``[B, N, D]`` tokens
    with ``[B, N, 3]`` coordinates and packed ``[T, D]`` tokens with ``[T, 3]`` coordinates alike."""

    def __init__(self, grid_size: Tuple[int, int, int], embed_dim: int, unit: float = 1.0) -> None:
        super().__init__()
        self.embed_dim = embed_dim
        self.grid_size = tuple(grid_size)
        self.unit = unit
        gx, gy, gz = self.grid_size
        self.weight_x = nn.Parameter(torch.empty(gx, embed_dim))
        self.weight_y = nn.Parameter(torch.empty(gy, embed_dim))
        self.weight_z = nn.Parameter(torch.empty(gz, embed_dim))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for w in (self.weight_x, self.weight_y, self.weight_z):
            nn.init.trunc_normal_(w, std=0.02)

    def forward(self, x: Tensor, coord: Tensor) -> Tensor:
        pos = torch.floor(coord / self.unit).to(torch.int64)
        return x + self.weight_x[pos[..., 0]] + self.weight_y[pos[..., 1]] + self.weight_z[pos[..., 2]]

    def extra_repr(self) -> str:
        return f"{self.embed_dim}, {self.grid_size}, unit={self.unit}"
