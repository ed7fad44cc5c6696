"""Host-side mirror of the reference's ``Attention`` and ``Block`` with the SDPA call swapped for
the B200 operator.

``Attention`` keeps the reference's constructor arguments, parameter names (``q``, ``k``, ``v``,
``proj``: checkpoints load unchanged, cf. ``src/nanobrain/misc.py:343``) and dense behaviour
(``src/nanobrain/modules.py:21-65``). It adds a packed path: given ``[T, dim]`` tokens of several
sequences and their ``cu_seqlens`` it views the Linear outputs as ``[T, H, 64]`` -- already the
varlen layout, no copy -- and calls the varlen operator.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
from torch import Tensor

from .ops import sdpa, sdpa_varlen


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
    """Pre-norm residual block, drop-in for ``nanobrain.modules.Block`` (``modules.py:92-131``,
    stochastic depth 0 as in ``default_pretrain.yaml:36``). ``cu_seqlens`` / ``max_seqlen`` are
    passed through to the attention, so the same block serves dense ``[B, N, dim]`` and packed
    ``[T, dim]`` tokens (LayerNorm and the MLP are token-wise)."""

    def __init__(self, dim: int, num_heads: int, qkv_bias: bool = False, proj_bias: bool = False,
                 context_dim: Optional[int] = None, mlp_ratio: float = 4) -> None:
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=1e-6)
        self.attn = Attention(dim, num_heads, qkv_bias=qkv_bias, proj_bias=proj_bias, context_dim=context_dim)
        self.drop_path1 = nn.Identity()
        self.norm2 = nn.LayerNorm(dim, eps=1e-6)
        self.mlp = Mlp(dim, mlp_ratio=mlp_ratio, bias=proj_bias)
        self.drop_path2 = nn.Identity()

    def forward(self, x: Tensor, context: Optional[Tensor] = None, cu_seqlens: Optional[Tensor] = None,
                max_seqlen: Optional[int] = None) -> Tensor:
        x = x + self.attn(self.norm1(x), context=context, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)
        return x + self.mlp(self.norm2(x))
