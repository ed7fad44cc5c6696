"""Seeded synthetic workloads with the shapes of the reference model's attention calls.

The reference publishes no attention benchmark or dataset for this path, so the inputs are
synthetic: values iid N(0, 1) from ``torch.Generator().manual_seed(seed)`` on the CPU in fp32,
drawn in the order Q, K, V, dO; per-sample visible-token counts from a separate generator with
the same seed. Shapes follow the reference's ViT-B MAE (12 heads of 64 in the encoder, 8 heads
of 64 in the decoder, ``src/nanobrain/config/default_pretrain.yaml:28-34``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

HEAD_DIM = 64


@dataclass(frozen=True)
class Workload:
    name: str
    batch: int
    heads: int
    seqlen: Optional[int] = None       # dense length, or None for varlen
    len_lo: Optional[int] = None       # varlen: inclusive bounds of the per-sample length
    len_hi: Optional[int] = None
    description: str = ""

    @property
    def varlen(self) -> bool:
        return self.seqlen is None


WORKLOADS = {
    "cpu_check": Workload("cpu_check", 2, 12, seqlen=820,
                          description="fp32 dense B=2 H=12 L=820 D=64 (CPU-runnable parity case)"),
    "vitb_encoder_varlen": Workload("vitb_encoder_varlen", 32, 12, len_lo=720, len_hi=920,
                                    description="ViT-B MAE encoder, 16^3 grid, ~80% masked, B=32 packed"),
    "mae_decoder_dense": Workload("mae_decoder_dense", 32, 8, seqlen=4096,
                                  description="MAE decoder over the full 4096-token grid, B=32, H=8"),
    "vitl_encoder_varlen": Workload("vitl_encoder_varlen", 16, 16, len_lo=1700, len_hi=2140,
                                    description="20x24x20 grid, ~80% masked, B=16, H=16"),
    "vitb_encoder_varlen_b256": Workload("vitb_encoder_varlen_b256", 256, 12, len_lo=720, len_hi=920,
                                         description="scaling sweep: global B=256 sharded B/N per GPU"),
}


def draw_lengths(w: Workload, seed: int = 0) -> torch.Tensor:
    """Per-sample token counts (int64, CPU) for a workload."""
    if not w.varlen:
        return torch.full((w.batch,), w.seqlen, dtype=torch.int64)
    g = torch.Generator().manual_seed(seed)
    return torch.randint(w.len_lo, w.len_hi + 1, (w.batch,), generator=g)


def cu_seqlens_from_lengths(lengths: torch.Tensor) -> torch.Tensor:
    """int32 [B+1] prefix sums, the varlen addressing the packed entry point takes."""
    cu = torch.zeros(lengths.numel() + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lengths, 0).to(torch.int32)
    return cu


def shard_lengths(lengths: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Contiguous B/N slice of the global batch for one rank (no data-path collective)."""
    b = lengths.numel()
    if b % world != 0:
        raise ValueError(f"batch {b} is not divisible by world size {world}")
    per = b // world
    return lengths[rank * per:(rank + 1) * per]


def attention_flops(lengths_q: torch.Tensor, lengths_k: torch.Tensor, heads: int, fwd: bool = True,
                    bwd: bool = True) -> int:
    """Algorithmic FLOPs: 4*H*D*sum(Lq*Lk) forward (2 GEMMs), 10*H*D*sum(Lq*Lk) backward (5 GEMMs).

    These equal torch's ``sdpa_flop_count`` / ``sdpa_backward_flop_count`` that the reference's
    own TFLOP/s meter uses through ``FlopCounterMode`` (``src/nanobrain/train.py:414-432``).
    Padding to tile multiples is not counted."""
    pairs = int((lengths_q.to(torch.int64) * lengths_k.to(torch.int64)).sum())
    return (4 * fwd + 10 * bwd) * heads * HEAD_DIM * pairs


def attention_bytes(total_tokens: int, heads: int) -> int:
    """Algorithmic HBM bytes of fwd+bwd: 12 bf16 tensor passes plus three fp32 LSE passes."""
    return 12 * total_tokens * heads * HEAD_DIM * 2 + 3 * total_tokens * heads * 4


def make_packed_inputs(lengths: torch.Tensor, heads: int, seed: int = 0, dtype=torch.float32):
    """Q, K, V, dO as packed [T, H, 64] CPU tensors (values independent of the lengths' generator)."""
    total = int(lengths.sum())
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn(total, heads, HEAD_DIM, generator=g, dtype=torch.float32).to(dtype) for _ in range(4))


def make_dense_inputs(batch: int, heads: int, seqlen: int, seed: int = 0, dtype=torch.float32):
    """Q, K, V, dO as logical [B, H, L, 64] CPU tensors, contiguous."""
    g = torch.Generator().manual_seed(seed)
    return tuple(
        torch.randn(batch, heads, seqlen, HEAD_DIM, generator=g, dtype=torch.float32).to(dtype) for _ in range(4)
    )
