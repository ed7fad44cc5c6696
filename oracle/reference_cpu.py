"""The reference's own CPU implementation of the hot path, for timing and cross-checks.

TEST / BENCHMARK INFRASTRUCTURE ONLY (see ``attn_oracle.py``): imported by ``bench.py`` for the
``cpu_baseline`` leg and the ``--impl reference`` arm, and by tests.

The reference computes attention with ``F.scaled_dot_product_attention(q, k, v,
is_causal=self.causal)`` (``src/nanobrain/modules.py:62``, ``causal=False``) and differentiates
it with autograd (``src/nanobrain/misc.py:371``). On a machine without a usable GPU that call
runs torch's CPU kernel; this file makes exactly that call, per sequence for ragged batches as
the reference itself does (``src/nanobrain/model.py:254-270``).
"""

from __future__ import annotations

import time

import torch
import torch.nn.functional as F


def sdpa_fwd_bwd_cpu(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, d_out: torch.Tensor):
    """fp32 CPU forward + backward of the reference call for logical [B, H, L, 64] tensors."""
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    v = v.detach().clone().requires_grad_(True)
    out = F.scaled_dot_product_attention(q, k, v, is_causal=False)
    out.backward(d_out)
    return out.detach(), q.grad, k.grad, v.grad


def time_packed_sample(q, k, v, d_out, cu_seqlens, n_sequences: int, repeats: int = 1) -> tuple[float, int]:
    """Time the reference call over the first ``n_sequences`` sequences of a packed batch
    ([T, H, 64] fp32 CPU tensors), all heads. Returns (seconds for one pass, sum of L^2)."""
    slices = []
    for i in range(n_sequences):
        a, b = int(cu_seqlens[i]), int(cu_seqlens[i + 1])
        slices.append(tuple(t[a:b].transpose(0, 1)[None].contiguous() for t in (q, k, v, d_out)))
    sum_l2 = sum(s[0].shape[2] ** 2 for s in slices)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        for s in slices:
            sdpa_fwd_bwd_cpu(*s)
        best = min(best, time.perf_counter() - t0)
    return best, sum_l2
