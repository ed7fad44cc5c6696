"""CPU oracle for bidirectional scaled-dot-product attention, forward and backward.

TEST INFRASTRUCTURE ONLY. Nothing in the ``nanobrain_b200`` package imports this file; it is
used by ``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` leg of
``bench.py`` as the checker for the CUDA kernels, never as the thing being shipped.

What it restates: the arithmetic of the one call on the reference's hot path,
``F.scaled_dot_product_attention(q, k, v, is_causal=self.causal)`` with ``causal=False``
(``src/nanobrain/modules.py:62``), and of the backward autograd derives for it when
``loss.backward()`` runs (``src/nanobrain/misc.py:368-371``). The arithmetic itself lives in a
third-party dependency of the reference, PyTorch (pinned ``torch==2.14.0`` in the reference's
``pyproject.toml:23``; this container has torch 2.11.0), so the restatement below follows the
published definition ``softmax(Q K^T * scale) V`` with ``scale = 1/sqrt(head_dim)``
(``modules.py:33`` gives head_dim = dim // num_heads = 64) and its analytic gradient.

Pinning: the reference ships no tests or golden vectors for this path. The oracle is pinned
instead against outputs of the reference's own call run in the build container:
``tests/golden/make_golden.py`` calls torch's CPU SDPA (and the reference's unmodified
``Attention`` module imported from its source tree) in fp32 and stores inputs and outputs under
``tests/golden/``; ``tests/test_oracle.py`` checks this file against those fixtures and
against torch's CPU SDPA live.

All functions take and return numpy arrays. ``dtype`` selects the working precision
(``float64`` for the small pinned cases, ``float32`` for speed on large ones).
"""

from __future__ import annotations

import math

import numpy as np


def default_scale(head_dim: int) -> float:
    """``F.scaled_dot_product_attention``'s default: 1/sqrt(head_dim) (modules.py:62 passes none)."""
    return 1.0 / math.sqrt(head_dim)


def sdpa_forward(q, k, v, scale=None, dtype=np.float64):
    """Forward of the call at ``src/nanobrain/modules.py:62`` for one or more (batch, head) slices.

    q: [..., Lq, D], k, v: [..., Lk, D]. Returns (out [..., Lq, D], lse [..., Lq]) where ``lse`` is
    the natural-log row log-sum-exp of the scaled scores (what a fused kernel saves for backward).
    """
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    scale = default_scale(q.shape[-1]) if scale is None else scale
    s = np.matmul(q, np.swapaxes(k, -1, -2)) * dtype(scale)
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(axis=-1, keepdims=True)
    out = np.matmul(e / l, v)
    lse = (m + np.log(l))[..., 0]
    return out, lse


def sdpa_backward(q, k, v, d_out, scale=None, dtype=np.float64):
    """Gradient of ``sdpa_forward`` w.r.t. q, k, v for upstream gradient ``d_out``.

    This is what autograd computes for the call at ``src/nanobrain/modules.py:62`` when
    ``loss.backward()`` runs (``src/nanobrain/misc.py:371``):
        P = softmax(S),  dV = P^T dO,  dP = dO V^T,
        dS = P o (dP - rowsum(dO o O)),  dQ = scale dS K,  dK = scale dS^T Q.
    """
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    d_out = np.asarray(d_out, dtype=dtype)
    scale = default_scale(q.shape[-1]) if scale is None else scale
    s = np.matmul(q, np.swapaxes(k, -1, -2)) * dtype(scale)
    s -= s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=-1, keepdims=True)
    out = np.matmul(p, v)
    dv = np.matmul(np.swapaxes(p, -1, -2), d_out)
    dp = np.matmul(d_out, np.swapaxes(v, -1, -2))
    delta = (d_out * out).sum(axis=-1, keepdims=True)
    ds = p * (dp - delta)
    dq = np.matmul(ds, k) * dtype(scale)
    dk = np.matmul(np.swapaxes(ds, -1, -2), q) * dtype(scale)
    return dq, dk, dv


def sdpa_fwd_bwd(q, k, v, d_out, scale=None, dtype=np.float64):
    """Convenience: (out, lse, dq, dk, dv) for logical [B, H, L, D] (or any leading dims)."""
    out, lse = sdpa_forward(q, k, v, scale, dtype)
    dq, dk, dv = sdpa_backward(q, k, v, d_out, scale, dtype)
    return out, lse, dq, dk, dv


def varlen_fwd_bwd(q, k, v, d_out, cu_seqlens_q, cu_seqlens_k, scale=None, dtype=np.float64):
    """Packed form: q, d_out [Tq, H, D], k, v [Tk, H, D]; sequence i owns rows
    [cu_seqlens[i], cu_seqlens[i+1]). Each sequence is an independent dense problem, which is how
    the reference treats ragged lengths (one forward per image, ``src/nanobrain/model.py:254-270``).

    Returns (out [Tq,H,D], lse [H,Tq], dq, dk, dv)."""
    q = np.asarray(q)
    k = np.asarray(k)
    tq, h, d = q.shape
    out = np.zeros((tq, h, d), dtype=dtype)
    lse = np.zeros((h, tq), dtype=dtype)
    dq = np.zeros((tq, h, d), dtype=dtype)
    dk = np.zeros(k.shape, dtype=dtype)
    dv = np.zeros(k.shape, dtype=dtype)
    for i in range(len(cu_seqlens_q) - 1):
        q0, q1 = int(cu_seqlens_q[i]), int(cu_seqlens_q[i + 1])
        k0, k1 = int(cu_seqlens_k[i]), int(cu_seqlens_k[i + 1])
        if q1 == q0 or k1 == k0:
            continue
        qs = np.swapaxes(q[q0:q1], 0, 1)
        ks = np.swapaxes(k[k0:k1], 0, 1)
        vs = np.swapaxes(np.asarray(v)[k0:k1], 0, 1)
        gs = np.swapaxes(np.asarray(d_out)[q0:q1], 0, 1)
        o, l, a, b, c = sdpa_fwd_bwd(qs, ks, vs, gs, scale, dtype)
        out[q0:q1] = np.swapaxes(o, 0, 1)
        lse[:, q0:q1] = l
        dq[q0:q1] = np.swapaxes(a, 0, 1)
        dk[k0:k1] = np.swapaxes(b, 0, 1)
        dv[k0:k1] = np.swapaxes(c, 0, 1)
    return out, lse, dq, dk, dv
