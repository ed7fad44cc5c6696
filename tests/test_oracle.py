"""The CPU oracle against the golden fixtures made from the reference's own call, and against
torch's CPU SDPA (the reference's implementation of the path) live."""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from nanobrain_b200 import workloads as W
from oracle import attn_oracle as O


def test_oracle_matches_golden_sdpa(golden_dir):
    g = np.load(golden_dir / "sdpa_small.npz")
    out, lse, dq, dk, dv = O.sdpa_fwd_bwd(g["q"], g["k"], g["v"], g["d_out"])
    for name, got in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        np.testing.assert_allclose(got, g[name], rtol=0, atol=2e-6, err_msg=name)
    # lse is consistent with the scores it summarises
    s = np.einsum("bhqd,bhkd->bhqk", g["q"].astype(np.float64), g["k"].astype(np.float64)) / 8.0
    np.testing.assert_allclose(lse, np.log(np.exp(s).sum(-1)), atol=1e-9)


def test_oracle_matches_torch_cpu_sdpa_cpu_check_config():
    # the CPU-runnable parity case: fp32 dense B=2 H=12 L=820 D=64, seed 0, scale 1/8
    w = W.WORKLOADS["cpu_check"]
    q, k, v, g = W.make_dense_inputs(w.batch, w.heads, w.seqlen, seed=0)
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    out = F.scaled_dot_product_attention(q, k, v, is_causal=False)
    out.backward(g)
    got = O.sdpa_fwd_bwd(q.detach().numpy(), k.detach().numpy(), v.detach().numpy(), g.numpy(), dtype=np.float32)
    for name, a, b in (("out", got[0], out), ("dq", got[2], q.grad), ("dk", got[3], k.grad), ("dv", got[4], v.grad)):
        np.testing.assert_allclose(a, b.detach().numpy(), rtol=0, atol=5e-6, err_msg=name)


def test_varlen_oracle_equals_per_sequence_dense():
    lengths = torch.tensor([1, 7, 64, 129])
    cu = W.cu_seqlens_from_lengths(lengths).numpy()
    q, k, v, g = (t.numpy() for t in W.make_packed_inputs(lengths, heads=2, seed=3))
    out, lse, dq, dk, dv = O.varlen_fwd_bwd(q, k, v, g, cu, cu)
    for i in range(len(lengths)):
        a, b = cu[i], cu[i + 1]
        sl = lambda t: np.swapaxes(t[a:b], 0, 1)
        o_i, lse_i, dq_i, dk_i, dv_i = O.sdpa_fwd_bwd(sl(q), sl(k), sl(v), sl(g))
        np.testing.assert_allclose(np.swapaxes(out[a:b], 0, 1), o_i, atol=1e-12)
        np.testing.assert_allclose(lse[:, a:b], lse_i, atol=1e-12)
        np.testing.assert_allclose(np.swapaxes(dk[a:b], 0, 1), dk_i, atol=1e-12)
    # a length-1 sequence attends only to itself: out = v, dq = 0
    np.testing.assert_allclose(out[0], v[0], atol=1e-12)
    np.testing.assert_allclose(dq[0], 0, atol=1e-12)


def test_oracle_gradient_is_the_derivative():
    rng = np.random.default_rng(0)
    q, k, v, g = (rng.standard_normal((1, 1, 5, 64)) for _ in range(4))
    _, _, dq, dk, dv = O.sdpa_fwd_bwd(q, k, v, g)
    f = lambda q_, k_, v_: (O.sdpa_forward(q_, k_, v_)[0] * g).sum()
    eps = 1e-6
    for arr, grad in ((q, dq), (k, dk), (v, dv)):
        idx = (0, 0, 2, 17)
        pert = arr.copy()
        pert[idx] += eps
        args = [pert if a is arr else a for a in (q, k, v)]
        num = (f(*args) - f(q, k, v)) / eps
        assert abs(num - grad[idx]) < 1e-4


def test_workload_shapes_match_the_benchmark_definition():
    l1 = W.draw_lengths(W.WORKLOADS["vitb_encoder_varlen"])
    assert l1.numel() == 32 and int(l1.min()) >= 720 and int(l1.max()) <= 920
    assert torch.equal(l1, W.draw_lengths(W.WORKLOADS["vitb_encoder_varlen"]))  # deterministic
    flops = W.attention_flops(l1, l1, 12)
    assert flops == 14 * 12 * 64 * int((l1 * l1).sum())
    dense = W.draw_lengths(W.WORKLOADS["mae_decoder_dense"])
    assert W.attention_flops(dense, dense, 8) == 14 * 8 * 64 * 32 * 4096 * 4096
    cu = W.cu_seqlens_from_lengths(l1)
    assert cu.dtype == torch.int32 and cu[0] == 0 and cu[-1] == l1.sum()
    shards = [W.shard_lengths(W.draw_lengths(W.WORKLOADS["vitb_encoder_varlen_b256"]), r, 8) for r in range(8)]
    assert sum(s.numel() for s in shards) == 256
    with pytest.raises(ValueError):
        W.shard_lengths(l1, 0, 5)
