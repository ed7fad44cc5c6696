"""The varlen tile scheduler on the GPU: the device-built work list against the host version of
the same rule, parity of the attention kernels on skewed length mixes (where the list order
matters most), and the device-side validation of cu_seqlens."""

import numpy as np
import pytest
import torch

import nanobrain_b200
from nanobrain_b200 import _lib, ops, schedule
from nanobrain_b200 import workloads as W
from oracle import attn_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def lists(lengths_q, lengths_k, side, total_q=None, total_k=None, max_q=None, max_k=None):
    lq, lk = torch.tensor(lengths_q), torch.tensor(lengths_k)
    cu_q, cu_k = W.cu_seqlens_from_lengths(lq), W.cu_seqlens_from_lengths(lk)
    args = (max_q or int(lq.max()), max_k or int(lk.max()), total_q or int(lq.sum()), total_k or int(lk.sum()))
    host = schedule.work_list_host(cu_q, cu_k, *args, side)
    dev, status = schedule.work_list_device(cu_q.to(DEV), cu_k.to(DEV), *args, 12, side)
    torch.cuda.synchronize()
    return host, dev.cpu(), int(status[0])


@pytest.mark.parametrize("lengths", [
    [820], [1], [127, 129, 256, 1, 0, 700], [200] * 30 + [2000],
    W.draw_lengths(W.WORKLOADS["vitb_encoder_varlen"]).tolist(),
    torch.randint(0, 3000, (1500,), generator=torch.Generator().manual_seed(1)).tolist(),
])
def test_device_list_equals_host_list_up_to_order_inside_a_cost_class(lengths):
    for side in (0, 1):
        host, dev, status = lists(lengths, lengths, side)
        assert status == 0 and host.shape == dev.shape
        h, d = schedule.decode(host), schedule.decode(dev)
        assert sorted(h) == sorted(d)                                  # the same items, each once
        n_used = len(h)
        assert bool((dev[n_used:, 0] < 0).all())                       # unused entries at the end
        assert sorted(map(tuple, host[:n_used].tolist())) == sorted(map(tuple, dev[:n_used].tolist()))
        # same cost (steps) and same kind (full before ragged) at every position
        steps = [(l + 127) // 128 for l in lengths] + [0]
        lens = list(lengths) + [0]
        kind = lambda it: (steps[it[0]], it[1] == lens[it[0]] // 128 and lens[it[0]] % 128 != 0)
        assert [kind(x) for x in h] == [kind(x) for x in d]


def test_device_list_with_cross_lengths_and_spare_rows():
    host, dev, status = lists([130, 5, 64], [3, 900, 129], 1, total_q=400, total_k=2000)
    assert status == 0 and sorted(schedule.decode(host)) == sorted(schedule.decode(dev))
    assert (3, 0) in schedule.decode(dev)                               # the rows past the last sequence


@pytest.mark.parametrize("case", ["too_long", "beyond_total", "decreasing"])
def test_invalid_cu_seqlens_are_reported_and_nothing_runs(case):
    lengths = torch.tensor([100, 200])
    cu = W.cu_seqlens_from_lengths(lengths)
    max_len, total = 200, 300
    if case == "too_long":
        max_len = 150          # max_seqlen must be a true upper bound: no tile is silently dropped
    elif case == "beyond_total":
        total = 299
    else:
        cu = torch.tensor([0, 200, 100], dtype=torch.int32)
    _, status = schedule.work_list_device(cu.to(DEV), cu.to(DEV), max_len, max_len, total, total, 2, 0)
    torch.cuda.synchronize()
    assert int(status[0]) == _lib.STATUS_BAD_SEQLENS
    # through the op: the kernels leave the outputs alone and the next call (or check_status) raises
    t = torch.randn(300, 2, 64, device=DEV).to(torch.bfloat16)
    cud = cu.to(DEV)
    out, _ = ops.sdpa_varlen_fwd(t[:total], t[:total], t[:total], cud, cud, max_len, max_len, 0.125)
    with pytest.raises(RuntimeError, match="cu_seqlens"):
        ops.check_status()
    ops.check_status()         # the word was cleared by the raise
    out = nanobrain_b200.sdpa_varlen(t, t, t, W.cu_seqlens_from_lengths(lengths).to(DEV),
                                     W.cu_seqlens_from_lengths(lengths).to(DEV), 200, 200)
    ops.check_status()
    assert torch.isfinite(out.float()).all()


def run_varlen(lengths, heads, seed):
    q, k, v, g = (t.to(torch.bfloat16).float() for t in W.make_packed_inputs(lengths, heads, seed=seed))
    cu = W.cu_seqlens_from_lengths(lengths)
    qd, kd, vd = (t.to(DEV, torch.bfloat16).requires_grad_(True) for t in (q, k, v))
    out = nanobrain_b200.sdpa_varlen(qd, kd, vd, cu.to(DEV), cu.to(DEV), int(lengths.max()), int(lengths.max()))
    out.backward(g.to(DEV, torch.bfloat16))
    ops.check_status()
    want = O.varlen_fwd_bwd(q.numpy(), k.numpy(), v.numpy(), g.numpy(), cu.numpy(), cu.numpy(), dtype=np.float32)
    return (out, qd.grad, kd.grad, vd.grad), (want[0], want[2], want[3], want[4])


@pytest.mark.parametrize("lengths", [
    [200] * 30 + [2000],                   # one long sequence among many short ones
    [2000] + [200] * 30,
    [16, 1500, 17, 129, 640, 15, 1, 128],  # ragged tiles of every size next to full ones
    [129, 130, 144, 145, 820],             # lengths around the 16-row trimming granularity
])
def test_skewed_length_mixes_match_the_oracle(lengths):
    got, want = run_varlen(torch.tensor(lengths), heads=2, seed=len(lengths))
    for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        err = np.abs(a.detach().float().cpu().numpy() - b)
        assert np.isfinite(err).all(), name
        assert err.max() <= MAX_ABS * max(1.0, np.abs(b).max()) and err.mean() <= MEAN_ABS, (name, err.max(), err.mean())


def test_many_short_units_per_persistent_cta_match_the_oracle():
    # 500 sequences of 1..300 tokens and 3 heads: about 2400 backward work units of one, two or three
    # steps for the 148 persistent CTAs, so that every CTA runs a dozen units back to back (K buffer
    # alternation, one-step units, dV / dK leaving while the next unit has started) and the forward
    # runs several waves of short CTAs.
    g = torch.Generator().manual_seed(7)
    lengths = torch.randint(1, 301, (500,), generator=g)
    got, want = run_varlen(lengths, heads=3, seed=11)
    for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        err = np.abs(a.detach().float().cpu().numpy() - b)
        assert np.isfinite(err).all(), name
        assert err.max() <= MAX_ABS * max(1.0, np.abs(b).max()) and err.mean() <= MEAN_ABS, (name, err.max(), err.mean())

