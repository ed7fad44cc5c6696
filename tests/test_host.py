"""Host-side logic of the custom ops that needs no GPU: argument policing (no fallback), fake
kernels (shapes and strides as the real op), and the drop-in module's parameter layout."""

import pytest
import torch

import nanobrain_b200
from nanobrain_b200 import modules, ops
from nanobrain_b200 import workloads as W


def test_unsupported_arguments_raise_instead_of_falling_back():
    q = torch.zeros(1, 2, 8, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="attn_mask"):
        nanobrain_b200.sdpa(q, q, q, attn_mask=torch.ones(8, 8, dtype=torch.bool))
    with pytest.raises(RuntimeError, match="dropout"):
        nanobrain_b200.sdpa(q, q, q, dropout_p=0.1)
    with pytest.raises(RuntimeError, match="is_causal"):
        nanobrain_b200.sdpa(q, q, q, is_causal=True)
    with pytest.raises(RuntimeError, match="enable_gqa"):
        nanobrain_b200.sdpa(q, q, q, enable_gqa=True)


def test_cpu_tensors_have_no_kernel():
    q = torch.zeros(1, 2, 8, 64, dtype=torch.bfloat16)
    with pytest.raises((RuntimeError, NotImplementedError)):
        nanobrain_b200.sdpa(q, q, q)


def test_fake_kernels_give_the_real_layouts():
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        x = torch.empty(3, 50, 12 * 64, dtype=torch.bfloat16, device="cuda")
        q = x.view(3, 50, 12, 64).transpose(1, 2)
        out, lse = ops.sdpa_fwd(q, q, q, 0.125)
        assert out.shape == (3, 12, 50, 64) and out.dtype == torch.bfloat16
        # memory is [B, L, H, 64] so the head merge of modules.py:63 stays a view
        assert out.stride() == (50 * 12 * 64, 64, 12 * 64, 1)
        assert out.transpose(1, 2).reshape(3, 50, 768).shape == (3, 50, 768)
        assert lse.shape == (3, 12, 50) and lse.dtype == torch.float32
        dq, dk, dv = ops.sdpa_bwd(out, q, q, q, out, lse, 0.125)
        assert dq.shape == q.shape and dk.stride() == out.stride()

        t = torch.empty(123, 12, 64, dtype=torch.bfloat16, device="cuda")
        cu = torch.empty(4, dtype=torch.int32, device="cuda")
        out, lse = ops.sdpa_varlen_fwd(t, t, t, cu, cu, 60, 60, 0.125)
        assert out.shape == (123, 12, 64) and lse.shape == (12, 123)
        grads = ops.sdpa_varlen_bwd(out, t, t, t, out, lse, cu, cu, 60, 60, 0.125)
        assert [g.shape for g in grads] == [t.shape] * 3


def test_attention_module_mirrors_reference_parameters(golden_dir):
    import numpy as np

    g = np.load(golden_dir / "attention_module.npz")
    attn = modules.Attention(dim=128, num_heads=2, qkv_bias=True, proj_bias=True)
    names = {n for n, _ in attn.named_parameters()}
    assert names == {k[len("param."):] for k in g.files if k.startswith("param.")}
    for n, p in attn.named_parameters():
        assert tuple(p.shape) == g["param." + n].shape
    with pytest.raises(ValueError):
        modules.Attention(dim=128, num_heads=4)  # head_dim 32
    with pytest.raises(ValueError):
        modules.Attention(dim=128, num_heads=2, causal=True)


def test_split_sequences_covers_every_sequence_once_and_balances_tokens():
    from nanobrain_b200.host_pipeline import split_sequences

    lengths = [int(x) for x in W.draw_lengths(W.WORKLOADS["vitb_encoder_varlen"])]
    for groups in (1, 3, 8, 32, 100):
        runs = split_sequences(lengths, groups)
        assert [i for r in runs for i in r] == list(range(len(lengths)))  # consecutive, complete, no overlap
        assert 1 <= len(runs) <= min(groups, len(lengths)) and all(len(r) > 0 for r in runs)
    tokens = [sum(lengths[i] for i in r) for r in split_sequences(lengths, 8)]
    assert max(tokens) <= 1.5 * sum(lengths) / 8
    assert split_sequences([5], 4) == [range(0, 1)]
    assert [list(r) for r in split_sequences([1, 1, 1], 3)] == [[0], [1], [2]]


def test_host_pipeline_refuses_a_cpu_device():
    from nanobrain_b200 import HostPipeline

    with pytest.raises(RuntimeError, match="CUDA"):
        HostPipeline([10, 20], 2, torch.device("cpu"))
