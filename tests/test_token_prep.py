"""Packed-token preparation (CPU): the varlen replacement for the reference's fixed-length visible
gather (src/nanobrain/model.py:186-199, sample_sequences at model.py:347-363)."""

import torch

from nanobrain_b200 import token_prep as T


def _setup(seed=0, b=4, p=60, dim=5):
    g = torch.Generator().manual_seed(seed)
    mask_frac = torch.rand(b, p, generator=g)
    mask_frac[0, : p - 7] = 0.0  # an image with only 7 in-mask patches
    patches = torch.randn(b, p, dim, generator=g)
    coords = torch.stack(torch.meshgrid(torch.arange(3), torch.arange(4), torch.arange(5), indexing="ij"), -1).reshape(1, p, 3)
    return mask_frac, patches, coords, g


def test_order_puts_out_of_mask_patches_last_like_the_reference():
    mask_frac, _, _, g = _setup()
    order = T.sample_order(mask_frac, num_samples=3, generator=g)
    assert order.shape == (4, 3, 60)
    for b in range(4):
        n_in = int((mask_frac[b] >= 0.25).sum())
        for s in range(3):
            assert sorted(order[b, s].tolist()) == list(range(60))  # a permutation
            assert bool((mask_frac[b][order[b, s, :n_in]] >= 0.25).all())  # in-mask patches first
            assert bool((mask_frac[b][order[b, s, n_in:]] < 0.25).all())


def test_visible_counts_follow_the_mask():
    mask_frac, _, _, _ = _setup()
    counts = T.visible_counts(mask_frac, visible_ratio=0.2)
    want = [max(1, int(0.2 * int((mask_frac[b] >= 0.25).sum()))) for b in range(4)]
    assert counts.tolist() == want
    assert counts[0] == 1  # 7 in-mask patches -> 1 visible, not padded up with background


def test_pack_matches_a_per_sequence_loop():
    mask_frac, patches, coords, g = _setup()
    order = T.sample_order(mask_frac, num_samples=2, generator=g)
    counts = T.visible_counts(mask_frac, 0.3)
    tokens, tcoords, cu, seq_id, patch_id, valid = T.pack_visible_tokens(patches, coords, order, counts)
    assert cu.dtype == torch.int32 and cu[0] == 0 and valid.all()
    row = 0
    for b in range(4):
        for s in range(2):
            n = int(counts[b])
            ids = order[b, s, :n]
            seq = b * 2 + s
            assert cu[seq] == row and cu[seq + 1] == row + n
            assert torch.equal(tokens[row:row + n], patches[b, ids])
            assert torch.equal(tcoords[row:row + n], coords[0, ids])
            assert (seq_id[row:row + n] == seq).all() and torch.equal(patch_id[row:row + n], ids)
            row += n
    assert row == tokens.shape[0]


def test_capacity_mode_needs_no_sync_and_pads():
    mask_frac, patches, coords, g = _setup()
    order = T.sample_order(mask_frac, num_samples=1, generator=g)
    counts = T.visible_counts(mask_frac, 0.3)
    exact = T.pack_visible_tokens(patches, coords, order, counts)
    cap = 4 * 60
    padded = T.pack_visible_tokens(patches, coords, order, counts, capacity=cap)
    assert padded[0].shape[0] == cap
    assert int(padded[5].sum()) == exact[0].shape[0]
    assert torch.equal(padded[0][padded[5]], exact[0])
    assert torch.equal(padded[2], exact[2])  # same cu_seqlens: padding rows belong to no sequence


def test_unpack_and_segment_mean_roundtrip():
    mask_frac, patches, coords, g = _setup()
    order = T.sample_order(mask_frac, num_samples=1, generator=g)
    counts = T.visible_counts(mask_frac, 0.3)
    tokens, _, cu, seq_id, _, valid = T.pack_visible_tokens(patches, coords, order, counts, capacity=100)
    dense, mask = T.unpack_to_padded(tokens, cu, int(counts.max()), seq_id)
    means = T.segment_mean(tokens, cu, seq_id, valid)
    for i in range(4):
        n = int(counts[i])
        assert mask[i].sum() == n and torch.equal(dense[i, :n], tokens[cu[i]:cu[i + 1]])
        assert torch.all(dense[i, n:] == 0)
        assert torch.allclose(means[i], tokens[cu[i]:cu[i + 1]].mean(0), atol=1e-6)
