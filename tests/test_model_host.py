"""Host-side parts of the packed-token model path, checked on the CPU against fixtures generated
from the reference's own ``Block``, ``ViTMAE3D``, ``sample_sequences`` and gather
(``tests/golden/make_golden.py``). Attention itself has no CPU path: the numerics of the modules
are covered by the GPU tests."""

import importlib.util

import numpy as np
import pytest
import torch

from nanobrain_b200 import model as M
from nanobrain_b200 import modules
from nanobrain_b200 import token_prep as T


@pytest.fixture(scope="module")
def golden(golden_dir):
    spec = importlib.util.spec_from_file_location("make_golden", golden_dir / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def tiny(golden_dir):
    return np.load(golden_dir / "mae_tiny.npz")


def test_block_takes_the_keyword_arguments_the_reference_model_passes(golden_dir):
    # src/nanobrain/model.py:68-75 builds Block(dim=, num_heads=, qkv_bias=, proj_bias=, mlp_ratio=, drop_path=)
    blk = modules.Block(dim=128, num_heads=2, qkv_bias=True, proj_bias=True, mlp_ratio=4, drop_path=0.0)
    assert isinstance(blk.drop_path1, torch.nn.Identity) and isinstance(blk.drop_path2, torch.nn.Identity)
    f = np.load(golden_dir / "block_module.npz")
    assert {n for n, _ in blk.named_parameters()} == {k[len("gsum."):] for k in f.files if k.startswith("gsum.")}
    dropped = modules.Block(dim=128, num_heads=2, drop_path=0.25, norm_layer=modules.LayerNorm)
    assert isinstance(dropped.drop_path1, modules.DropPath) and dropped.drop_path2.drop_prob == 0.25
    assert blk.norm1.eps == 1e-6


def test_drop_path_drops_whole_samples_and_whole_packed_sequences():
    dp = modules.DropPath(0.5).train()
    torch.manual_seed(0)
    y = dp(torch.ones(64, 5, 3))
    per_sample = y.reshape(64, -1)
    assert all(row.unique().numel() == 1 for row in per_sample)      # a sample is kept or dropped as a whole
    assert set(y.unique().tolist()) == {0.0, 2.0}                    # kept samples are scaled by 1 / keep
    seq_id = torch.tensor([0, 0, 0, 1, 2, 2])
    z = dp(torch.ones(6, 4), seq_id=seq_id, num_seqs=3)
    assert z[0].equal(z[1]) and z[1].equal(z[2]) and z[4].equal(z[5])
    assert dp.eval()(torch.ones(4, 2)).equal(torch.ones(4, 2))


def test_model_has_the_reference_parameter_names(golden, tiny):
    model = M.ViTMAE3D(**golden.TINY)
    want = {k[len("gsum."):] for k in tiny.files if k.startswith("gsum.")}
    assert {n for n, _ in model.named_parameters()} == want
    assert model.coord_grid.shape == (1, 64, 3) and "coord_grid" not in model.state_dict()


def test_sample_sequences_matches_the_reference_under_the_same_seed(tiny):
    mask_patches = M.patchify3d(torch.from_numpy(tiny["mask"]), 4)
    torch.manual_seed(11)
    assert np.array_equal(M.sample_sequences(mask_patches, 2).numpy(), tiny["order_s2_all"])
    torch.manual_seed(12)
    assert np.array_equal(M.sample_sequences(mask_patches, 3, 20).numpy(), tiny["order_s3_len20"])


def test_packed_gather_matches_the_reference_gather(tiny):
    # The reference gathers a fixed number of visible patches per sequence (model.py:186-199); with
    # equal counts the packed gather must produce the same rows in the same order.
    images, mask = torch.from_numpy(tiny["images"]), torch.from_numpy(tiny["mask"])
    patches, mask_patches = M.patchify3d(images, 4), M.patchify3d(mask, 4)
    torch.manual_seed(13)
    order = M.sample_sequences(mask_patches, 2, 32)
    coord = M.make_coord_grid((16, 16, 16), 4).expand(3, -1, -1)
    counts = torch.full((3, 2), 12, dtype=torch.int64)
    tokens, tok_coord, cu, seq_id, patch_id, valid = T.pack_visible_tokens(patches, coord, order, counts)
    assert cu.tolist() == [12 * i for i in range(7)] and bool(valid.all())
    assert np.array_equal(tokens.reshape(6, 12, 64).numpy(), tiny["state.vis_patches"])
    assert np.array_equal(patch_id.reshape(6, 12).numpy(), tiny["state.vis_ids"])
    assert torch.equal(tok_coord, coord[0][patch_id])
    # the same with a fixed-capacity buffer (no device-to-host sync): padding rows at the end
    tokens_c, _, cu_c, _, _, valid_c = T.pack_visible_tokens(patches, coord, order, counts, capacity=80)
    assert tokens_c.shape[0] == 80 and int(valid_c.sum()) == 72 and torch.equal(cu_c, cu)
    assert torch.equal(tokens_c[:72], tokens)
    # targets of the dense path: the remaining patches of every sequence, as model.py:193-197 splits them
    bid = torch.arange(3)[:, None, None]
    assert np.array_equal(patches[bid, order].flatten(0, 1)[:, 12:].numpy(), tiny["state.target_patches"])


def test_class_token_offsets_of_the_packed_encoder_layout():
    # model.py:135-136 prepends R class tokens to every sequence; packed, sequence i moves by R*i rows
    model = M.ViTMAE3D(grid_size=(16, 16, 16), patch_size=4, depth=0, embed_dim=128, num_heads=2, decoder_depth=0,
                       decoder_embed_dim=128, decoder_num_heads=2, class_tokens=2)
    lengths = torch.tensor([3, 1, 4])
    cu = T.cu_seqlens_from_counts(lengths)
    tokens = torch.randn(10, 64)  # two spare rows at the end (fixed-capacity packing)
    coord = torch.zeros(10, 3)
    x, cu_r, max_r, seq_r, is_cls = model.forward_encoder_packed(tokens, coord, cu, 4)
    assert cu_r.tolist() == [0, 5, 8, 14] and max_r == 6 and x.shape == (16, 128)
    assert is_cls.tolist() == [True, True, False, False, False, True, True, False, True, True] + [False] * 6
    assert seq_r[:14].tolist() == [0] * 5 + [1] * 3 + [2] * 6
    # class-token rows carry the (normalised) class token, patch rows the embedded patches in order
    body = model.norm(model.pos_embed(model.patch_embed(tokens), coord))
    assert torch.allclose(x[2:5], body[0:3]) and torch.allclose(x[7:8], body[3:4]) and torch.allclose(x[10:14], body[4:8])
    assert torch.allclose(x[0:2], model.norm(model.cls_token[0])) and torch.allclose(x[5:7], x[0:2])
