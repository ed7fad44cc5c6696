"""The packed-token model path on the GPU: the mirrors of the reference's ``Block`` and ``ViTMAE3D``
against fixtures generated from the reference's own modules (``tests/golden/make_golden.py``), and
the packed (varlen) encoder / MAE step / batched eval against the dense per-sequence path built
from those fixture-checked modules."""

import importlib.util

import numpy as np
import pytest
import torch

from nanobrain_b200 import model as M
from nanobrain_b200 import modules, ops
from nanobrain_b200 import token_prep as T

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def golden(golden_dir):
    spec = importlib.util.spec_from_file_location("make_golden", golden_dir / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def tiny(golden_dir):
    return np.load(golden_dir / "mae_tiny.npz")


def rel_err(got, want):
    want = torch.as_tensor(np.asarray(want), dtype=torch.float32)
    got = got.detach().float().cpu()
    return ((got - want).abs().max() / want.abs().max().clamp_min(1e-6)).item()


def check_grad_summaries(module, fixture, rtol):
    """Gradient of every parameter against the reference's: first values and the squared norm."""
    worst = 0.0
    for name, p in module.named_parameters():
        ref_sq = float(fixture["gsq." + name])
        got_sq = float(p.grad.double().square().sum().item()) if p.grad is not None else 0.0
        # A gradient is measured against its own size, but not below that of the largest gradient of
        # the same kind (weight / bias) in the module: the key bias gradient, for one, is analytically
        # zero (softmax ignores a per-row constant) and only carries rounding noise.
        kind = name.rsplit(".", 1)[-1]
        family_sq = max(float(fixture["gsq." + n]) / max(q.numel(), 1) for n, q in module.named_parameters()
                        if n.rsplit(".", 1)[-1] == kind)
        scale = max(ref_sq ** 0.5, (family_sq * p.numel()) ** 0.5 * 0.1)
        assert abs(got_sq ** 0.5 - ref_sq ** 0.5) <= rtol * scale, name
        head = p.grad.reshape(-1)[:8].float().cpu().numpy() if p.grad is not None else np.zeros(8, np.float32)
        ref_head = fixture["ghead." + name]
        # individual entries against the size of a typical entry of this gradient (or of its family)
        typical = max((ref_sq / max(p.numel(), 1)) ** 0.5, 0.1 * family_sq ** 0.5, 1e-6)
        err = np.abs(head[:ref_head.size] - ref_head).max() / typical
        worst = max(worst, err)
        assert err <= 40 * rtol, (name, err)
    return worst


def test_block_matches_the_reference_block_fixture(golden, golden_dir):
    f = np.load(golden_dir / "block_module.npz")
    blk = modules.Block(dim=128, num_heads=2, qkv_bias=True, proj_bias=True, mlp_ratio=4, drop_path=0.0)
    golden.fill_parameters(blk)
    blk = blk.to(DEV)
    x = torch.from_numpy(f["x"]).to(DEV).requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):  # as the reference trains (train.py:286)
        y = blk(x)
    y.float().backward(torch.from_numpy(f["d_y"]).to(DEV))
    ops.check_status()
    assert rel_err(y, f["y"]) < 2e-2 and rel_err(x.grad, f["dx"]) < 3e-2
    check_grad_summaries(blk, f, rtol=3e-2)
    # the packed path over the same two sequences gives the same tokens
    cu = torch.tensor([0, 40, 80], dtype=torch.int32, device=DEV)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y_packed = blk(x.detach().reshape(80, 128), cu_seqlens=cu, max_seqlen=40)
    assert rel_err(y_packed.reshape(2, 40, 128), f["y"]) < 2e-2


def test_dense_training_forward_matches_the_reference_model_fixture(golden, tiny):
    # model.py:167-233 on the reference's own model, same weights, same global RNG state
    model = M.ViTMAE3D(**golden.TINY)
    golden.fill_parameters(model)
    model = model.to(DEV)
    images, mask = torch.from_numpy(tiny["images"]).to(DEV), torch.from_numpy(tiny["mask"]).to(DEV)
    order = torch.from_numpy(np.concatenate([tiny["state.vis_ids"], tiny["state.target_ids"]], axis=1))
    order = order.reshape(3, 2, 32).to(DEV)
    p = model.patch_size[0]
    patches, mask_patches = M.patchify3d(images, p), M.patchify3d(mask, p)
    bid = torch.arange(3, device=DEV)[:, None, None]
    seq_patches, seq_mask = patches[bid, order].flatten(0, 1), mask_patches[bid, order].flatten(0, 1)
    seq_coord = model.coord_grid.expand(3, -1, -1)[bid, order].flatten(0, 1)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        embeds = model.forward_encoder(seq_patches[:, :12], seq_coord[:, :12])
        pred = model.forward_decoder(embeds, seq_coord[:, 12:])
    loss = (seq_mask[:, 12:] * (pred.float() - seq_patches[:, 12:]) ** 2).sum() / seq_mask[:, 12:].sum()
    loss.backward()
    ops.check_status()
    assert rel_err(embeds, tiny["state.embeds"]) < 3e-2
    assert rel_err(pred, tiny["state.pred_patches"]) < 3e-2
    assert abs(loss.item() - float(tiny["loss"])) < 2e-2 * float(tiny["loss"])
    check_grad_summaries(model, tiny, rtol=5e-2)


def per_sequence_dense_step(model, images, mask, order, counts):
    """The same MAE step with every sequence run alone through the dense operator."""
    p = model.patch_size[0]
    b, s, seq_length = order.shape
    patches, mask_patches = M.patchify3d(images, p), M.patchify3d(mask, p)
    coord = model.coord_grid.expand(b, -1, -1)
    num = torch.zeros((), device=images.device)
    den = torch.zeros((), device=images.device)
    preds = []
    for i in range(b):
        for j in range(s):
            n = int(counts[i * s + j])
            ids = order[i, j]
            with torch.autocast("cuda", dtype=torch.bfloat16):
                emb = model.forward_encoder(patches[i, ids[:n]][None], coord[i, ids[:n]][None])
                pred = model.forward_decoder(emb, coord[i, ids[n:]][None])
            w = mask_patches[i, ids[n:]][None]
            num = num + (w * (pred.float() - patches[i, ids[n:]][None]) ** 2).sum()
            den = den + w.sum()
            preds.append(pred[0])
    return num / den, preds


def test_packed_mae_step_matches_the_per_sequence_dense_path(golden, tiny):
    # patchify -> counts -> order -> pack -> encoder blocks (varlen) -> unpack -> decoder block
    # (dense) -> masked MSE -> backward, against the per-sequence dense path of the same modules
    model = M.ViTMAE3D(**golden.TINY)
    golden.fill_parameters(model)
    model = model.to(DEV)
    images, mask = torch.from_numpy(tiny["images"]).to(DEV), torch.from_numpy(tiny["mask"]).to(DEV)
    mask_frac = M.patchify3d(mask, 4).mean(dim=2)
    counts = T.visible_counts(mask_frac, visible_ratio=0.4)        # ragged: in-mask counts differ per image
    assert len(set(counts.tolist())) > 1
    torch.manual_seed(3)
    order = M.sample_sequences(M.patchify3d(mask, 4), 2, 40)
    counts_seq = counts[:, None].expand(3, 2).reshape(-1)

    def grads():
        out = [p.grad.detach().float().clone() for p in model.parameters()]
        for p in model.parameters():
            p.grad = None
        return out

    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss_p, state = model.forward_packed(images, mask, counts, max_visible=int(counts.max()), seq_length=40,
                                             num_samples=2, order=order)
    loss_p.backward()
    g_p = grads()
    loss_d, preds = per_sequence_dense_step(model, images, mask, order, counts_seq)
    loss_d.backward()
    g_d = grads()
    ops.check_status()
    assert abs(loss_p.item() - loss_d.item()) < 1e-2 * abs(loss_d.item())
    for n, pred in enumerate(preds):
        c = int(counts_seq[n])
        assert rel_err(state["pred_patches"][n, c:], pred.detach().float().cpu().numpy()) < 3e-2
    for (name, _), a, b in zip(model.named_parameters(), g_p, g_d):
        assert (a - b).abs().max() <= 4e-2 * max(b.abs().max().item(), 1e-4), name
    # with equal counts the packed step is the reference's fixed-length step: the fixture's loss
    order13 = torch.from_numpy(np.concatenate([tiny["state.vis_ids"], tiny["state.target_ids"]], 1)).reshape(3, 2, 32)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss_eq, _ = model.forward_packed(images, mask, torch.full((3,), 12, device=DEV), max_visible=12,
                                          seq_length=32, num_samples=2, order=order13.to(DEV))
    ops.check_status()
    assert abs(loss_eq.item() - float(tiny["loss"])) < 2e-2 * float(tiny["loss"])


def test_batched_varlen_eval_matches_the_one_image_per_forward_loop(golden, tiny):
    # model.py:247-286 runs one encoder forward per image; embed_packed runs all images in one pass
    model = M.ViTMAE3D(**golden.TINY)
    golden.fill_parameters(model)
    model = model.to(DEV).eval()
    images = torch.from_numpy(tiny["images"]).to(DEV)
    in_mask = torch.from_numpy(tiny["in_mask"]).to(DEV)
    patches = M.patchify3d(images, 4)
    lengths = in_mask.sum(dim=1).tolist()
    assert len(set(lengths)) == 3                                    # ragged
    samples = [(patches[i], in_mask[i]) for i in range(3)]
    outs = model.embed_packed(samples, return_dense=True)
    ops.check_status()
    for i, out in enumerate(outs):
        assert rel_err(out["global_embedding"], tiny[f"embed.{i}"]) < 3e-2     # the reference's own output
        dense = out["dense_embedding"].reshape(-1, model.embed_dim)
        assert rel_err(dense[in_mask[i]], tiny[f"tokens.{i}"]) < 3e-2
        assert bool((dense[~in_mask[i]] == 0).all()) and out["dense_mask"].sum().item() == lengths[i]
        # and the per-image loop on the same device with the same modules
        with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
            tokens = model.forward_encoder(patches[i:i + 1, in_mask[i]], model.coord_grid[:, in_mask[i]])
        want = tokens[0, model.class_tokens:].float().mean(dim=0)
        assert rel_err(out["global_embedding"], want.cpu().numpy()) < 2e-2


def test_fixed_capacity_packing_leaves_no_undefined_rows():
    # Packing into a buffer of fixed capacity (no device-to-host sync) leaves unused rows at the end;
    # the operator writes zeros there, so garbage can never leak into weight gradients.
    lengths = torch.tensor([70, 129, 33])
    total, cap, heads = int(lengths.sum()), 400, 2
    cu = T.cu_seqlens_from_counts(lengths).to(DEV)
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(cap, heads, 64, generator=g).to(DEV, torch.bfloat16).requires_grad_(True) for _ in range(3))
    out, lse = ops.sdpa_varlen_fwd(q, k, v, cu, cu, 129, 129, 0.125)
    d_out = torch.randn(cap, heads, 64, generator=g).to(DEV, torch.bfloat16)
    d_out[total:] = 1000.0     # whatever (finite) values autograd hands back for rows nobody owns
    out.backward(d_out)
    ops.check_status()
    assert bool((out[total:] == 0).all()) and bool(torch.isinf(lse[:, total:]).all())
    for t in (q.grad, k.grad, v.grad):
        assert bool((t[total:] == 0).all()) and bool(torch.isfinite(t.float()).all())
    ref_q, ref_k, ref_v = (t.detach()[:total].clone().requires_grad_(True) for t in (q, k, v))
    ref = ops.sdpa_varlen(ref_q, ref_k, ref_v, cu, cu, 129, 129)
    ref.backward(d_out[:total])
    assert torch.equal(ref, out[:total]) and torch.equal(ref_k.grad, k.grad[:total])
