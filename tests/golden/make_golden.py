"""Generates the golden fixtures in this directory from the reference's own code path.

Run where a checkout of the reference project is available, giving its root directory:

    python tests/golden/make_golden.py <path to the nanobrain checkout>

Fixtures written (fp32, CPU):

``sdpa_small.npz``
    Inputs and outputs of ``F.scaled_dot_product_attention(q, k, v, is_causal=False)`` followed by
    ``out.backward(d_out)`` -- the exact call of ``src/nanobrain/modules.py:62`` -- for a small
    ragged-size case (Lq != Lk, neither a multiple of any tile size).

``attention_module.npz``
    The reference's unmodified ``Attention`` module (``src/nanobrain/modules.py:21-65``) imported
    from the source tree, with seeded weights: input, output, and gradients of the input and of
    the four Linear weights. ``timm.layers.DropPath`` (imported at ``modules.py:13``, not
    installed here and unused by ``Attention``) is stubbed.

``block_module.npz``
    The reference's unmodified ``Block`` (``src/nanobrain/modules.py:92-131``) built with the
    keyword arguments its model passes (``src/nanobrain/model.py:68-75``): input, output, input
    gradient and a checksum of every parameter gradient. Parameters are not stored: both sides
    fill them with :func:`fill_parameters`, a function of the parameter's name only.

``mae_tiny.npz``
    The reference's unmodified ``ViTMAE3D`` (``src/nanobrain/model.py:21-233``) on a 16^3 grid
    with 4^3 patches: ``sample_sequences`` orders under a seeded global RNG
    (``model.py:347-363``), the gathered visible / target patches (``model.py:186-199``), the
    encoder output, the loss and gradient checksums of one training forward + backward, and the
    per-image encoder output of the eval loop of ``model.py:254-276`` for ragged in-mask counts.
    ``brainmarks_smri``, ``nibabel`` and ``timm`` (not installed here, unused on this path) are
    stubbed; the decoder head, which the reference initialises to zero, gets seeded values so
    that gradients reach the rest of the network.

The fixtures travel with the repository; the reference tree does not, so tests only read the
``.npz`` files.
"""

from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent


def fill_parameters(module: torch.nn.Module, std: float = 0.05) -> None:
    """Deterministic parameter values that depend only on the parameter's NAME and shape, so that
    the reference module and its mirror get identical weights without storing them."""
    import zlib

    with torch.no_grad():
        for name, p in module.named_parameters():
            g = torch.Generator().manual_seed(zlib.crc32(name.encode()))
            v = torch.randn(p.shape, generator=g) * std
            if name.endswith("norm.weight") or ".norm1.weight" in name or ".norm2.weight" in name:
                v = 1.0 + v
            p.copy_(v)


def stub_missing_packages() -> None:
    timm = types.ModuleType("timm")
    layers = types.ModuleType("timm.layers")

    class DropPath(torch.nn.Identity):
        def __init__(self, drop_prob: float = 0.0):
            super().__init__()

    layers.DropPath = DropPath
    timm.layers = layers
    sys.modules.setdefault("timm", timm)
    sys.modules.setdefault("timm.layers", layers)
    bm = types.ModuleType("brainmarks_smri")
    bm_models = types.ModuleType("brainmarks_smri.models")
    bm_models.EmbeddingOutput = dict
    bm_models.ImageInput = dict
    bm_models.register_model = lambda fn: fn
    bm.models = bm_models
    sys.modules.setdefault("brainmarks_smri", bm)
    sys.modules.setdefault("brainmarks_smri.models", bm_models)
    sys.modules.setdefault("nibabel", types.ModuleType("nibabel"))


def load_reference_package(ref_root: Path):
    """Import the reference's ``nanobrain.modules`` and ``nanobrain.model`` from its source tree
    (it has no ``__init__.py``: a namespace package on the source path)."""
    stub_missing_packages()
    src = str(ref_root / "src")
    if src not in sys.path:
        sys.path.insert(0, src)
    import importlib

    return importlib.import_module("nanobrain.modules"), importlib.import_module("nanobrain.model")


def load_reference_modules(ref_root: Path):
    timm = types.ModuleType("timm")
    layers = types.ModuleType("timm.layers")

    class DropPath(torch.nn.Identity):
        def __init__(self, drop_prob: float = 0.0):
            super().__init__()

    layers.DropPath = DropPath
    timm.layers = layers
    sys.modules.setdefault("timm", timm)
    sys.modules.setdefault("timm.layers", layers)
    spec = importlib.util.spec_from_file_location("nanobrain_ref_modules", ref_root / "src/nanobrain/modules.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def make_sdpa_small():
    g = torch.Generator().manual_seed(1234)
    q = torch.randn(2, 3, 37, 64, generator=g)
    k = torch.randn(2, 3, 53, 64, generator=g)
    v = torch.randn(2, 3, 53, 64, generator=g)
    d_out = torch.randn(2, 3, 37, 64, generator=g)
    q.requires_grad_(True)
    k.requires_grad_(True)
    v.requires_grad_(True)
    out = F.scaled_dot_product_attention(q, k, v, is_causal=False)
    out.backward(d_out)
    np.savez_compressed(
        HERE / "sdpa_small.npz",
        q=q.detach().numpy(), k=k.detach().numpy(), v=v.detach().numpy(), d_out=d_out.numpy(),
        out=out.detach().numpy(), dq=q.grad.numpy(), dk=k.grad.numpy(), dv=v.grad.numpy(),
    )


def make_attention_module(ref_root: Path):
    ref = load_reference_modules(ref_root)
    torch.manual_seed(4321)
    attn = ref.Attention(dim=128, num_heads=2, qkv_bias=True, proj_bias=True)
    x = torch.randn(2, 50, 128, requires_grad=True)
    d_y = torch.randn(2, 50, 128)
    y = attn(x)
    y.backward(d_y)
    arrays = {"x": x.detach().numpy(), "d_y": d_y.numpy(), "y": y.detach().numpy(), "dx": x.grad.numpy()}
    for name, p in attn.named_parameters():
        arrays["param." + name] = p.detach().numpy()
        arrays["grad." + name] = p.grad.numpy()
    np.savez_compressed(HERE / "attention_module.npz", **arrays)


def checksums(module: torch.nn.Module) -> dict:
    """Per-parameter gradient summaries: sum, sum of squares and the first 8 values."""
    out = {}
    for name, p in module.named_parameters():
        g = p.grad if p.grad is not None else torch.zeros_like(p)
        out["gsum." + name] = np.float64(g.double().sum().item())
        out["gsq." + name] = np.float64(g.double().square().sum().item())
        out["ghead." + name] = g.reshape(-1)[:8].numpy().copy()
    return out


def make_block_module(ref_root: Path):
    ref_modules, _ = load_reference_package(ref_root)
    # the keyword arguments of src/nanobrain/model.py:68-75
    blk = ref_modules.Block(dim=128, num_heads=2, qkv_bias=True, proj_bias=True, mlp_ratio=4, drop_path=0.0)
    fill_parameters(blk)
    g = torch.Generator().manual_seed(99)
    x = torch.randn(2, 40, 128, generator=g).requires_grad_(True)
    d_y = torch.randn(2, 40, 128, generator=g)
    y = blk(x)
    y.backward(d_y)
    np.savez_compressed(HERE / "block_module.npz", x=x.detach().numpy(), d_y=d_y.numpy(), y=y.detach().numpy(),
                        dx=x.grad.numpy(), **checksums(blk))


TINY = dict(grid_size=(16, 16, 16), patch_size=4, depth=2, embed_dim=128, num_heads=2, decoder_depth=1,
            decoder_embed_dim=128, decoder_num_heads=2, class_tokens=1)


def tiny_inputs():
    g = torch.Generator().manual_seed(7)
    images = torch.randn(3, 16, 16, 16, generator=g)
    # ball-shaped masks of different radii: the in-mask patch counts differ per image
    ax = torch.arange(16, dtype=torch.float32) - 7.5
    r2 = ax[:, None, None] ** 2 + ax[None, :, None] ** 2 + ax[None, None, :] ** 2
    mask = torch.stack([(r2 <= rad ** 2).float() for rad in (7.5, 6.0, 4.5)])
    return images, mask


def make_mae_tiny(ref_root: Path):
    _, ref_model = load_reference_package(ref_root)
    model = ref_model.ViTMAE3D(target_spacing=1.0, **TINY)
    fill_parameters(model)
    images, mask = tiny_inputs()
    arrays = {"images": images.numpy(), "mask": mask.numpy()}

    # sample_sequences under a seeded global RNG (model.py:347-363)
    mask_patches = ref_model.patchify3d(mask, 4)
    torch.manual_seed(11)
    arrays["order_s2_all"] = ref_model.sample_sequences(mask_patches, 2).numpy()
    torch.manual_seed(12)
    arrays["order_s3_len20"] = ref_model.sample_sequences(mask_patches, 3, 20).numpy()

    # one training forward + backward (model.py:167-233), fixed num_visible
    torch.manual_seed(13)
    loss, state = model(images, mask, num_visible=12, num_predict=20, num_samples=2)
    loss.backward()
    arrays["loss"] = np.float64(loss.item())
    for key in ("vis_patches", "target_patches", "target_mask_patches", "embeds", "pred_patches", "vis_ids",
                "target_ids"):
        arrays["state." + key] = state[key].detach().numpy()
    arrays.update(checksums(model))

    # the eval loop of model.py:254-276: one encoder forward per image over its in-mask patches
    patches = ref_model.patchify3d(images, 4)
    in_mask = (mask_patches > 0).any(dim=2)
    with torch.no_grad():
        for i in range(images.shape[0]):
            tokens = model.forward_encoder(patches[i:i + 1, in_mask[i]], model.coord_grid[:, in_mask[i]])
            tokens = tokens[0, model.class_tokens:].float()
            arrays[f"embed.{i}"] = tokens.mean(dim=0).numpy()
            arrays[f"tokens.{i}"] = tokens.numpy()
    arrays["in_mask"] = in_mask.numpy()
    np.savez_compressed(HERE / "mae_tiny.npz", **arrays)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the nanobrain checkout>")
    root = Path(sys.argv[1])
    make_sdpa_small()
    make_attention_module(root)
    make_block_module(root)
    make_mae_tiny(root)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))
