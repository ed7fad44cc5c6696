"""Generates the golden fixtures in this directory from the reference's own code path.

Run where a checkout of the reference project is available, giving its root directory:

    python tests/golden/make_golden.py <path to the nanobrain checkout>

Two fixtures are written (fp32, CPU):

``sdpa_small.npz``
    Inputs and outputs of ``F.scaled_dot_product_attention(q, k, v, is_causal=False)`` followed by
    ``out.backward(d_out)`` -- the exact call of ``src/nanobrain/modules.py:62`` -- for a small
    ragged-size case (Lq != Lk, neither a multiple of any tile size).

``attention_module.npz``
    The reference's unmodified ``Attention`` module (``src/nanobrain/modules.py:21-65``) imported
    from the source tree, with seeded weights: input, output, and gradients of the input and of
    the four Linear weights. ``timm.layers.DropPath`` (imported at ``modules.py:13``, not
    installed here and unused by ``Attention``) is stubbed.

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


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the nanobrain checkout>")
    root = Path(sys.argv[1])
    make_sdpa_small()
    make_attention_module(root)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))
