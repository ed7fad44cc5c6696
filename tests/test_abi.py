"""The C-ABI library loads on a machine without a GPU, exports every symbol the header declares,
and rejects bad arguments before it touches CUDA."""

import ctypes as C
import re
from pathlib import Path

import pytest

from nanobrain_b200 import _lib, build

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def declared_functions():
    text = (ROOT / "include" / "nb_attn.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nb_attn_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_list_the_same_symbols():
    assert declared_functions() == sorted(_lib.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol(lib):
    for name in declared_functions():
        assert hasattr(lib, name), name


def test_abi_version_and_strerror(lib):
    assert lib.nb_attn_abi_version() == _lib.ABI_VERSION
    assert lib.nb_attn_strerror(0) == b"ok"
    texts = {lib.nb_attn_strerror(c) for c in range(1, 10)}
    assert len(texts) == 9 and b"unknown error code" not in texts
    assert lib.nb_attn_strerror(999) == b"unknown error code"


def test_workspace_bytes(lib):
    # dense: fp32 dQ accumulator [T][H][64] + fp32 delta [H*T]; the forward needs nothing
    dense = _shape(batch=2, heads=12, max_seqlen_q=820, max_seqlen_k=820, total_q=1640, total_k=1640)
    assert _lib.bwd_workspace_bytes(dense) == 1640 * 12 * (64 * 4 + 4)
    assert _lib.fwd_workspace_bytes(dense) == 0
    # varlen: plus the work list, total / 128 + batch + 1 entries of 32 bytes (after 256-byte alignment)
    packed = _shape(batch=32, heads=12, max_seqlen_q=920, max_seqlen_k=920, total_q=26253, total_k=26253,
                    cu_seqlens_q=0x100, cu_seqlens_k=0x100)
    items = 26253 // 128 + 32 + 1
    assert lib.nb_attn_schedule_capacity(26253, 32) == items
    assert _lib.fwd_workspace_bytes(packed) == 32 * items
    accum = 26253 * 12 * (64 * 4 + 4)
    assert _lib.bwd_workspace_bytes(packed) == (accum + 255) // 256 * 256 + 32 * items
    assert _lib.bwd_workspace_bytes(_shape(batch=0)) == 0


def _shape(**kw):
    base = dict(batch=1, heads=2, head_dim=64, max_seqlen_q=16, max_seqlen_k=16, total_q=16, total_k=16,
                cu_seqlens_q=None, cu_seqlens_k=None, scale=0.125)
    base.update(kw)
    return _lib.Shape(**base)


def _tensor(ptr=0x10000, sb=2048, st=128, sh=64):
    return _lib.Tensor(ptr, sb, st, sh)


def test_fwd_rejects_bad_arguments_without_a_gpu(lib):
    ok = _tensor()
    cases = [
        (_lib.FwdArgs(_shape(head_dim=128), ok, ok, ok, ok, 0x10000, None, None, 0), 2),
        (_lib.FwdArgs(_shape(batch=0), ok, ok, ok, ok, 0x10000, None, None, 0), 3),
        (_lib.FwdArgs(_shape(total_q=17), ok, ok, ok, ok, 0x10000, None, None, 0), 3),
        (_lib.FwdArgs(_shape(scale=0.0), ok, ok, ok, ok, 0x10000, None, None, 0), 3),
        (_lib.FwdArgs(_shape(cu_seqlens_q=0x100), ok, ok, ok, ok, 0x10000, None, None, 0), 3),
        (_lib.FwdArgs(_shape(), _tensor(ptr=None), ok, ok, ok, 0x10000, None, None, 0), 1),
        (_lib.FwdArgs(_shape(), _tensor(ptr=0x10008), ok, ok, ok, 0x10000, None, None, 0), 4),
        (_lib.FwdArgs(_shape(), ok, _tensor(st=100), ok, ok, 0x10000, None, None, 0), 4),
        (_lib.FwdArgs(_shape(), ok, ok, ok, ok, None, None, None, 0), 1),
    ]
    for args, want in cases:
        assert lib.nb_attn_fwd(C.byref(args), None) == want
    assert lib.nb_attn_fwd(None, None) == 1
    # varlen mode needs the work-list workspace
    packed = _shape(cu_seqlens_q=0x100, cu_seqlens_k=0x100)
    assert lib.nb_attn_fwd(C.byref(_lib.FwdArgs(packed, ok, ok, ok, ok, 0x10000, None, None, 0)), None) == 5
    assert lib.nb_attn_fwd(C.byref(_lib.FwdArgs(packed, ok, ok, ok, ok, 0x10000, None, 0x20000, 3)), None) == 5


def test_bwd_rejects_bad_workspace_without_a_gpu(lib):
    ok = _tensor()
    need = _lib.bwd_workspace_bytes(_shape())
    mk = lambda ws, nbytes: _lib.BwdArgs(_shape(), ok, ok, ok, ok, ok, ok, ok, ok, 0x10000, ws, nbytes, None, None, None)
    assert lib.nb_attn_bwd(C.byref(mk(None, need)), None) == 5
    assert lib.nb_attn_bwd(C.byref(mk(0x20000, need - 1)), None) == 5
    assert lib.nb_attn_bwd(C.byref(mk(0x20010, need)), None) == 5  # not 256-byte aligned
    with pytest.raises(RuntimeError, match="workspace"):
        _lib.check(5, "nb_attn_bwd")
