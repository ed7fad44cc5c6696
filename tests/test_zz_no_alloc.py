"""`nb_attn_bwd_builtin_scratch`: the backward entry point for callers that cannot allocate.

Some users of the library hold device pointers but no allocator: a host process that borrows
buffers from another runtime, a memory-planned training step whose pool is fully committed, or a
latency-critical loop where a `cudaMalloc` would stall the device. They pass inputs and outputs as
usual; the scratch the backward needs (fp32 dQ accumulator + row dots) lives in a fixed array
inside the library instead of in `args.workspace`.

The first call on a device resolves the array's address, so the GPU test passes in a fresh
process as well as after other tests have used the library.
"""

import ctypes as C

import pytest
import torch

from nanobrain_b200 import _lib, build
from nanobrain_b200 import workloads as W


def test_problems_beyond_the_builtin_scratch_are_refused_without_a_gpu():
    build.build()
    lib = _lib.load()
    ok = _lib.Tensor(0x10000, 2048, 128, 64)
    rows = _lib.BUILTIN_SCRATCH_ROWS
    too_big = _lib.Shape(1, 16, 64, rows // 16 + 1, rows // 16 + 1, rows // 16 + 1, rows // 16 + 1, None, None, 0.125)
    args = _lib.BwdArgs(too_big, ok, ok, ok, ok, ok, ok, ok, ok, 0x10000, None, 0, None, None, None)
    assert lib.nb_attn_bwd_builtin_scratch(C.byref(args), None) == 9
    assert b"NB_ATTN_BUILTIN_SCRATCH_ROWS" in lib.nb_attn_strerror(9)
    assert lib.nb_attn_bwd_builtin_scratch(None, None) == 1
    # a packed batch with more work-list entries than the array has room for
    many = _lib.BUILTIN_SCRATCH_ITEMS + 1
    too_many = _lib.Shape(many, 1, 64, 1, 1, many, many, 0x10000, 0x10000, 0.125)
    args = _lib.BwdArgs(too_many, ok, ok, ok, ok, ok, ok, ok, ok, 0x10000, None, 0, None, None, None)
    assert lib.nb_attn_bwd_builtin_scratch(C.byref(args), None) == 9


def test_builtin_scratch_entry_validates_like_the_workspace_entry_without_a_gpu():
    # Bad tensors are refused with the same codes as nb_attn_bwd, before CUDA is touched.
    build.build()
    lib = _lib.load()
    ok = _lib.Tensor(0x10000, 2048, 128, 64)
    shape = _lib.Shape(1, 2, 64, 16, 16, 16, 16, None, None, 0.125)
    cases = [(_lib.Tensor(None, 2048, 128, 64), 1), (_lib.Tensor(0x10008, 2048, 128, 64), 4),
             (_lib.Tensor(0x10000, 2048, 100, 64), 4)]
    for bad, want in cases:
        for slot in range(8):
            tensors = [ok] * 8
            tensors[slot] = bad
            args = _lib.BwdArgs(shape, *tensors, 0x10000, 0x20000, 1 << 20, None, None, None)
            assert lib.nb_attn_bwd_builtin_scratch(C.byref(args), None) == want
            assert lib.nb_attn_bwd(C.byref(args), None) == want
    args = _lib.BwdArgs(shape, *([ok] * 8), None, 0x20000, 1 << 20, None, None, None)  # lse missing
    assert lib.nb_attn_bwd_builtin_scratch(C.byref(args), None) == 1


def _backward_both_ways(lengths, heads, seed):
    """Run forward once, then backward through the caller-workspace entry point and through the
    built-in-scratch entry point, all through the C ABI. Returns the two (dq, dk, dv) triples."""
    dev = torch.device("cuda", 0)
    lib = _lib.load()
    total, max_len, nseq = int(lengths.sum()), int(lengths.max()), lengths.numel()
    cu = W.cu_seqlens_from_lengths(lengths).to(dev)
    q, k, v, g = (t.to(dev, torch.bfloat16) for t in W.make_packed_inputs(lengths, heads, seed=seed))
    out = torch.empty_like(q)
    lse = torch.empty((heads, total), dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    desc = lambda t: _lib.Tensor(t.data_ptr(), 0, t.stride(0), t.stride(1))
    shape = _lib.Shape(nseq, heads, 64, max_len, max_len, total, total, cu.data_ptr(), cu.data_ptr(), 0.125)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    fws_bytes = _lib.fwd_workspace_bytes(shape)
    fws = torch.empty(fws_bytes, dtype=torch.uint8, device=dev)
    fwd = _lib.FwdArgs(shape, desc(q), desc(k), desc(v), desc(out), lse.data_ptr(), status.data_ptr(),
                       fws.data_ptr(), fws_bytes)
    _lib.check(lib.nb_attn_fwd(C.byref(fwd), stream), "nb_attn_fwd")

    results = []
    for builtin in (False, True):
        dq, dk, dv = (torch.full_like(q, float("nan")) for _ in range(3))
        if builtin:
            ws, ws_ptr, ws_bytes = None, None, 0  # no workspace is passed at all
        else:
            ws_bytes = _lib.bwd_workspace_bytes(shape)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            ws_ptr = ws.data_ptr()
        args = _lib.BwdArgs(shape, desc(q), desc(k), desc(v), desc(out), desc(g), desc(dq), desc(dk), desc(dv),
                            lse.data_ptr(), ws_ptr, ws_bytes, status.data_ptr(), None, None)
        fn = lib.nb_attn_bwd_builtin_scratch if builtin else lib.nb_attn_bwd
        _lib.check(fn(C.byref(args), stream), fn.__name__)
        torch.cuda.synchronize()
        results.append((dq, dk, dv))
    assert int(status.item()) == 0
    return results


@pytest.mark.gpu
def test_builtin_scratch_matches_caller_workspace_on_two_calls_in_a_row():
    # Two different problems back to back: the second call finds the first one's leftovers in the
    # shared array and must not be affected by them.
    for lengths, heads, seed in ((torch.tensor([300, 129, 64, 1]), 3, 21), (torch.tensor([257, 40]), 2, 22)):
        (dq_a, dk_a, dv_a), (dq_b, dk_b, dv_b) = _backward_both_ways(lengths, heads, seed)
        for name, a, b in (("dq", dq_a, dq_b), ("dk", dk_a, dk_b), ("dv", dv_a, dv_b)):
            assert torch.isfinite(b.float()).all(), name
            err = (a.float() - b.float()).abs()
            # the library-wide bf16 tolerance; the two paths differ only in fp32 summation order
            assert err.max().item() <= 2e-2 and err.mean().item() <= 2e-3, (name, err.max().item())
