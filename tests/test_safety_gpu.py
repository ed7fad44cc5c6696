"""What the kernels must NOT do, checked through the C ABI on a GPU: write outside the rows and
columns they own (sentinel-filled buffers with a wide row pitch), let one packed sequence's
Inf / NaN leak into its neighbour, or hang when a wait cannot complete."""

import ctypes as C

import pytest
import torch

import nanobrain_b200
from nanobrain_b200 import _lib, ops, schedule
from nanobrain_b200 import workloads as W

pytestmark = pytest.mark.gpu
DEV = "cuda"
SENTINEL = -12345.0   # buffers are compared with the same value rounded to their own dtype


class Padded:
    """A [rows, heads, 64] bf16 view inside a larger sentinel-filled buffer: spare rows before and
    after, and a row pitch of heads*64 + 64 elements (a gap after every token row)."""

    def __init__(self, rows, heads, fill=None):
        self.rows, self.heads = rows, heads
        self.pitch = heads * 64 + 64
        self.buf = torch.full((rows + 16, self.pitch), SENTINEL, dtype=torch.bfloat16, device=DEV)
        self.view = self.buf[8:8 + rows, :heads * 64].view(rows, heads, 64)
        if fill is not None:
            self.view.copy_(fill)

    def desc(self):
        return _lib.Tensor(self.view.data_ptr(), 0, self.pitch, 64)

    def sentinels_intact(self):
        s = torch.tensor(SENTINEL, dtype=torch.bfloat16, device=DEV)
        return bool((self.buf[:8] == s).all() and (self.buf[8 + self.rows:] == s).all()
                    and (self.buf[:, self.heads * 64:] == s).all())


def fwd_bwd_in_padded_buffers(lengths, heads, dense_len=None):
    lib = _lib.load()
    if dense_len is None:
        total, nseq, max_len = int(lengths.sum()), lengths.numel(), int(lengths.max())
        cu = W.cu_seqlens_from_lengths(lengths).to(DEV)
        cu_ptr = cu.data_ptr()
    else:
        nseq, max_len = 1, dense_len
        total, cu_ptr = dense_len, None
    g = torch.Generator().manual_seed(total)
    q, k, v, d_o = (Padded(total, heads, torch.randn(total, heads, 64, generator=g).to(DEV, torch.bfloat16))
                    for _ in range(4))
    o, dq, dk, dv = (Padded(total, heads) for _ in range(4))
    # LSE is contiguous ([heads][total] packed, [1][heads][L] dense): an exact-size block in a sentinel frame
    lse_frame = torch.full((heads * total + 64,), SENTINEL, dtype=torch.float32, device=DEV)
    lse = lse_frame[32:32 + heads * total]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    shape = _lib.Shape(nseq, heads, 64, max_len, max_len, total, total, cu_ptr, cu_ptr, 0.125)
    fws_bytes, ws_bytes = _lib.fwd_workspace_bytes(shape), _lib.bwd_workspace_bytes(shape)
    fws = torch.empty(max(fws_bytes, 256), dtype=torch.uint8, device=DEV)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
    sb = total * (heads * 64 + 64)   # batch stride of the single dense sequence (unused beyond batch 0)

    def d(t):
        x = t.desc()
        x.stride_batch = sb
        return x

    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    fwd = _lib.FwdArgs(shape, d(q), d(k), d(v), d(o), lse.data_ptr(), status.data_ptr(), fws.data_ptr(), fws_bytes)
    _lib.check(lib.nb_attn_fwd(C.byref(fwd), stream), "nb_attn_fwd")
    bwd = _lib.BwdArgs(shape, d(q), d(k), d(v), d(o), d(d_o), d(dq), d(dk), d(dv), lse.data_ptr(), ws.data_ptr(),
                       ws_bytes, status.data_ptr(), None, None)
    _lib.check(lib.nb_attn_bwd(C.byref(bwd), stream), "nb_attn_bwd")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return (q, k, v, d_o), (o, dq, dk, dv), lse_frame, lse


@pytest.mark.parametrize("lengths", [[70, 129], [128, 1, 300, 52], [820]])
def test_varlen_kernels_write_only_their_own_rows_and_columns(lengths):
    lengths = torch.tensor(lengths)
    ins, outs, lse_frame, lse = fwd_bwd_in_padded_buffers(lengths, heads=3)
    for t in ins + outs:
        assert t.sentinels_intact()
    for t in outs:
        assert torch.isfinite(t.view.float()).all()                    # every owned element was written
    assert bool((lse_frame[:32] == SENTINEL).all() and (lse_frame[32 + lse.numel():] == SENTINEL).all())
    assert torch.isfinite(lse).all()
    # the same numbers as the op computes in ordinary contiguous tensors
    cu = W.cu_seqlens_from_lengths(lengths).to(DEV)
    q, k, v = (t.view.clone().requires_grad_(True) for t in ins[:3])
    out = nanobrain_b200.sdpa_varlen(q, k, v, cu, cu, int(lengths.max()), int(lengths.max()))
    out.backward(ins[3].view.clone())
    ops.check_status()
    assert torch.equal(out, outs[0].view) and torch.equal(k.grad, outs[2].view) and torch.equal(v.grad, outs[3].view)
    assert (q.grad.float() - outs[1].view.float()).abs().max() <= 2e-2


@pytest.mark.parametrize("length", [52, 130, 257])
def test_dense_kernels_write_only_their_own_rows_and_columns(length):
    ins, outs, lse_frame, lse = fwd_bwd_in_padded_buffers(None, heads=2, dense_len=length)
    for t in ins + outs:
        assert t.sentinels_intact()
    for t in outs:
        assert torch.isfinite(t.view.float()).all()
    assert bool((lse_frame[:32] == SENTINEL).all() and (lse_frame[32 + lse.numel():] == SENTINEL).all())


@pytest.mark.parametrize("poison", [float("inf"), float("nan")])
def test_forward_keeps_a_poisoned_sequence_away_from_its_neighbours(poison):
    # The reference runs one SDPA per sequence, so sequences are isolated. Packed, a ragged tile
    # brings rows of the next sequence into shared memory; the forward kernel clears them, so they
    # cannot reach this sequence's output even as 0 x Inf. (The backward kernels do not clear them:
    # there, non-finite values in the first rows of a sequence also turn the gradients of the
    # sequence before it into NaN. Finite data is unaffected either way.)
    lengths = torch.tensor([70, 129, 33, 200])
    cu = W.cu_seqlens_from_lengths(lengths).to(DEV)
    heads, total = 2, int(lengths.sum())
    g = torch.Generator().manual_seed(3)
    base = [torch.randn(total, heads, 64, generator=g).to(DEV, torch.bfloat16) for _ in range(3)]
    clean_out, clean_lse = ops.sdpa_varlen_fwd(*base, cu, cu, 200, 200, 0.125)
    a, b = int(cu[2]), int(cu[3])          # poison all of sequence 2 (33 tokens, inside its neighbours' tiles)
    keep = torch.ones(total, dtype=torch.bool, device=DEV)
    keep[a:b] = False
    for which in range(3):                 # Q, K, V in turn
        dirty = [t.clone() for t in base]
        dirty[which][a:b] = poison
        out, lse = ops.sdpa_varlen_fwd(*dirty, cu, cu, 200, 200, 0.125)
        ops.check_status()
        assert torch.isfinite(out[keep].float()).all() and torch.isfinite(lse[:, keep]).all(), "qkv"[which]
        assert torch.equal(out[keep], clean_out[keep]) and torch.equal(lse[:, keep], clean_lse[:, keep])


def test_a_wait_that_cannot_complete_gives_up_and_frees_tensor_memory():
    # One CTA waits 2 ms for a barrier nobody arrives on: the kernel returns, reports the time-out,
    # and has freed its tensor memory (it held all 512 columns: the attention call right after
    # would otherwise never get any).
    code, out = schedule.selftest_wait(2_000_000, torch.device(DEV))
    assert code == _lib.STATUS_WAIT_TIMEOUT and out.tolist() == [1, 1]
    lengths = torch.tensor([150, 129, 64])
    cu = W.cu_seqlens_from_lengths(lengths).to(DEV)
    t = torch.randn(int(lengths.sum()), 2, 64, device=DEV).to(torch.bfloat16).requires_grad_(True)
    out = nanobrain_b200.sdpa_varlen(t, t, t, cu, cu, 150, 150)
    out.float().sum().backward()
    ops.check_status()
    assert torch.isfinite(out.float()).all() and torch.isfinite(t.grad.float()).all()


def test_a_reported_status_surfaces_at_the_next_call_without_a_sync():
    word = ops._status_word(torch.device(DEV, torch.cuda.current_device()))
    word[0] = _lib.STATUS_WAIT_TIMEOUT      # what a kernel would have written
    t = torch.randn(64, 2, 64, device=DEV).to(torch.bfloat16)
    cu = torch.tensor([0, 64], dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="bounded wait"):
        nanobrain_b200.sdpa_varlen(t, t, t, cu, cu, 64, 64)
    nanobrain_b200.sdpa_varlen(t, t, t, cu, cu, 64, 64)   # cleared by the raise
    ops.check_status()
