"""Forward + backward of packed attention for callers whose tensors live in pinned HOST memory.

The reference stages each step's batch from pinned host memory with non-blocking copies
(``DataLoader(pin_memory=True)`` at ``src/nanobrain/train.py:148-158``, ``send_data`` at
``src/nanobrain/misc.py:449-461``, called at ``train.py:279``). ``HostPipeline`` does the
same for the attention operator alone and hides the copies behind the kernels: the packed batch is
cut into groups of whole sequences (attention never crosses a sequence, so the groups are
independent problems), and three CUDA streams run the groups as a pipeline

    copy-in stream : Q, K, V, dO of group c+1   host -> device
    compute stream : nb_attn_fwd + nb_attn_bwd of group c   (the C ABI, on slices of one device buffer)
    copy-out stream: O, dQ, dK, dV of group c-1  device -> host

so that the two PCIe directions and the GPU work at the same time. All device memory is allocated
once in the constructor; ``run`` allocates nothing and only queues work, ``wait`` makes the caller's
current stream wait for everything queued so far. Successive ``run`` calls overlap as well (the
copy-in of the next step runs under the kernels and the copy-out of the current one); events per
group keep a step from overwriting device buffers the previous step still uses.
"""

from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional, Sequence

import torch
from torch import Tensor

from . import _lib

HEAD_DIM = 64


def split_sequences(lengths: Sequence[int], groups: int) -> List[range]:
    """Cut sequences 0..B-1 into at most ``groups`` runs of consecutive sequences with roughly equal
    token counts (never an empty run)."""
    lengths = [int(x) for x in lengths]
    n = len(lengths)
    groups = max(1, min(int(groups), n))
    total = sum(lengths)
    runs, start, acc = [], 0, 0
    for i, length in enumerate(lengths):
        acc += length
        left = groups - len(runs) - 1          # runs still to open after the current one
        remaining = n - (i + 1)                # sequences after this one
        if left > 0 and remaining >= left and (acc >= total * (len(runs) + 1) / groups or remaining == left):
            runs.append(range(start, i + 1))
            start = i + 1
    runs.append(range(start, n))
    return [r for r in runs if len(r) > 0]


class HostPipeline:
    """Packed self-attention fwd+bwd with pinned host inputs and outputs.

    ``lengths`` are the sequence lengths of the packed batch (host integers: the same knowledge the
    caller needs for ``max_seqlen``), ``heads`` the number of heads; tensors are ``[T, heads, 64]``
    bfloat16 with T = sum(lengths).
    """

    def __init__(self, lengths: Sequence[int], heads: int, device: torch.device, groups: int = 8,
                 scale: Optional[float] = None):
        if torch.device(device).type != "cuda":
            raise RuntimeError("HostPipeline needs a CUDA device: there is no CPU path for the operator")
        self.device = torch.device(device)
        self.heads = int(heads)
        self.lengths = [int(x) for x in lengths]
        if not self.lengths or min(self.lengths) < 0:
            raise ValueError("lengths must be a non-empty list of non-negative integers")
        self.total = sum(self.lengths)
        self.scale = 1.0 / math.sqrt(HEAD_DIM) if scale is None else float(scale)
        self.lib = _lib.load()
        starts = [0]
        for length in self.lengths:
            starts.append(starts[-1] + length)
        shape = (self.total, self.heads, HEAD_DIM)
        with torch.cuda.device(self.device):
            self.dev_in = [torch.empty(shape, dtype=torch.bfloat16, device=self.device) for _ in range(4)]
            self.dev_out = [torch.empty(shape, dtype=torch.bfloat16, device=self.device) for _ in range(4)]
            # Pinned host memory the kernels can write to: readable at any time without a sync.
            self.status = torch.zeros(1, dtype=torch.int32).pin_memory()
            self.s_in, self.s_compute, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self.groups = []
        for run in split_sequences(self.lengths, groups):
            t0, t1 = starts[run.start], starts[run.stop]
            tokens = t1 - t0
            if tokens == 0:
                continue
            lens = self.lengths[run.start:run.stop]
            cu = torch.tensor([s - t0 for s in starts[run.start:run.stop + 1]], dtype=torch.int32, device=self.device)
            sh = _lib.Shape(len(lens), self.heads, HEAD_DIM, max(lens), max(lens), tokens, tokens,
                            cu.data_ptr(), cu.data_ptr(), self.scale)
            ws_bytes, fws_bytes = _lib.bwd_workspace_bytes(sh), _lib.fwd_workspace_bytes(sh)
            with torch.cuda.device(self.device):
                lse = torch.empty((self.heads, tokens), dtype=torch.float32, device=self.device)
                ws = torch.empty(ws_bytes, dtype=torch.uint8, device=self.device)
                fws = torch.empty(fws_bytes, dtype=torch.uint8, device=self.device)
            sl = slice(t0, t1)
            q, k, v, g = (t[sl] for t in self.dev_in)
            o, dq, dk, dv = (t[sl] for t in self.dev_out)
            d = self._desc
            fwd = _lib.FwdArgs(sh, d(q), d(k), d(v), d(o), lse.data_ptr(), self.status.data_ptr(),
                               fws.data_ptr(), fws_bytes)
            bwd = _lib.BwdArgs(sh, d(q), d(k), d(v), d(o), d(g), d(dq), d(dk), d(dv), lse.data_ptr(),
                               ws.data_ptr(), ws_bytes, self.status.data_ptr(), None, None)
            self.groups.append({"slice": sl, "fwd": fwd, "bwd": bwd, "keep": (cu, lse, ws, fws),
                                "ev_in": torch.cuda.Event(), "ev_done": torch.cuda.Event(),
                                "ev_out": torch.cuda.Event()})

    @staticmethod
    def _desc(t: Tensor) -> _lib.Tensor:
        return _lib.Tensor(t.data_ptr(), 0, t.stride(0), t.stride(1))

    @property
    def bytes_per_direction(self) -> int:
        return 4 * self.total * self.heads * HEAD_DIM * 2

    def _check_host(self, tensors: Sequence[Tensor], what: str) -> None:
        for t in tensors:
            if t.device.type != "cpu" or not t.is_pinned():
                raise RuntimeError(f"{what} must be pinned host tensors")
            if t.dtype != torch.bfloat16 or tuple(t.shape) != (self.total, self.heads, HEAD_DIM) or not t.is_contiguous():
                raise RuntimeError(f"{what} must be contiguous bfloat16 [{self.total}, {self.heads}, {HEAD_DIM}]")

    def run(self, q: Tensor, k: Tensor, v: Tensor, d_out: Tensor, out: Tensor, dq: Tensor, dk: Tensor,
            dv: Tensor) -> None:
        """Queue one forward + backward. Inputs ``q, k, v, d_out`` and outputs ``out, dq, dk, dv`` are
        pinned host tensors. The inputs must stay unchanged, and the outputs are not complete, until
        ``wait()`` has been called and the caller's stream has reached that point."""
        self._check_host((q, k, v, d_out), "inputs")
        self._check_host((out, dq, dk, dv), "outputs")
        # What the caller queued before comes first; an earlier run is ordered by the events below.
        self.s_in.wait_stream(torch.cuda.current_stream(self.device))
        host_in, host_out = (q, k, v, d_out), (out, dq, dk, dv)
        sptr = C.c_void_p(self.s_compute.cuda_stream)
        with torch.cuda.device(self.device):
            for grp in self.groups:
                sl = grp["slice"]
                self.s_in.wait_event(grp["ev_done"])      # the previous run has finished with these inputs
                with torch.cuda.stream(self.s_in):
                    for d, h in zip(self.dev_in, host_in):
                        d[sl].copy_(h[sl], non_blocking=True)
                    grp["ev_in"].record(self.s_in)
                self.s_compute.wait_event(grp["ev_in"])
                self.s_compute.wait_event(grp["ev_out"])  # the previous run's results have left the device
                with torch.cuda.stream(self.s_compute):
                    _lib.check(self.lib.nb_attn_fwd(C.byref(grp["fwd"]), sptr), "nb_attn_fwd")
                    _lib.check(self.lib.nb_attn_bwd(C.byref(grp["bwd"]), sptr), "nb_attn_bwd")
                    grp["ev_done"].record(self.s_compute)
                self.s_out.wait_event(grp["ev_done"])
                with torch.cuda.stream(self.s_out):
                    for h, d in zip(host_out, self.dev_out):
                        h[sl].copy_(d[sl], non_blocking=True)
                    grp["ev_out"].record(self.s_out)

    def wait(self) -> None:
        """Make the caller's current stream wait for every run queued so far."""
        main = torch.cuda.current_stream(self.device)
        for s in (self.s_out, self.s_compute, self.s_in):
            main.wait_stream(s)

    def check_status(self) -> None:
        """Synchronise and raise if a kernel reported a timed-out wait."""
        self.wait()
        torch.cuda.synchronize(self.device)
        code = int(self.status[0])
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"attention kernel reported device status {code}: "
                               f"{_lib.STATUS_TEXT.get(code, 'unknown code')}")
