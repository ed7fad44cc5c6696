"""Benchmark of the attention hot path: forward + backward TFLOP/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one forward + backward pass of bidirectional attention over one batch of synthetic
packed visible-token sequences (default workload: ViT-B MAE encoder attention, B=32 sequences of
U[720,920] tokens, H=12, head_dim 64, bf16). With N > 1 every rank (one process per GPU, launched
by ``torch.distributed.run``) runs its own batch of the same shape -- replicas, no collective on
the data path -- and the reported value is the aggregate over ranks divided by the slowest
rank's device time. ``--global-batch B`` shards one global batch of B sequences B/N per rank
instead (strong scaling).

Rank 0 prints ONE JSON line. ``value`` is device-resident throughput through the C ABI;
``e2e`` goes through the package's host-buffer entry (``nanobrain_b200.HostPipeline``: H2D of Q, K,
V, dO and D2H of O, dQ, dK, dV inside the timed region, pipelined with the kernels); ``roofline`` times the dominant kernel (backward main) with CUDA
events recorded around it inside the timed region; ``cpu_baseline`` times the reference's own CPU
path (torch CPU SDPA, fp32) on this machine's host cores.
"""

from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import socket
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "attn_fwd_bwd_tflops"
UNIT = "TFLOP/s"
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum of one attn_bwd_kernel launch, from an ncu capture of
# this workload (only known for that workload; not measured by the run itself).
NCU_DRAM_BYTES_BWD_MAIN = {"vitb_encoder_varlen": 600.6e6}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="vitb_encoder_varlen")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="shard one global batch of this many sequences across ranks (strong scaling)")
    ap.add_argument("--e2e-steps", type=int, default=40)
    ap.add_argument("--e2e-groups", type=int, default=8, help="sequence groups of the host-buffer pipeline")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-comparators", action="store_true", help="do not time torch SDPA / flash_attn beside ours")
    ap.add_argument("--skip-other-workloads", action="store_true", help="time the headline workload only")
    ap.add_argument("--skip-e2e", action="store_true", help="no host-buffer pass (for profiler captures)")
    ap.add_argument("--skip-eval", action="store_true", help="do not time the batched varlen eval of the model mirror")
    return ap.parse_args()


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Polls NVML (read-only) for SM clock and throttle reasons while the timed region runs."""

    REASONS = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _poll_once(self):
        nv = self.nv
        self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
        try:
            mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
        except Exception:
            mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
        for bit, name in self.REASONS.items():
            if mask & bit:
                self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                self._poll_once()
            except Exception:
                return
            time.sleep(0.01)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        if self.nv is not None and not self.samples:
            try:
                self._poll_once()
            except Exception:
                pass

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def gather_over_ranks(stats, world: int):
    """All-gather one row of per-rank numbers (a 1-D tensor) -> [world, n] tensor on the CPU.
    Works for NCCL (CUDA tensors) and gloo (CPU tensors); world == 1 needs no process group."""
    import torch
    import torch.distributed as dist

    if world == 1:
        return stats[None].cpu()
    gathered = [torch.zeros_like(stats) for _ in range(world)]
    dist.all_gather(gathered, stats)
    return torch.stack(gathered).cpu()


def aggregate(allstats, steps: int):
    """Whole-job numbers from per-rank rows [elapsed_ms, e2e_ms_per_step, flops_per_step, tokens, ...]:
    time is the MAX over ranks, work is the SUM over ranks."""
    max_ms, max_e2e_ms = float(allstats[:, 0].max()), float(allstats[:, 1].max())
    flops_all, tokens_all = float(allstats[:, 2].sum()), int(allstats[:, 3].sum())
    return {
        "max_ms": max_ms, "max_e2e_ms": max_e2e_ms, "flops_all": flops_all, "tokens_all": tokens_all,
        "value_tflops": flops_all * steps / (max_ms * 1e-3) / 1e12,
        "e2e_tflops": flops_all / (max_e2e_ms * 1e-3) / 1e12,
    }


def rank_lengths(args, rank: int, world: int):
    from nanobrain_b200 import workloads as W

    w = W.WORKLOADS[args.workload]
    if args.global_batch:
        import dataclasses

        lengths = W.draw_lengths(dataclasses.replace(w, batch=args.global_batch), seed=0)
        return w, W.shard_lengths(lengths, rank, world), "strong"
    return w, W.draw_lengths(w, seed=rank), "weak"


def cpu_reference_tflops(lengths, heads, budget_s: float, steps: int = 1, warmup: int = 0):
    """Time the reference's CPU path (torch CPU SDPA fp32 fwd+bwd) on the first n sequences of the
    batch, n chosen so that (steps + warmup) passes fit the budget. Returns (tflops, info)."""
    import torch

    from nanobrain_b200 import workloads as W
    from oracle import reference_cpu as R

    q, k, v, g = W.make_packed_inputs(lengths, heads, seed=0)
    cu = W.cu_seqlens_from_lengths(lengths)
    t_one, l2_one = R.time_packed_sample(q, k, v, g, cu, 1)  # also warms the thread pool
    t_one, l2_one = R.time_packed_sample(q, k, v, g, cu, 1)
    n = int(max(1, min(lengths.numel(), budget_s / max(t_one, 1e-6) / max(1, steps + warmup))))
    for _ in range(warmup):
        R.time_packed_sample(q, k, v, g, cu, n)
    times = []
    for _ in range(steps):
        t, sum_l2 = R.time_packed_sample(q, k, v, g, cu, n)
        times.append(t)
    flops = 14 * heads * W.HEAD_DIM * sum_l2
    total = sum(times)
    info = {
        "cores": torch.get_num_threads(),
        "host_cpus": len(os.sched_getaffinity(0)),
        "sample": f"first {n} of {lengths.numel()} sequences, all {heads} heads, fp32 torch CPU SDPA fwd+bwd, "
                  f"{steps} timed passes",
        "ms_per_step": 1e3 * total / steps,
    }
    return flops * steps / total / 1e12, info


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    import torch

    # torch.distributed.run exports OMP_NUM_THREADS=1; the reference arm uses every host core it may.
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    w, lengths, scaling = rank_lengths(args, 0, 1)
    tflops, info = cpu_reference_tflops(lengths, w.heads, budget_s=150.0, steps=args.steps, warmup=max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": info["ms_per_step"],
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, w, max(1, args.gpus)),
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": info["cores"], "kind": "reference",
                         "sample": info["sample"]},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


class Problem:
    """One workload's device buffers and C-ABI argument blocks for this rank."""

    def __init__(self, w, lengths, dev, seed: int, host=None):
        import torch

        from nanobrain_b200 import _lib
        from nanobrain_b200 import workloads as W

        self.w, self.lengths, self.dev = w, lengths, dev
        self.heads = w.heads
        self.total = int(lengths.sum())
        self.nseq = lengths.numel()
        self.max_len = int(lengths.max())
        self.flops = W.attention_flops(lengths, lengths, w.heads)
        self.bwd_flops = W.attention_flops(lengths, lengths, w.heads, fwd=False, bwd=True)
        self.lib = _lib.load()
        if w.varlen:
            self.cu = W.cu_seqlens_from_lengths(lengths).to(dev)
            if host is None:
                g = torch.Generator(device=dev).manual_seed(seed)
                self.inputs = [torch.randn(self.total, w.heads, W.HEAD_DIM, generator=g, device=dev).to(torch.bfloat16)
                               for _ in range(4)]
            else:
                self.inputs = [t.to(dev) for t in host]
            cu_ptr = self.cu.data_ptr()
            self.lse = torch.empty((w.heads, self.total), dtype=torch.float32, device=dev)
            desc = lambda t: _lib.Tensor(t.data_ptr(), 0, t.stride(0), t.stride(1))
        else:
            g = torch.Generator(device=dev).manual_seed(seed)
            # [B, L, H, 64] memory, the layout the reference's Linear + view produce (modules.py:59-61)
            self.inputs = [torch.randn(w.batch, w.seqlen, w.heads, W.HEAD_DIM, generator=g, device=dev).to(torch.bfloat16)
                           for _ in range(4)]
            cu_ptr = None
            self.lse = torch.empty((w.batch, w.heads, w.seqlen), dtype=torch.float32, device=dev)
            desc = lambda t: _lib.Tensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))
        self.q, self.k, self.v, self.g = self.inputs
        self.out, self.dq, self.dk, self.dv = (torch.empty_like(self.q) for _ in range(4))
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.shape = _lib.Shape(self.nseq, w.heads, W.HEAD_DIM, self.max_len, self.max_len, self.total, self.total,
                                cu_ptr, cu_ptr, 0.125)
        self.ws_bytes, fws_bytes = _lib.bwd_workspace_bytes(self.shape), _lib.fwd_workspace_bytes(self.shape)
        self.workspace = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        self.fwd_workspace = torch.empty(max(fws_bytes, 16), dtype=torch.uint8, device=dev)
        self.desc = desc
        self.fwd_args = _lib.FwdArgs(self.shape, desc(self.q), desc(self.k), desc(self.v), desc(self.out),
                                     self.lse.data_ptr(), self.status.data_ptr(), self.fwd_workspace.data_ptr(), fws_bytes)
        self.plain_bwd = self.bwd_args()
        # kernels per step: work list (packed mode), forward, row-dot prologue (+ list), backward main, dQ epilogue
        self.launches_per_step = 5 if w.varlen else 4

    def bwd_args(self, ev0=None, ev1=None):
        from nanobrain_b200 import _lib

        d = self.desc
        return _lib.BwdArgs(self.shape, d(self.q), d(self.k), d(self.v), d(self.out), d(self.g), d(self.dq), d(self.dk),
                            d(self.dv), self.lse.data_ptr(), self.workspace.data_ptr(), self.ws_bytes,
                            self.status.data_ptr(), ev0, ev1)

    def step(self, sptr, bargs=None):
        from nanobrain_b200 import _lib

        _lib.check(self.lib.nb_attn_fwd(C.byref(self.fwd_args), sptr), "nb_attn_fwd")
        _lib.check(self.lib.nb_attn_bwd(C.byref(bargs if bargs is not None else self.plain_bwd), sptr), "nb_attn_bwd")

    def check_status(self):
        code = int(self.status.item())
        if code != 0:
            raise RuntimeError(f"kernel reported device status {code}")

    @property
    def working_set_bytes(self):
        return 8 * self.q.numel() * 2 + self.ws_bytes


PROBE_EVERY = 16


def time_problem(prob, steps: int, warmup: int, stream, sync_ranks=None):
    """W warm-up steps, then exactly `steps` timed steps between two CUDA events on `stream`.
    Every PROBE_EVERY-th step also records events around the backward main kernel (the events sit
    between kernels, where they switch off the programmatic overlap of that step's prologue / main /
    epilogue boundaries, so the other steps run without them). Returns (elapsed_ms, bwd_main_ms)."""
    import torch

    sptr = C.c_void_p(stream.cuda_stream)
    probes = []
    for _ in range((steps + PROBE_EVERY - 1) // PROBE_EVERY):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream), e1.record(stream)  # creates the underlying handles
        probes.append((e0, e1, prob.bwd_args(e0.cuda_event, e1.cuda_event)))
    for _ in range(max(warmup, 3)):
        prob.step(sptr)
    torch.cuda.synchronize()
    prob.check_status()
    if sync_ranks is not None:
        sync_ranks()
    torch.cuda.synchronize()
    ev_start, ev_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev_start.record(stream)
    for i in range(steps):
        prob.step(sptr, probes[i // PROBE_EVERY][2] if i % PROBE_EVERY == 0 else None)
    ev_end.record(stream)
    torch.cuda.synchronize()
    if sync_ranks is not None:
        sync_ranks()
    prob.check_status()
    return ev_start.elapsed_time(ev_end), statistics.mean(e0.elapsed_time(e1) for e0, e1, _ in probes)


def time_callable(fn, steps: int, warmup: int):
    """Median-free plain timing of a callable that launches on the current stream: ms per call."""
    import torch

    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def gpu_comparators(prob_varlen, prob_dense, steps: int):
    """What the reference would get on this GPU by doing nothing: torch's own bf16
    F.scaled_dot_product_attention (forward + backward) on the same device inputs -- the dense decoder
    workload directly, the packed encoder workload as the per-sequence loop of the reference's eval
    path (src/nanobrain/model.py:254-270) and as one zero-padded dense call -- and flash_attn's
    varlen kernel if it imports. Reported only: nothing in the product depends on them."""
    import torch
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    out = {}
    backends = [("cudnn", SDPBackend.CUDNN_ATTENTION), ("flash", SDPBackend.FLASH_ATTENTION),
                ("efficient", SDPBackend.EFFICIENT_ATTENTION)]

    def best_backend(make_call, flops):
        res, errors = None, {}
        for name, be in backends:
            try:
                with sdpa_kernel([be]):
                    ms = time_callable(make_call, steps, 3)
                if res is None or ms < res["ms_per_step"]:
                    res = {"backend": name, "ms_per_step": ms, "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT}
            except Exception as exc:  # a backend that refuses the shape / dtype on this GPU
                errors[name] = type(exc).__name__
        if res is None:
            return {"unavailable": errors}
        if errors:
            res["backends_refused"] = errors
        return res

    if prob_dense is not None:
        q, k, v, g = (t.transpose(1, 2).detach().requires_grad_(True) if i < 3 else t.transpose(1, 2)
                      for i, t in enumerate(prob_dense.inputs))

        def dense_call():
            o = F.scaled_dot_product_attention(q, k, v, is_causal=False)
            o.backward(g)
            q.grad = k.grad = v.grad = None

        out["torch_sdpa_" + prob_dense.w.name] = best_backend(dense_call, prob_dense.flops)

    p = prob_varlen
    cu = p.cu.cpu().tolist()
    seqs = []
    for i in range(p.nseq):
        a, b = cu[i], cu[i + 1]
        seqs.append(tuple((t[a:b].transpose(0, 1)[None].detach().requires_grad_(i_t < 3))
                          for i_t, t in enumerate(p.inputs)))

    def loop_call():
        for q, k, v, g in seqs:
            o = F.scaled_dot_product_attention(q, k, v, is_causal=False)
            o.backward(g)
            q.grad = k.grad = v.grad = None

    out["torch_sdpa_per_sequence_loop_" + p.w.name] = best_backend(loop_call, p.flops)

    pad = torch.zeros(p.nseq, p.heads, p.max_len, 64, dtype=torch.bfloat16, device=p.dev)
    padded = []
    for i_t, t in enumerate(p.inputs):
        x = pad.clone()
        for i in range(p.nseq):
            x[i, :, :cu[i + 1] - cu[i]] = t[cu[i]:cu[i + 1]].transpose(0, 1)
        padded.append(x.requires_grad_(i_t < 3))

    def padded_call():
        o = F.scaled_dot_product_attention(padded[0], padded[1], padded[2], is_causal=False)
        o.backward(padded[3])
        padded[0].grad = padded[1].grad = padded[2].grad = None

    res = best_backend(padded_call, p.flops)
    if "unavailable" not in res:
        res["note"] = "zero-padded to max_seqlen without a mask (padding keys take part: a timing yardstick, not the same result)"
    out["torch_sdpa_padded_dense_" + p.w.name] = res

    try:
        from flash_attn import flash_attn_varlen_func

        q, k, v = (t.detach().requires_grad_(True) for t in p.inputs[:3])

        def fa_call():
            o = flash_attn_varlen_func(q, k, v, p.cu, p.cu, p.max_len, p.max_len, causal=False)
            o.backward(p.g)
            q.grad = k.grad = v.grad = None

        ms = time_callable(fa_call, steps, 3)
        out["flash_attn_varlen_" + p.w.name] = {"ms_per_step": ms, "value": p.flops / (ms * 1e-3) / 1e12, "unit": UNIT}
    except Exception as exc:
        out["flash_attn_varlen_" + p.w.name] = {"unavailable": type(exc).__name__ + ": " + str(exc)[:120]}
    return out


def batched_eval_images_per_s(dev, repeats: int = 3):
    """Embeddings of ragged images with the ViT-B encoder mirror (random weights): all images packed
    into one varlen pass (`ViTMAE3D.embed_packed`) against one encoder forward per image, the way the
    reference's `forward_embeddings` does it (src/nanobrain/model.py:254-276). In-mask patch counts as
    different as real brain masks are; 128^3 volumes, 8^3 patches (4096-patch grid)."""
    import torch

    from nanobrain_b200 import model as M

    counts = [3200, 2900, 3475, 1, 3050, 2600, 3300, 2750]
    torch.manual_seed(0)
    model = M.ViTMAE3D(grid_size=(128, 128, 128), patch_size=8).to(dev).eval()
    samples = []
    for i, n in enumerate(counts):
        g = torch.Generator(device=dev).manual_seed(i)
        patches = torch.randn(4096, 512, generator=g, device=dev)
        in_mask = torch.zeros(4096, dtype=torch.bool, device=dev)
        in_mask[torch.randperm(4096, generator=g, device=dev)[:n]] = True
        samples.append((patches, in_mask))

    def packed():
        return model.embed_packed(samples)

    def per_image():
        outs = []
        with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
            for patches, in_mask in samples:
                tokens = model.forward_encoder(patches[None, in_mask], model.coord_grid[:, in_mask])
                outs.append(tokens[0, model.class_tokens:].float().mean(dim=0))
        return outs

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(repeats):
            out = fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / repeats, out

    t_packed, a = timed(packed)
    t_loop, b = timed(per_image)
    worst = max(float((x["global_embedding"] - y).abs().max() / y.abs().max().clamp_min(1e-6)) for x, y in zip(a, b))
    return {
        "images": len(counts), "in_mask_patches": counts, "model": "ViT-B encoder mirror, depth 12, 768 wide, random weights",
        "packed_images_per_s": len(counts) / t_packed, "per_image_loop_images_per_s": len(counts) / t_loop,
        "max_rel_diff_of_embeddings": worst,
        "note": "wall clock of the whole encoder (Linears, LayerNorms, attention); the per-image loop uses the same dense operator",
    }


def copy_only_ms(host, host_out, dev, steps: int):
    """The host-buffer path's ceiling: the same pinned H2D + D2H traffic with no kernels at all, the
    two directions on their own streams."""
    import torch

    dev_bufs = [torch.empty_like(t, device=dev) for t in host]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def once():
        with torch.cuda.stream(s_in):
            for d, h in zip(dev_bufs, host):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s_out):
            for h, d in zip(host_out, dev_bufs):
                h.copy_(d, non_blocking=True)

    for _ in range(2):
        once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cur = torch.cuda.current_stream()
    e0.record(cur)
    s_in.wait_stream(cur), s_out.wait_stream(cur)
    for _ in range(steps):
        once()
    cur.wait_stream(s_in), cur.wait_stream(s_out)
    e1.record(cur)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def workload_config(args, w, world: int):
    """The `config` object, computed from shapes alone so that both arms print the same one."""
    from nanobrain_b200 import workloads as W

    per_rank = [rank_lengths(args, r, world)[1] for r in range(world)]
    tokens_all = sum(int(l.sum()) for l in per_rank)
    flops_all = sum(W.attention_flops(l, l, w.heads) for l in per_rank)
    t0 = int(per_rank[0].sum())
    working_set = 8 * t0 * w.heads * 64 * 2 + t0 * w.heads * 64 * 4
    return {
        "workload": args.workload, "sequences_per_gpu": per_rank[0].numel(), "heads": w.heads, "head_dim": 64,
        "tokens_per_gpu_rank0": t0, "max_seqlen": int(per_rank[0].max()),
        "global_batch": args.global_batch or per_rank[0].numel() * world,
        "tokens_all_ranks": tokens_all, "flops_per_step_all_ranks": float(flops_all),
        "parallelism": f"replicas x{world}, batch-sharded, no collective",
        "l2_policy": "no flush: the step's working set (8 bf16 tensors + fp32 dQ accumulator, "
                     f"{working_set / 1e6:.0f} MB on rank 0) exceeds the 126 MB L2",
    }


def run_ours(args, rank: int, world: int, local_rank: int):
    import dataclasses

    import torch
    import torch.distributed as dist

    import nanobrain_b200
    from nanobrain_b200 import workloads as W

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU path for the operator")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    barrier = dist.barrier if world > 1 else None
    stream = torch.cuda.current_stream()

    sampler = ClockSampler(local_rank)
    sampler.start()  # before warm-up: the timed region of the headline is a few milliseconds long

    w, lengths, scaling = rank_lengths(args, rank, world)
    heads = w.heads
    host = [t.to(torch.bfloat16).pin_memory() for t in W.make_packed_inputs(lengths, heads, seed=rank)] if w.varlen else None
    prob = Problem(w, lengths, dev, seed=rank, host=host)
    elapsed_ms, bwd_main_ms = time_problem(prob, args.steps, args.warmup, stream, barrier)

    # End to end with host buffers: pinned inputs in, pinned results out, through the package's
    # host-buffer entry (nanobrain_b200.HostPipeline: copies and kernels pipelined over groups of
    # sequences, successive steps overlapping like a prefetching input pipeline). Every step moves
    # all four inputs to the device and all four results back.
    e2e_ms, copy_ms = float("nan"), float("nan")
    e2e_steps = max(1, min(args.e2e_steps, args.steps))
    if w.varlen and not args.skip_e2e:
        host_out = [torch.empty_like(host[0]).pin_memory() for _ in range(4)]
        pipe = nanobrain_b200.HostPipeline(lengths.tolist(), heads, dev, groups=args.e2e_groups)
        for _ in range(2):
            pipe.run(*host, *host_out)
        pipe.check_status()
        if barrier:
            barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            pipe.run(*host, *host_out)
        pipe.wait()  # the timed region ends when the last step's results are in host memory
        e1.record(stream)
        torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps
        pipe.check_status()
        # The pipelined path must give what the device-resident path gave (same kernels, same inputs).
        if not (torch.equal(host_out[0], prob.out.cpu()) and torch.equal(host_out[2], prob.dk.cpu())):
            raise RuntimeError("host pipeline results differ from the device-resident results")
        # The same traffic with no kernels, all ranks at once: what the host and PCIe allow.
        if barrier:
            barrier()
        copy_ms = copy_only_ms(host, host_out, dev, e2e_steps)
    sampler.stop()

    # BASELINE config 4 next to the weak-scaling headline: ONE global batch of 256 sequences drawn
    # with seed 0 and sharded B/N per rank (no collective), timed the same way.
    strong = None
    if w.varlen and not args.global_batch and args.workload == "vitb_encoder_varlen" and not args.skip_other_workloads:
        glob = W.draw_lengths(dataclasses.replace(w, batch=256), seed=0)
        mine = W.shard_lengths(glob, rank, world)
        sprob = Problem(w, mine, dev, seed=1000 + rank)
        s_steps = max(4, args.steps // max(1, 8 // world))  # a rank's share shrinks with N: similar wall time
        s_ms, _ = time_problem(sprob, s_steps, 3, stream, barrier)
        strong = (s_ms, s_steps, float(sprob.flops), float(sprob.total))
        del sprob

    # Max over ranks of the device times; sums of the work.
    row = [elapsed_ms, e2e_ms, float(prob.flops), float(prob.total), copy_ms]
    row += list(strong) if strong else [0.0, 0.0, 0.0, 0.0]
    allstats = gather_over_ranks(torch.tensor(row, dtype=torch.float64, device=dev), world)
    agg = aggregate(allstats, args.steps)

    if rank == 0:
        peaks, peak_kind = load_peaks()
        peak = peaks["bf16_tflops"]
        value = agg["value_tflops"]
        bytes_tensor = prob.q.numel() * 2
        achieved = prob.bwd_flops / (bwd_main_ms * 1e-3) / 1e12
        config = workload_config(args, w, world)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": agg["max_ms"] / args.steps, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
            "pct_of_measured_bf16_peak": 100.0 * value / (world * peak),
            "pct_of_nominal_bf16_peak": 100.0 * value / (world * NOMINAL_BF16_TFLOPS),
            "gpu_launches": prob.launches_per_step * args.steps,
            "clocks": sampler.summary(),
            "roofline": {
                "kernel": "attn_bwd_kernel", "bound": "tensor", "achieved": achieved, "peak": peak,
                "unit": UNIT, "frac": achieved / peak, "peak_source": f"{peak_kind} bf16_tflops (burst)",
                "ms_per_launch": bwd_main_ms, "launches_timed": (args.steps + PROBE_EVERY - 1) // PROBE_EVERY,
                "algorithmic_flops_per_launch": prob.bwd_flops,
                "traffic": NCU_DRAM_BYTES_BWD_MAIN.get(args.workload) if not args.global_batch else None,
                "traffic_unit": "bytes of DRAM traffic per launch (one ncu capture of this workload on rank 0's batch shape)",
            },
        }
        if w.varlen and not args.skip_e2e:
            line["e2e"] = {"value": agg["e2e_tflops"], "unit": UNIT, "h2d_bytes_per_step": 4 * bytes_tensor,
                           "d2h_bytes_per_step": 4 * bytes_tensor, "steps": e2e_steps, "ms_per_step": agg["max_e2e_ms"],
                           "copy_only_ms": float(allstats[:, 4].max()),
                           "copy_only_note": "the same pinned H2D + D2H bytes with no kernels, all ranks at once (max over ranks)"}
        if strong:
            s_max_ms, s_steps = float(allstats[:, 5].max()), int(allstats[0, 6])
            s_flops = float(allstats[:, 7].sum())
            line["config4_strong"] = {
                "workload": "vitb_encoder_varlen, global batch 256 (seed 0) sharded B/N per GPU, no collective",
                "global_batch": 256, "sequences_per_gpu": 256 // world, "n_gpus": world, "scaling": "strong",
                "steps": s_steps, "ms_per_step": s_max_ms / s_steps, "tokens_all_ranks": int(allstats[:, 8].sum()),
                "value": s_flops * s_steps / (s_max_ms * 1e-3) / 1e12, "unit": UNIT,
            }
        if world == 1 and not args.skip_other_workloads:
            other = {}
            for name in ("mae_decoder_dense", "vitl_encoder_varlen"):
                if name == args.workload:
                    continue
                ow = W.WORKLOADS[name]
                oprob = Problem(ow, W.draw_lengths(ow, seed=0), dev, seed=0)
                o_steps = max(4, min(args.steps, 20))
                o_ms, o_main = time_problem(oprob, o_steps, 3, stream)
                other[name] = {
                    "value": oprob.flops * o_steps / (o_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": o_ms / o_steps,
                    "steps": o_steps, "description": ow.description,
                    "pct_of_measured_bf16_peak": 100.0 * oprob.flops * o_steps / (o_ms * 1e-3) / 1e12 / peak,
                    "roofline_bwd_main": {"ms_per_launch": o_main, "achieved": oprob.bwd_flops / (o_main * 1e-3) / 1e12,
                                          "frac": oprob.bwd_flops / (o_main * 1e-3) / 1e12 / peak, "unit": UNIT},
                }
                if name == "mae_decoder_dense" and not args.skip_comparators:
                    line["gpu_comparators"] = gpu_comparators(prob, oprob, steps=5)
                del oprob
                torch.cuda.empty_cache()
            line["other_workloads"] = other
        if world == 1 and not args.skip_eval and not args.skip_other_workloads:
            line["batched_eval"] = batched_eval_images_per_s(dev)
        if world == 1:
            if not args.skip_cpu_baseline:
                torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
                tf, info = cpu_reference_tflops(lengths, heads, budget_s=20.0, steps=3, warmup=1)
                line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": info["cores"], "kind": "reference",
                                        "sample": info["sample"], "host_cpus": info["host_cpus"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and "RANK" not in os.environ:
        # Convenience: re-launch under torch.distributed.run, one process per GPU.
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()), str(Path(__file__).resolve()),
               *sys.argv[1:]]
        sys.exit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
