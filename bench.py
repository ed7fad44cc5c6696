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
# dram__bytes_read.sum + dram__bytes_write.sum of one attn_bwd_kernel launch, from the ncu capture
# summarised in profiles/attn_kernels_vitb_encoder_varlen.md (only known for that workload).
NCU_DRAM_BYTES_BWD_MAIN = {"vitb_encoder_varlen": 364.6e6}


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
    """Whole-job numbers from per-rank rows [elapsed_ms, e2e_ms_per_step, flops_per_step, tokens]:
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
        "config": {"workload": args.workload, "heads": w.heads, "head_dim": 64, "sample": info["sample"]},
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": info["cores"], "kind": "reference",
                         "sample": info["sample"]},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    import nanobrain_b200
    from nanobrain_b200 import _lib, ops
    from nanobrain_b200 import workloads as W

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU path for the operator")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w, lengths, scaling = rank_lengths(args, rank, world)
    heads = w.heads
    total = int(lengths.sum())
    max_len = int(lengths.max())
    nseq = lengths.numel()
    flops_step = W.attention_flops(lengths, lengths, heads)
    cu = W.cu_seqlens_from_lengths(lengths).to(dev)
    host = [t.to(torch.bfloat16).pin_memory() for t in W.make_packed_inputs(lengths, heads, seed=rank)]
    q, k, v, g = (t.to(dev) for t in host)
    out, dq, dk, dv = (torch.empty_like(q) for _ in range(4))
    lse = torch.empty((heads, total), dtype=torch.float32, device=dev)
    lib = _lib.load()
    ws_bytes = lib.nb_attn_bwd_workspace_bytes(total, heads, W.HEAD_DIM)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def desc(t):
        return _lib.Tensor(t.data_ptr(), 0, t.stride(0), t.stride(1))

    shape = _lib.Shape(nseq, heads, W.HEAD_DIM, max_len, max_len, total, total, cu.data_ptr(), cu.data_ptr(), 0.125)
    fwd_args = _lib.FwdArgs(shape, desc(q), desc(k), desc(v), desc(out), lse.data_ptr(), status.data_ptr())

    def bwd_args(ev0=None, ev1=None):
        return _lib.BwdArgs(shape, desc(q), desc(k), desc(v), desc(out), desc(g), desc(dq), desc(dk), desc(dv),
                            lse.data_ptr(), workspace.data_ptr(), ws_bytes, status.data_ptr(), ev0, ev1)

    plain_bwd = bwd_args()
    stream = torch.cuda.current_stream()
    sptr = C.c_void_p(stream.cuda_stream)

    def step(bargs):
        _lib.check(lib.nb_attn_fwd(C.byref(fwd_args), sptr), "nb_attn_fwd")
        _lib.check(lib.nb_attn_bwd(C.byref(bargs), sptr), "nb_attn_bwd")

    # Events around the backward main kernel for the first few timed steps.
    n_probe = min(args.steps, 64)
    probe_events = []
    for _ in range(n_probe):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream), e1.record(stream)  # creates the underlying handles
        probe_events.append((e0, e1, bwd_args(e0.cuda_event, e1.cuda_event)))

    for _ in range(max(args.warmup, 3)):
        step(plain_bwd)
    torch.cuda.synchronize()
    ops_status = int(status.item())
    if ops_status != 0:
        raise RuntimeError(f"kernel reported device status {ops_status}")

    sampler = ClockSampler(local_rank)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    ev_start, ev_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev_start.record(stream)
    for i in range(args.steps):
        step(probe_events[i][2] if i < n_probe else plain_bwd)
    ev_end.record(stream)
    torch.cuda.synchronize()
    sampler.stop()
    if world > 1:
        dist.barrier()
    elapsed_ms = ev_start.elapsed_time(ev_end)
    bwd_main_ms = statistics.mean(e0.elapsed_time(e1) for e0, e1, _ in probe_events)
    if int(status.item()) != 0:
        raise RuntimeError("kernel reported a device status during the timed region")

    # End to end with host buffers: pinned inputs in, pinned results out, through the package's
    # host-buffer entry (nanobrain_b200.HostPipeline: copies and kernels pipelined over groups of
    # sequences, successive steps overlapping like a prefetching input pipeline). Every step moves
    # all four inputs to the device and all four results back.
    e2e_steps = max(1, min(args.e2e_steps, args.steps))
    host_out = [torch.empty_like(host[0]).pin_memory() for _ in range(4)]
    pipe = nanobrain_b200.HostPipeline(lengths.tolist(), heads, dev, groups=args.e2e_groups)

    def e2e_step():
        pipe.run(*host, *host_out)

    for _ in range(2):
        e2e_step()
    pipe.check_status()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    pipe.wait()  # the timed region ends when the last step's results are in host memory
    e1.record(stream)
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    pipe.check_status()
    # The pipelined path must give what the device-resident path gave (same kernels, same inputs).
    if not (torch.equal(host_out[0], out.cpu()) and torch.equal(host_out[2], dk.cpu())):
        raise RuntimeError("host pipeline results differ from the device-resident results")

    # Max over ranks of the device times; sums of the work.
    stats = torch.tensor([elapsed_ms, e2e_ms, float(flops_step), float(total)], dtype=torch.float64, device=dev)
    agg = aggregate(gather_over_ranks(stats, world), args.steps)
    max_ms, max_e2e_ms = agg["max_ms"], agg["max_e2e_ms"]
    flops_all, tokens_all = agg["flops_all"], agg["tokens_all"]

    if rank == 0:
        peaks, peak_kind = load_peaks()
        value, e2e_value = agg["value_tflops"], agg["e2e_tflops"]
        bytes_tensor = total * heads * W.HEAD_DIM * 2
        bwd_flops = W.attention_flops(lengths, lengths, heads, fwd=False, bwd=True)
        achieved = bwd_flops / (bwd_main_ms * 1e-3) / 1e12
        peak = peaks["bf16_tflops"]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": max_ms / args.steps, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": args.workload, "sequences_per_gpu": nseq, "heads": heads, "head_dim": W.HEAD_DIM,
                "tokens_per_gpu_rank0": total, "tokens_all_ranks": tokens_all, "max_seqlen": max_len,
                "flops_per_step_all_ranks": flops_all, "parallelism": f"replicas x{world}, batch-sharded, no collective",
                "l2_policy": "no flush: the step's working set (8 bf16 tensors + fp32 dQ accumulator, "
                             f"{(8 * bytes_tensor + ws_bytes) / 1e6:.0f} MB) exceeds the 126 MB L2",
            },
            "pct_of_measured_bf16_peak": 100.0 * value / (world * peak),
            "pct_of_nominal_bf16_peak": 100.0 * value / (world * NOMINAL_BF16_TFLOPS),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * bytes_tensor,
                    "d2h_bytes_per_step": 4 * bytes_tensor, "steps": e2e_steps, "ms_per_step": max_e2e_ms},
            "gpu_launches": 4 * args.steps,
            "clocks": sampler.summary(),
            "roofline": {
                "kernel": "attn_bwd_kernel", "bound": "tensor", "achieved": achieved, "peak": peak,
                "unit": UNIT, "frac": achieved / peak, "peak_source": f"{peak_kind} bf16_tflops (burst)",
                "ms_per_launch": bwd_main_ms, "launches_timed": n_probe,
                "algorithmic_flops_per_launch": bwd_flops,
                "traffic": NCU_DRAM_BYTES_BWD_MAIN.get(args.workload) if not args.global_batch else None,
                "traffic_unit": "bytes of DRAM traffic per launch (ncu, rank-0 batch shape)",
            },
        }
        if world == 1 and not args.skip_cpu_baseline:
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
