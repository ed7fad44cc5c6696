"""Multi-rank host logic on CPU (gloo, world size 2): batch sharding with no data-path collective
and the 'max over ranks' timing aggregation bench.py uses."""

import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import argparse

    import bench
    from nanobrain_b200 import workloads as W

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        # weak scaling: every rank draws its own batch of the benchmark shape
        args = argparse.Namespace(workload="vitb_encoder_varlen", global_batch=0)
        w, lengths, scaling = bench.rank_lengths(args, rank, world)
        assert scaling == "weak" and lengths.numel() == 32
        # strong scaling: one global batch of 256 sequences sharded B/N per rank
        args = argparse.Namespace(workload="vitb_encoder_varlen", global_batch=256)
        _, shard, scaling = bench.rank_lengths(args, rank, world)
        assert scaling == "strong" and shard.numel() == 128
        flops = W.attention_flops(shard, shard, w.heads)
        # pretend rank 1 was slower; the job time must be the slowest rank's
        stats = torch.tensor([10.0 + 5.0 * rank, 100.0 + rank, float(flops), float(shard.sum())], dtype=torch.float64)
        allstats = bench.gather_over_ranks(stats, world)
        agg = bench.aggregate(allstats, steps=10)
        dist.barrier()
        if rank == 0:
            out.put((agg, [int(x) for x in allstats[:, 3]], [int(x) for x in shard[:3]]))
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_the_batch_and_report_the_slowest_rank():
    from nanobrain_b200 import workloads as W

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    agg, tokens, head = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    full = W.draw_lengths(W.Workload("x", 256, 12, len_lo=720, len_hi=920), seed=0)
    # the two shards partition the global batch: no sequence lost or duplicated
    assert tokens == [int(full[:128].sum()), int(full[128:].sum())]
    assert head == [int(x) for x in full[:3]]
    assert agg["tokens_all"] == int(full.sum())
    assert agg["max_ms"] == 15.0 and agg["max_e2e_ms"] == 101.0
    total_flops = W.attention_flops(full, full, 12)
    assert abs(agg["flops_all"] - total_flops) / total_flops < 1e-12
    assert abs(agg["value_tflops"] - total_flops * 10 / 15e-3 / 1e12) < 1e-6


def test_single_rank_needs_no_process_group():
    import bench

    stats = torch.tensor([2.0, 3.0, 4e9, 100.0], dtype=torch.float64)
    agg = bench.aggregate(bench.gather_over_ranks(stats, 1), steps=4)
    assert agg["max_ms"] == 2.0 and agg["tokens_all"] == 100
    assert abs(agg["value_tflops"] - 4e9 * 4 / 2e-3 / 1e12) < 1e-9


def test_both_bench_arms_describe_the_same_config():
    # the driver compares the `config` objects of the two arms; both come from shapes alone
    import argparse

    import bench
    from nanobrain_b200 import workloads as W

    for gpus in (1, 2, 8):
        args = argparse.Namespace(workload="vitb_encoder_varlen", global_batch=0, gpus=gpus)
        cfg = bench.workload_config(args, W.WORKLOADS[args.workload], gpus)
        assert cfg["global_batch"] == 32 * gpus and cfg["sequences_per_gpu"] == 32
        lengths = [W.draw_lengths(W.WORKLOADS[args.workload], seed=r) for r in range(gpus)]
        assert cfg["tokens_all_ranks"] == sum(int(l.sum()) for l in lengths)
        assert cfg["flops_per_step_all_ranks"] == float(sum(W.attention_flops(l, l, 12) for l in lengths))
    strong = argparse.Namespace(workload="vitb_encoder_varlen", global_batch=256, gpus=8)
    cfg = bench.workload_config(strong, W.WORKLOADS["vitb_encoder_varlen"], 8)
    assert cfg["sequences_per_gpu"] == 32 and cfg["global_batch"] == 256
