"""The N > 1 protocol on CPU: two gloo ranks, no GPU.  Replicas share three scalars, never data."""
import json
import os
import subprocess
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flame_b200 import replicas

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        env = replicas.ReplicaEnv.from_env()
        assert (env.rank, env.world, env.local_rank) == (rank, world, rank)
        replicas.barrier(world)
        ms = [100.0, 125.0][rank]                      # rank 1 is the slower replica
        slowest = replicas.max_over_ranks(ms, world)
        gbs = replicas.aggregate_gbs(10e9 * (rank + 1), world, slowest)
        out[rank] = (replicas.workload_seed(rank), slowest, gbs)
    finally:
        dist.destroy_process_group()


def test_two_replicas_report_the_slowest_time_and_the_summed_bytes():
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, 29541, out), nprocs=world, join=True)
        res = dict(out)
    assert res[0][0] != res[1][0]                      # different data per replica
    for r in range(world):
        assert res[r][1] == 125.0                      # max over ranks
        assert res[r][2] == pytest.approx(30e9 / 0.125 * 1e-9)  # (10 + 20) GB over the slowest time


def test_single_process_needs_no_process_group():
    assert replicas.max_over_ranks(7.0, 1) == 7.0
    assert replicas.aggregate_gbs(5e9, 1, 1000.0) == pytest.approx(5.0)
    replicas.barrier(1)


def test_reference_arm_runs_on_rank_zero_only():
    """`bench.py --impl reference`: ranks other than 0 exit 0 without work or output."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                       env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""


def _plan_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flame_b200.policy import Block, Decision, plan_blocks

        # what a probe run by all replicas at once reports on a box whose replicas share host links unevenly
        d2h, h2d = [(46.6, 55.6), (9.7, 28.8)][rank]
        blocks = [Block(340 << 20, 1.7, 3.7) for _ in range(20)]
        p = plan_blocks(blocks, d2h_gbs=d2h, h2d_gbs=h2d, interference=0.065, overhead_cap_ms=0.04 * 20 * 5.4)
        mine = float(sum(d == Decision.OFFLOAD_INT8 for d in p.decisions))
        everyone = replicas.gather_over_ranks(mine, world)
        est = replicas.max_over_ranks(p.est_stall_ms + p.est_recompute_ms + p.est_interference_ms, world)
        out[rank] = (everyone, est, p.resident_bytes)
    finally:
        dist.destroy_process_group()


def test_each_replica_plans_from_the_link_rate_it_measured():
    """The N > 1 overhead leg: every replica probes, plans under the same cap and the figures are gathered in rank order."""
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_plan_worker, args=(world, 29543, out), nprocs=world, join=True)
        res = dict(out)
    assert res[0][0] == res[1][0] and len(res[0][0]) == 2          # the same gathered list on both ranks
    fast, slow = res[0][0]
    assert fast > slow >= 0                                         # the replica behind the slower link offloads fewer blocks
    assert res[0][1] == res[1][1] <= 0.04 * 20 * 5.4 + 1e-9         # and both stay under the cap
    assert res[1][2] > res[0][2]                                    # keeping more resident instead
