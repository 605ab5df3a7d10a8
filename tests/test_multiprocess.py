"""The N > 1 bookkeeping of the benchmark on CPU: two gloo ranks, no GPU."""
import json
import os
import subprocess
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    import bench
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        local_ms = 10.0 + 5.0 * rank                      # rank 1 is the slow one
        slowest = bench.max_over_ranks(local_ms)
        value = bench.whole_job_gbs(232.8e6, world, slowest)
        # every rank shards by batch: its own generator seed, no data-path collective
        g = torch.Generator().manual_seed(1234 + rank)
        mine = torch.randn(4, generator=g)
        gathered = [torch.empty(4) for _ in range(world)]
        dist.all_gather(gathered, mine)
        out[rank] = (slowest, value, [t.tolist() for t in gathered])
    finally:
        dist.destroy_process_group()


def test_two_ranks_take_the_slowest_time_and_sum_the_work():
    world, port = 2, 29500 + os.getpid() % 2000
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        res = dict(out)
    assert set(res) == {0, 1}
    for rank in (0, 1):
        slowest, value, gathered = res[rank]
        assert slowest == 15.0
        assert value == pytest.approx(2 * 232.8e6 / 15e-3 / 1e9)
        assert gathered[0] != gathered[1]                 # the replicas work on different batches
    assert res[0][2] == res[1][2]


def test_single_process_needs_no_process_group():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.max_over_ranks(3.5) == 3.5
    assert bench.whole_job_gbs(1e9, 4, 1000.0) == pytest.approx(4.0)
    assert bench.algorithmic_bytes(51380224, 2, 2) == pytest.approx(116408320.0)


def test_reference_arm_prints_one_line_on_rank_zero_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "1", "--gpus", "2"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == ""
    env["RANK"] = "0"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "1", "--gpus", "2"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["gpu_launches"] == 0
