"""``ops.sync_batch_norm`` across two ranks (reference: actnn/actnn/ops.py:505-614) against
``torch.nn.SyncBatchNorm`` on the same shards, with UNEQUAL per-rank batch sizes so that the
per-rank counts in the gathered ``[mean, invstd, count]`` message and in the backward matter.

Needs two GPUs that may talk to each other: each rank is a child process on its own device,
NCCL between them (NVLS off), every wait bounded (a process-group timeout of one minute, a
join timeout of three).  It runs only when ``ACTNN_TEST_GPUS`` is set to 2 or more (and that
many devices are visible): on a one-GPU allotment of a larger machine the other devices may
be visible without being usable.  The single-rank path is covered in ``test_batch_norm_gpu.py``.

    ACTNN_TEST_GPUS=2 python -m pytest tests/test_sync_bn_multi_gpu.py -m gpu
"""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, result_dir):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0"})
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import actnn_b200 as actnn
    from actnn_b200.conf import QuantizationConfig

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=60))
    try:
        actnn.config.__dict__.update(QuantizationConfig().__dict__)
        actnn.set_optimization_level("L0")                     # exact activations: only the sync logic differs
        C = 12
        sizes = [5, 3]                                         # unequal shards
        g = torch.Generator().manual_seed(100)
        full_x = torch.randn(sum(sizes), C, 7, 9, generator=g) * 2 + 0.5
        full_gy = torch.randn(sum(sizes), C, 7, 9, generator=g)
        lo = sum(sizes[:rank])
        x = full_x[lo:lo + sizes[rank]].to(dev)
        gy = full_gy[lo:lo + sizes[rank]].to(dev)

        torch.manual_seed(1)
        ref = torch.nn.SyncBatchNorm(C).to(dev)
        with torch.no_grad():
            ref.weight.uniform_(0.5, 1.5)
            ref.bias.uniform_(-1, 1)
        ours = actnn.QSyncBatchNorm(C).to(dev)
        ours.load_state_dict(ref.state_dict())
        ref.train()
        ours.train()
        outs = {}
        for name, mod in (("ref", ref), ("ours", ours)):
            xi = x.clone().requires_grad_(True)
            y = mod(xi)
            y.backward(gy)
            outs[name] = (y.detach(), xi.grad, mod.weight.grad, mod.bias.grad, mod.running_mean.clone(),
                          mod.running_var.clone())
        ok = True
        worst = 0.0
        for a, b in zip(outs["ref"], outs["ours"]):
            err = float((a - b).abs().max()) / max(1.0, float(a.abs().max()))
            worst = max(worst, err)
            ok = ok and err <= 2e-5
        # every rank must end with the same running statistics
        mine = torch.cat([ours.running_mean, ours.running_var])
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        same = all(torch.equal(gathered[0], t) for t in gathered[1:])
        with open(os.path.join(result_dir, "rank%d.txt" % rank), "w") as f:
            f.write("%d %d %.3e\n" % (int(ok), int(same), worst))
    finally:
        dist.destroy_process_group()


def test_sync_batch_norm_two_ranks_unequal_batches(tmp_path):
    if int(os.environ.get("ACTNN_TEST_GPUS", "1")) < 2:
        pytest.skip("set ACTNN_TEST_GPUS=2 on a machine with two usable GPUs")
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = 29600 + os.getpid() % 300
    import time
    ctx = mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=False)
    deadline = time.time() + 180
    done = False
    while not done and time.time() < deadline:           # join() returns as soon as ONE child has ended
        done = ctx.join(timeout=5)
    if not done:
        for proc in ctx.processes:                      # exactly the children started above
            if proc.is_alive():
                proc.kill()
        pytest.fail("the two ranks did not finish within three minutes")
    for rank in range(2):
        ok, same, worst = open(os.path.join(str(tmp_path), "rank%d.txt" % rank)).read().split()
        assert ok == "1", "rank %d differs from torch.nn.SyncBatchNorm (worst relative error %s)" % (rank, worst)
        assert same == "1", "running statistics differ across ranks"
