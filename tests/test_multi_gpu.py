"""Two-GPU test of the in-kernel loss-statistics exchange (peer stores over NVLink): skipped with fewer GPUs."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import importlib

    import torch.distributed as dist

    import __graft_entry__ as entry

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    entry.load_package()
    sharding = importlib.import_module("pcfg_nat_b200.sharding")
    ops = importlib.import_module("pcfg_nat_b200.custom_ops.pcfg_loss")
    ex = sharding.LossExchange(dev)
    ok = True
    for it in range(40):  # both parities of the exchange slots, many epochs
        g = torch.Generator().manual_seed(100 * it)
        B = 7 + it % 5
        losses = [-torch.rand(B, generator=g) * 30 for _ in range(world)]
        lens = [torch.randint(1, 20, (B,), generator=g) for _ in range(world)]
        for r in range(world):
            losses[r][it % B] = float("-inf") if (it + r) % 3 == 0 else losses[r][it % B]
        got = ex.stats(losses[rank].to(dev), lens[rank].to(dev)).cpu()
        want = torch.zeros(3, dtype=torch.float64)
        for r in range(world):
            fin = torch.isfinite(losses[r])
            want[0] += (losses[r][fin].double() / lens[r][fin].double()).sum()
            want[1] += B
            want[2] += (~fin).sum()
        ok = ok and abs(float(got[0]) - float(want[0])) <= 1e-5 * abs(float(want[0])) + 1e-6
        ok = ok and float(got[1]) == float(want[1]) and float(got[2]) == float(want[2])
    ok = ok and ops.read_status(dev) == 0
    out[rank] = ok
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_loss_stats_exchange_two_gpus():
    import torch.multiprocessing as mp

    world = 2
    with mp.Manager() as manager:
        out = manager.dict()
        mp.spawn(_worker, args=(world, 29541, out), nprocs=world, join=True)
        assert all(out.get(r) for r in range(world)), dict(out)
