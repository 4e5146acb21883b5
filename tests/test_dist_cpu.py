"""world_size-2 gloo test of the data-parallel gradient reduction (host logic, CPU only)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    from v1_glif_model_b200.training import FlatGradients
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fg = FlatGradients([4, 3, 2], "cpu")
        g = torch.Generator().manual_seed(100 + rank)
        for v in fg.views:
            v.copy_(torch.randn(v.numel(), generator=g))
        local = fg.flat.clone()
        fg.all_reduce()
        gathered = [torch.zeros_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        expect = sum(gathered)
        ok = torch.allclose(fg.flat, expect, rtol=1e-6, atol=0) and \
            torch.equal(fg.views[1], fg.flat[4:7])
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_flat_gradient_allreduce_two_ranks():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}
