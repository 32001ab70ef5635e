"""Multi-GPU host logic on CPU: shard plans and the gloo all-gather of outputs (world 2)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from shflbw_sparse_nn_b200.sharding import gather_output, shard_plan, shard_range


def test_shard_plan_covers_exactly():
    for total, world, mult in [(4096, 8, 8), (512, 8, 8), (16384, 4, 8), (256, 8, 1), (16, 8, 1), (24, 4, 8), (8, 4, 8)]:
        plan = shard_plan(total, world, mult)
        assert plan[0][0] == 0 and plan[-1][1] == total
        for (b0, e0), (b1, _) in zip(plan, plan[1:]):
            assert e0 == b1
        assert all((e - b) % mult == 0 and e >= b for b, e in plan)
        sizes = [e - b for b, e in plan]
        assert max(sizes) - min(sizes) <= mult
    with pytest.raises(ValueError):
        shard_range(100, 0, 4, 8)
    with pytest.raises(ValueError):
        shard_range(64, 4, 4, 8)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    full = torch.arange(M * N, dtype=torch.float32).reshape(M, N)
    b, e = shard_range(N, rank, world, 8)
    local = full[:, b:e].contiguous()          # this rank's slice of the dense columns
    got = gather_output(local, dim=1)
    assert torch.equal(got, full)
    nb, ne = shard_range(M, rank, world, 1)    # batch sharding: gather along dim 0
    got0 = gather_output(full[nb:ne].contiguous(), dim=0)
    assert torch.equal(got0, full)
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)   # the bench's max-over-ranks timing reduction
    assert t.item() == world
    dist.barrier()
    dist.destroy_process_group()


def test_gather_output_gloo_world2():
    mp.spawn(_worker, args=(2, _free_port(), 16, 64), nprocs=2, join=True)
