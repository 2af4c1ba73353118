"""Scene sharding helpers on two `gloo` ranks (CPU): partition, global PSH statistics, variable-length gather and
bucketed gradient all-reduce.  The sharded PSH oracle run reproduces the full-batch bucket ids scene by scene when
it is given the global statistics."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash3dtransformer_b200 import parallel, synthetic


def test_shard_scenes_partitions_contiguously():
    for sizes, world in [([10, 10, 10, 10], 2), ([100, 1, 1, 1, 100], 2), ([5], 4), ([7, 3, 9, 1, 4, 6, 2, 8], 4),
                         ([1] * 64, 8)]:
        b = parallel.shard_scenes(sizes, world)
        assert len(b) == world and b[0][0] == 0 and b[-1][1] == len(sizes)
        assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
    assert parallel.shard_scenes([10, 10, 10, 10], 2) == [(0, 2), (2, 4)]
    assert parallel.shard_scenes([200000] * 64, 8) == [(8 * i, 8 * i + 8) for i in range(8)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, sizes):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import psh_oracle as po
        c32, seps = synthetic.batch(synthetic.lidar_scan, sizes, seed=11)
        coords = torch.from_numpy(c32.astype(np.float16))
        seps_t = torch.from_numpy(seps.astype(np.int64))
        local, lseps, (r0, r1), scene0 = parallel.shard_batch(coords, seps_t, rank, world)
        (lo, hi), mean_n = parallel.global_psh_stats(local, lseps)
        assert torch.equal(lo, coords.float().min(0)[0].half()) and torch.equal(hi, coords.float().max(0)[0].half())
        assert abs(mean_n - float(np.mean(sizes))) < 1e-6
        # sharded PSH == the same scenes inside the full batch (bit-exact), given the global statistics
        nb = max(1, po.round_next_two_power(int(mean_n / 256)))
        div = -(-0xFFFF // nb)
        full = po.psh_scatter(coords.numpy(), seps, nb, div, 256, 0xFFFF, lo.numpy(), hi.numpy(), po.probe_table(),
                              coords.shape[0], 0.0, 2)
        mine = po.psh_scatter(local.numpy(), lseps.numpy(), nb, div, 256, 0xFFFF, lo.numpy(), hi.numpy(), po.probe_table(),
                              local.shape[0], 0.0, 2, scene_base=scene0)
        assert np.array_equal(mine["bucket_id"], full["bucket_id"][r0:r1])
        assert np.array_equal(mine["bucket_offs"], full["bucket_offs"][r0:r1])
        assert np.array_equal(mine["scattered_coord"].view(np.uint16), full["scattered_coord"][r0:r1].view(np.uint16))
        # variable-length gather restores the concatenation
        feat = torch.arange(coords.shape[0] * 4, dtype=torch.float32).reshape(-1, 4)
        gathered = parallel.gather_rows(feat[r0:r1])
        assert torch.equal(gathered, feat)
        # bucketed gradient all-reduce averages over ranks, including a parameter that has no gradient on one rank
        torch.manual_seed(0)
        lin = torch.nn.Linear(8, 4)
        extra = torch.nn.Parameter(torch.zeros(3))
        lin.weight.grad = torch.full_like(lin.weight, float(rank + 1))
        lin.bias.grad = torch.full_like(lin.bias, float(10 * (rank + 1)))
        if rank == 0:
            extra.grad = torch.ones(3)
        nb_ = parallel.allreduce_gradients([lin.weight, lin.bias, extra], bucket_bytes=64)
        assert nb_ >= 2
        assert torch.allclose(lin.weight.grad, torch.full_like(lin.weight, 1.5))
        assert torch.allclose(lin.bias.grad, torch.full_like(lin.bias, 15.0))
        assert torch.allclose(extra.grad, torch.full((3,), 0.5))
        # with the global batch known up front the statistics need no read-back and give the same values
        (lo2, hi2), mean2 = parallel.global_psh_stats(local, lseps, total_scenes=len(sizes), total_points=int(sum(sizes)))
        assert torch.equal(lo2, lo) and torch.equal(hi2, hi) and mean2 == mean_n
        # overlapped reduction: buckets issued from gradient hooks during the backward, two micro-batches per step,
        # a parameter that takes part in the loss on one rank only, and the same result as the plain all-reduce
        torch.manual_seed(1)
        net = torch.nn.Sequential(torch.nn.Linear(6, 16), torch.nn.GELU(), torch.nn.Linear(16, 16), torch.nn.GELU(),
                                  torch.nn.Linear(16, 3))
        side = torch.nn.Parameter(torch.ones(3))
        plist = list(net.parameters()) + [side]
        reducer = parallel.GradientBucketReducer(plist, bucket_bytes=256)
        assert len(reducer.buckets) >= 3
        g = torch.Generator().manual_seed(100 + rank)
        xs = [torch.randn(5, 6, generator=g) for _ in range(2)]
        for step in range(2):
            reducer.zero()
            for i, x in enumerate(xs):
                loss = net(x).square().mean() + ((side * (step + 1)).sum() if rank == 0 else 0.0)
                if i == len(xs) - 1:
                    with reducer.reducing():
                        loss.backward()
                else:
                    loss.backward()
            reducer.finish()
            got = [p.grad.clone() for p in plist]
            # the same gradients by plain autograd + all-reduce
            ref_net = [p.detach().clone().requires_grad_(True) for p in plist]
            def fwd(x):
                h = torch.nn.functional.gelu(x @ ref_net[0].t() + ref_net[1])
                h = torch.nn.functional.gelu(h @ ref_net[2].t() + ref_net[3])
                return h @ ref_net[4].t() + ref_net[5]
            for x in xs:
                (fwd(x).square().mean() + ((ref_net[6] * (step + 1)).sum() if rank == 0 else 0.0)).backward()
            for q in ref_net:
                if q.grad is None:
                    q.grad = torch.zeros_like(q)
                dist.all_reduce(q.grad)
                q.grad /= world
            for a, q in zip(got, ref_net):
                assert torch.allclose(a, q.grad, atol=1e-6), step
        reducer.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_gloo_sharding():
    mp.spawn(_worker, args=(2, _free_port(), [3000, 2500, 1800, 2200, 900]), nprocs=2, join=True)
