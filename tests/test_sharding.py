"""CPU tests of the multi-GPU sharding logic: group ranges, zero-copy shard views, and a world-size-2
gloo run in which each rank computes its shard (with the CPU oracle standing in for the device kernels)
and the gathered result equals the unsharded computation."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import util
from hopper_jeni_b200 import sharding


def test_group_range_partitions_everything():
    for n in (1, 7, 8, 32, 33):
        for world in (1, 2, 3, 4, 8):
            ranges = [sharding.group_range(r, world, n) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [e - b for b, e in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.group_range(2, 2, 8)


def test_shards_are_views_and_valid_gqa_problems():
    B, Hq, Hkv, S, D = 2, 6, 2, 16, 8
    q = torch.arange(B * Hq * S * D, dtype=torch.float32).reshape(B, Hq, S, D)
    k = torch.arange(B * Hkv * S * D, dtype=torch.float32).reshape(B, Hkv, S, D)
    qs, ks = sharding.shard(q, Hkv, 1, 2), sharding.shard(k, Hkv, 1, 2)
    assert qs.shape == (2, 3, S, D) and ks.shape == (2, 1, S, D)
    assert qs.data_ptr() == q[1].data_ptr() and ks.data_ptr() == k[1].data_ptr()
    assert qs.is_contiguous() and ks.is_contiguous()
    # group u = b*Hkv + hkv holds query heads hkv*G .. hkv*G+G-1 of batch b
    assert torch.equal(sharding.as_groups(q, Hkv)[3], q[1, 3:6])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, shape, causal, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import gqa_oracle

        B, Hq, Hkv, S, D = shape
        q, k, v, do = (torch.from_numpy(x) for x in util.make_inputs(B, Hq, Hkv, S, D, seed=9, bf16=False))
        sc = util.default_scale(D)

        def bwd(qs, ks, vs, dos):
            return [torch.from_numpy(x) for x in
                    gqa_oracle.backward(qs.numpy(), ks.numpy(), vs.numpy(), dos.numpy(), causal, sc)]

        n_groups = B * Hkv
        res = sharding.run_sharded(bwd, (q, k, v, do), Hkv, rank, world)
        G = Hq // Hkv
        if res is None:
            res = [q.new_zeros((0, G, S, D)), q.new_zeros((0, 1, S, D)), q.new_zeros((0, 1, S, D))]
        full = [sharding.gather_groups(t, n_groups, rank, world) for t in res]
        if rank == 0:
            np.savez(os.path.join(out_dir, "gathered.npz"), dq=full[0].reshape(B, Hq, S, D).numpy(),
                     dk=full[1].reshape(B, Hkv, S, D).numpy(), dv=full[2].reshape(B, Hkv, S, D).numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("shape,world", [((2, 6, 2, 64, 16), 2), ((1, 4, 1, 48, 8), 2), ((1, 6, 3, 32, 8), 2)])
def test_two_rank_gloo_sharded_backward_equals_unsharded(oracle, tmp_path, shape, world):
    causal = True
    mp.spawn(_worker, args=(world, _free_port(), shape, causal, str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / "gathered.npz")
    B, Hq, Hkv, S, D = shape
    q, k, v, do = util.make_inputs(B, Hq, Hkv, S, D, seed=9, bf16=False)
    dq, dk, dv = oracle.backward(q, k, v, do, causal, util.default_scale(D))
    np.testing.assert_array_equal(got["dq"], dq)
    np.testing.assert_array_equal(got["dk"], dk)
    np.testing.assert_array_equal(got["dv"], dv)
