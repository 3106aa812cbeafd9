"""The N > 1 host logic on CPU: two gloo ranks split each operator the way `rocmlir_b200.sharding` prescribes,
compute their share with the oracle, and the recombined result must equal the unsplit oracle result
(bit-exact: integer-valued data, so the order of the cross-rank sum cannot matter)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from rocmlir_b200 import sharding


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _int_data(shape, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(-5, 5, size=shape).astype(np.float32)


def _worker(rank: int, world: int, port: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        out = {}
        # --- GEMM, column split + gather ---
        G, M, N, K = 2, 24, 40, 16
        a = _int_data((G, M, K), 1)
        b = _int_data((G, K, N), 2)
        sh = sharding.gemm_column_shard(N, rank, world)
        c_local = oracle.gemm_f32(a, np.ascontiguousarray(b[:, :, sh.begin:sh.end]), G, M, sh.size, K)
        c_all = sharding.gather_columns(torch.from_numpy(c_local), N).numpy()
        out["gemm"] = bool(np.array_equal(c_all, oracle.gemm_f32(a, b, G, M, N, K)))
        # --- convolution backward weight: batch split + all-reduce of the partial gradients ---
        full = oracle.Conv(n=4, c=3, k=5, h=7, w=6, y=3, x=3, pad_h=1, pad_w=1)
        inp = _int_data((full.n, 1, full.c, full.h, full.w), 3)
        dy = _int_data((full.n, 1, full.k, full.ho, full.wo), 4)
        bs = sharding.conv_batch_shard(full.n, rank, world)
        part = oracle.Conv(n=bs.size, c=3, k=5, h=7, w=6, y=3, x=3, pad_h=1, pad_w=1)
        dw_part = oracle.conv_f32(part, oracle.BWD_WEIGHT, None, inp[bs.begin:bs.end], dy[bs.begin:bs.end])
        dw = sharding.allreduce_weight_gradient(torch.from_numpy(dw_part)).numpy()
        out["bwd_weight"] = bool(np.array_equal(dw, oracle.conv_f32(full, oracle.BWD_WEIGHT, None, inp, dy)))
        # --- convolution forward: batch split, no exchange ---
        fil = _int_data((1, full.k, full.c, full.y, full.x), 5)
        y_part = oracle.conv_f32(part, oracle.FWD, fil, inp[bs.begin:bs.end], None)
        y_full = oracle.conv_f32(full, oracle.FWD, fil, inp, None).reshape(full.n, -1)
        out["fwd"] = bool(np.array_equal(y_part.reshape(bs.size, -1), y_full[bs.begin:bs.end]))
        # --- job time = slowest rank ---
        out["time"] = sharding.job_time_ms(10.0 + 5.0 * rank)
        results[rank] = out
    finally:
        dist.destroy_process_group()


def test_two_ranks_recombine_to_the_unsplit_result():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert len(results) == world
        for rank in range(world):
            r = results[rank]
            assert r["gemm"], f"rank {rank}: gathered column-split GEMM differs"
            assert r["bwd_weight"], f"rank {rank}: all-reduced weight gradient differs"
            assert r["fwd"], f"rank {rank}: batch-split forward differs"
            assert r["time"] == 15.0


@pytest.mark.parametrize("total,world,granule", [(4096, 8, 8), (11008, 8, 8), (256, 8, 1), (512, 3, 1), (5, 8, 1),
                                                  (1000, 4, 8), (0, 2, 1), (7, 1, 1)])
def test_shards_tile_the_range(total, world, granule):
    ok, shards = sharding.covers_exactly(total, world, granule)
    assert ok, shards
    sizes = [s.size for s in shards]
    assert max(sizes) - min(sizes) <= granule or total < world * granule
    for s in shards[:-1]:
        assert s.size % granule == 0 or s.end == total


def test_shard_range_rejects_bad_arguments():
    with pytest.raises(ValueError):
        sharding.shard_range(10, 2, 2)
    with pytest.raises(ValueError):
        sharding.shard_range(-1, 0, 2)
