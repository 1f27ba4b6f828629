"""CPU tests of the multi-GPU host logic, including a world_size-2 gloo run."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_m_slabs_partition_exactly():
    from spork_b200.sharding import m_slab

    for M in (0, 1, 255, 256, 257, 8192, 65536, 65536 + 300, 1000):
        for world in (1, 2, 3, 4, 8):
            slabs = [m_slab(M, r, world) for r in range(world)]
            assert slabs[0].start == 0
            assert sum(s.count for s in slabs) == M
            for prev, nxt in zip(slabs, slabs[1:]):
                assert prev.stop == nxt.start
            for s in slabs:
                assert s.start % 256 == 0 or s.start == M
    # the headline case: 65536 rows over 8 ranks = 8192 rows each
    assert [m_slab(65536, r, 8).count for r in range(8)] == [8192] * 8
    with pytest.raises(ValueError):
        m_slab(10, 2, 2)


def test_head_slabs():
    from spork_b200.sharding import head_slab

    assert [head_slab(256, r, 8).count for r in range(8)] == [32] * 8
    counts = [head_slab(10, r, 4).count for r in range(4)]
    assert sum(counts) == 10 and max(counts) - min(counts) <= 1


def test_whole_job_rate():
    from spork_b200.sharding import whole_job_rate

    assert whole_job_rate([10.0, 10.0], 2.0) == 10.0
    with pytest.raises(ValueError):
        whole_job_rate([1.0], 0.0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from oracle import oracle as orc
    from spork_b200.sharding import m_slab

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        slab = m_slab(M, rank, world, align=64)
        # every rank regenerates B from the seed (the replica) and only its own rows of A
        a_full = orc.fill_f16(M, K, orc.DATA_UNIFORM_PM1, orc.SEED_A)
        b = orc.fill_f16(N, K, orc.DATA_UNIFORM_PM1, orc.SEED_B)
        c_slab = orc.gemm_f16f32(a_full[slab.start:slab.stop], b)
        np.save(os.path.join(out_dir, f"c_{rank}.npy"), c_slab)
        # timing protocol: barrier, then the max over ranks of the per-rank time
        dist.barrier()
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        units = torch.tensor([float(slab.count)], dtype=torch.float64)
        dist.all_reduce(units, op=dist.ReduceOp.SUM)
        assert t.item() == float(world)
        assert units.item() == float(M)
    finally:
        dist.destroy_process_group()


def test_m_sharded_gemm_two_ranks_gloo(tmp_path, orc):
    import torch.multiprocessing as mp

    M, N, K = 320, 96, 136
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, M, N, K, str(tmp_path)), nprocs=world, join=True)
    from spork_b200.sharding import m_slab

    a = orc.fill_f16(M, K, orc.DATA_UNIFORM_PM1, orc.SEED_A)
    b = orc.fill_f16(N, K, orc.DATA_UNIFORM_PM1, orc.SEED_B)
    ref = orc.gemm_f16f32(a, b)
    got = np.concatenate([np.load(tmp_path / f"c_{r}.npy") for r in range(world)], axis=0)
    assert got.shape == ref.shape
    assert (got == ref).all()
    assert m_slab(M, 0, world, align=64).count + m_slab(M, 1, world, align=64).count == M
