"""The N>1 data path on CPU: world_size-2 gloo ranks shard independent units with the library's partition
rule, compute their share (with the oracle standing in for the device), and the gathered result equals
the single-rank result.  There is no data-path collective; all_gather is only the test's own check."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _unit_inputs(u):
    rng = np.random.default_rng(1000 + u)
    q = rng.standard_normal((1, 2, 24, 64)).astype(np.float16)
    k = rng.standard_normal((1, 2, 24, 64)).astype(np.float16)
    v = rng.standard_normal((1, 2, 24, 64)).astype(np.float16)
    return q, k, v


def _rank(rank, world, port, n_units, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import crispasr_b200
    from oracle import oracle
    first, count = crispasr_b200.SegmentScheduler.partition(n_units, world, rank)
    mine = torch.zeros((n_units, 24 * 2 * 64), dtype=torch.float32)
    for u in range(first, first + count):
        q, k, v = _unit_inputs(u)
        mine[u] = torch.from_numpy(oracle.flash_attn_ext(q, k, v, scale=0.125).reshape(-1))
    owned = torch.zeros(n_units, dtype=torch.int32)
    owned[first:first + count] = 1
    dist.all_reduce(mine)
    dist.all_reduce(owned)
    if rank == 0:
        np.save(os.path.join(out_dir, "gathered.npy"), mine.numpy())
        np.save(os.path.join(out_dir, "owned.npy"), owned.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_equals_single_rank(tmp_path, b200, orc):
    n_units, world = 7, 2
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank, args=(world, port, n_units, str(tmp_path)), nprocs=world, join=True)
    gathered = np.load(tmp_path / "gathered.npy")
    owned = np.load(tmp_path / "owned.npy")
    assert (owned == 1).all(), "every unit is owned by exactly one rank"
    for u in range(n_units):
        q, k, v = _unit_inputs(u)
        assert np.array_equal(gathered[u], orc.flash_attn_ext(q, k, v, scale=0.125).reshape(-1))
