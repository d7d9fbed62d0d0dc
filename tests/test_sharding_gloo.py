"""The N>1 path on CPU: two gloo ranks shard the records with no data-path collective, and the
timing reduction used by the benchmark takes the maximum over ranks."""
import os
import socket

import torch.distributed as dist
import torch.multiprocessing as mp

from aeon_b200.sharding import shard_indices


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from aeon_b200.sharding import max_over_ranks, shard_indices as si
    mine = si(1000, 32, rank, world)
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)          # test-side check only; the data path itself never communicates
    slow = max_over_ranks(10.0 + rank)
    if rank == 0:
        out.put((gathered, slow))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_get_disjoint_shards_and_max_timing():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    gathered, slow = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    a, b = gathered
    assert len(a) == len(b) == 500 and not set(a) & set(b)
    assert a[:32] == list(range(0, 32)) and b[:32] == list(range(32, 64)) and a[32:64] == list(range(64, 96))
    assert slow == 11.0


def test_sharding_matches_the_reference_interleave_for_every_world_size():
    for world in (1, 2, 4, 8):
        shards = [shard_indices(1024, 128, r, world) for r in range(world)]
        flat = sorted(i for s in shards for i in s)
        assert flat == list(range(1024))
        assert all(len(s) == 1024 // world for s in shards)
    # tail handling (record count not a multiple of batch*world): aeon test/test_manifest_tsv.cpp:113-205
    s0, s1 = shard_indices(10, 3, 0, 2), shard_indices(10, 3, 1, 2)
    assert s0 == [0, 1, 2, 6, 7] and s1 == [3, 4, 5, 8, 9]
