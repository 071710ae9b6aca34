"""CPU, world_size 2 over gloo: the host-side logic of the multi-GPU path (sequence sharding, no
data-path collective; the only collectives are the timing reductions)."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import __graft_entry__ as entry
    ak = entry.load_package()
    from akasha_core_b200 import sharding
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    mine = sharding.shard_round_robin(11, rank, world)
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    # every rank generates ITS OWN prompts from rank-dependent seeds (weak scaling)
    lens = ak.uniform_ints(4, 16, 448, seed=2 + 1000 * rank).tolist()
    all_lens = [None] * world
    dist.all_gather_object(all_lens, lens)
    thr, units, secs = sharding.aggregate(dist, 100 * (rank + 1), 1.0 + rank)
    q.put((rank, gathered, all_lens, thr, units, secs))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_shard_without_overlap_and_aggregate_on_slowest():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29731 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, gathered, all_lens, thr, units, secs in res:
        flat = sorted(i for part in gathered for i in part)
        assert flat == list(range(11))                         # every sequence has exactly one owner
        assert gathered[0] == [0, 2, 4, 6, 8, 10] and gathered[1] == [1, 3, 5, 7, 9]
        assert all_lens[0] != all_lens[1]                      # ranks draw different workloads
        assert units == 300 and secs == 2.0 and abs(thr - 150.0) < 1e-9   # sum of units / slowest rank


def test_least_loaded_dispatch():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    from akasha_core_b200 import sharding
    parts = sharding.shard_least_loaded([5, 1, 1, 1, 4, 2], 2)
    assert parts == [[0, 5], [1, 2, 3, 4]]
    assert sharding.shard_round_robin(5, 1, 2) == [1, 3]
    with pytest.raises(ValueError):
        sharding.shard_round_robin(5, 2, 2)
