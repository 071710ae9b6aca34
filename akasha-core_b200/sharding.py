"""Multi-GPU host logic: sequences are independent, so N GPUs = N engines and NO data-path
collective. These helpers decide which rank owns which sequence and combine per-rank results;
`torch.distributed` is used only for the timing barrier and the max-over-ranks reduction."""
from __future__ import annotations


def shard_round_robin(n_items: int, rank: int, world: int):
    """Indices owned by `rank` when arrivals are dealt round-robin (arrival order kept)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    return list(range(rank, n_items, world))


def shard_least_loaded(costs, world: int):
    """Greedy dispatcher: each arriving sequence goes to the rank with the least outstanding
    cost (KV blocks); ties go to the lowest rank. Returns one index list per rank."""
    load = [0] * world
    out = [[] for _ in range(world)]
    for i, c in enumerate(costs):
        r = min(range(world), key=lambda j: (load[j], j))
        out[r].append(i)
        load[r] += int(c)
    return out


def aggregate(dist, units_local: int, seconds_local: float, device=None):
    """Whole-job throughput: units summed over ranks divided by the SLOWEST rank's time.
    `dist` is torch.distributed (initialised) or None for a single process."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return units_local / seconds_local, units_local, seconds_local
    import torch
    t = torch.tensor([float(units_local)], dtype=torch.float64, device=device)
    s = torch.tensor([float(seconds_local)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    dist.all_reduce(s, op=dist.ReduceOp.MAX)
    return t.item() / s.item(), int(t.item()), s.item()
