"""How one `flash_kda.fwd` workload is split over ranks (one process per GPU).

Every (sequence, head) pair is an independent recurrence (the reference loops over them
independently, tests/torch_ref.py:185-195), so ranks never exchange data on the path: a rank
just runs the operator on its own shard.  Two plans:
  * "seq"  (weak scaling): every rank gets the workload's own number of sequences; the global
    batch is world x that.  Seeds differ per rank so the shards are distinct sequences.
  * "head" (strong scaling): the workload is fixed and its heads are cut into `world`
    contiguous ranges; each rank holds contiguous [B,T,H/world,128] tensors.
The only collective is the harness's: a MAX all-reduce of the per-rank times.
"""
from dataclasses import dataclass, replace
from typing import Optional

from .workloads import Workload


@dataclass
class Shard:
    workload: Workload           # what this rank generates and runs
    heads: Optional[range]       # head slice of the global workload ("head" plan) or None
    tokens_global: int           # tokens processed by all ranks together per step
    scaling: str                 # "weak" | "strong"


def plan(w: Workload, world: int, rank: int, mode: str = "seq") -> Shard:
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if mode == "head" and world > 1:
        if w.H % world:
            raise ValueError(f"H={w.H} is not divisible by {world} ranks")
        per = w.H // world
        return Shard(w, range(rank * per, (rank + 1) * per), w.total_tokens, "strong")
    if mode not in ("seq", "head"):
        raise ValueError(mode)
    return Shard(replace(w, seed=w.seed + rank), None, w.total_tokens * world, "weak")


def reduce_max_ms(values, world: int, device=None):
    """MAX over ranks of a list of per-rank millisecond figures (torch.distributed must be
    initialised when world > 1).  Works on NCCL (CUDA tensor) and gloo (CPU tensor)."""
    import torch
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()
