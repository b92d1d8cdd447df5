"""CPU-only, world_size 2 over gloo: the multi-GPU path of bench.py without GPUs -- shard
plans are disjoint and complete, no data-path collective is needed (each rank's oracle result
equals the corresponding slice of the unsharded result), and the timing reduction is a MAX."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from flashkda_b200.sharding import plan, reduce_max_ms  # noqa: E402
from flashkda_b200.workloads import Workload, baseline_workload, make_inputs  # noqa: E402


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    w = Workload("t", H=4, B=2, T=40, state_in="fp32", state_out="fp32", seed=5)
    # strong plan: my heads of the same global problem
    sh = plan(w, world, rank, "head")
    x = make_inputs(w)                                  # every rank can regenerate the global tensors
    hs = sh.heads
    cut = lambda t, dim: t.index_select(dim, torch.tensor(list(hs))).contiguous()
    o_loc, s_loc = oracle.recurrence_f64(cut(x["q"], 2), cut(x["k"], 2), cut(x["v"], 2), cut(x["g"], 2),
                                         cut(x["beta"], 2), x["scale"], cut(x["A_log"], 0), cut(x["dt_bias"], 0),
                                         x["lower_bound"], initial_state=cut(x["initial_state"], 1), nthreads=1)
    o_all, s_all = oracle.recurrence_f64(x["q"], x["k"], x["v"], x["g"], x["beta"], x["scale"], x["A_log"],
                                         x["dt_bias"], x["lower_bound"], initial_state=x["initial_state"], nthreads=1)
    ok_slice = bool(torch.equal(o_loc, cut(o_all, 2)) and torch.equal(s_loc, cut(s_all, 1)))
    # weak plan: distinct seeds, global token count scales with the world
    shw = plan(w, world, rank, "seq")
    ms = reduce_max_ms([10.0 + rank, 1.0], world)
    gathered = [None] * world
    dist.all_gather_object(gathered, (list(hs), shw.workload.seed, shw.tokens_global, sh.tokens_global))
    if rank == 0:
        q.put(dict(ok_slice=ok_slice, ms=ms, gathered=gathered))
    else:
        q.put(dict(ok_slice=ok_slice))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_over_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r["ok_slice"] for r in res), "a head shard computed alone differs from its slice of the full result"
    r0 = next(r for r in res if "ms" in r)
    assert r0["ms"] == [11.0, 1.0]                      # MAX over ranks
    heads = sorted(h for g in r0["gathered"] for h in g[0])
    assert heads == [0, 1, 2, 3]                        # disjoint and complete
    assert sorted(g[1] for g in r0["gathered"]) == [5, 6]
    assert all(g[2] == 2 * 80 and g[3] == 80 for g in r0["gathered"])


def test_plan_rejects_bad_splits():
    import pytest
    w = baseline_workload(1)
    with pytest.raises(ValueError):
        plan(w, 3, 0, "head")
    with pytest.raises(ValueError):
        plan(w, 2, 2, "seq")
    assert plan(w, 8, 3, "head").heads == range(12, 16)
    assert plan(w, 8, 3, "seq").tokens_global == 8 * 32768
