"""The N>1 host path on CPU: two gloo ranks shard a ragged request list, each plans only its own sequences with the
host planner, and the ranks agree (through one all-gather, the path's only collective) that every sequence is served
exactly once and that the load is balanced."""
import importlib
import os
import sys

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = "llada2-orin-cuda_b200"


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = importlib.import_module(PKG)
        api = importlib.import_module(PKG + ".api")
        lens = pkg.workload.ragged_lengths(40)
        mine = pkg.sharding.shard_lpt(lens, world)[rank]
        st, items, cta_first = api.plan_preview([int(lens[i]) for i in mine], 148)
        units = int(items[:, 4:6].sum())
        assert units == st.total_units == 4 * sum(int(lens[i]) + 1 for i in mine)
        served = torch.zeros(40, dtype=torch.int64)
        served[mine] = 1
        dist.all_reduce(served)                                   # every sequence exactly once over all ranks
        loads = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(loads, torch.tensor([units]))             # stands in for the final output gather
        loads = [int(x) for x in loads]
        q.put((rank, bool((served == 1).all()), max(loads) / (sum(loads) / world)))
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_and_plan():
    world, port = 2, 29531 + os.getpid() % 200
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] for r in res)
    assert all(r[2] <= 1.05 for r in res)
