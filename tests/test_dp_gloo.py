"""Data-parallel request sharding with two CPU ranks over gloo: every request is served by exactly one rank, the shards
are balanced, and the aggregate throughput reduction used by bench.py (max of the per-rank times) behaves. Host logic only:
each rank builds the layouts of its own requests with the C++ builder."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ojb200 import trees


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ojb200 import layout as PL
    from ojb200.server import shard_requests
    n_req = 7
    mine = shard_requests(n_req, rank, world)
    rows = 0
    for i in mine:
        seqs, groups = trees.example_tree(i)
        d, *_ = PL.gtree_host(seqs, groups, 0)
        rows += d["Nreal"]
    served = torch.zeros(n_req, dtype=torch.int64)
    served[mine] = 1
    dist.all_reduce(served)
    t = torch.tensor([1.0 + rank], dtype=torch.float64)      # stand-in for the rank's timed region
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    tot = torch.tensor([rows], dtype=torch.int64)
    dist.all_reduce(tot)
    if rank == 0:
        out.put((served.tolist(), float(t), int(tot), len(mine)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    served, tmax, rows, n0 = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert served == [1] * 7            # each request exactly once
    assert tmax == 2.0                  # max over ranks
    assert rows == 7 * 277 and n0 == 4  # all rows accounted for; shards differ by at most one request
