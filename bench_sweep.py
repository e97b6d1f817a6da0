"""Length / width sweep of the full model on the GPUs of one node, data parallel.

    python bench_sweep.py --requests 64                         # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench_sweep.py --requests 256

Requests are seeded synthetic trees: shared prefix length log-uniform in [256, 16384], 1-3 questions with stems of 4-40
tokens, 2-12 candidate leaves of 2-40 tokens. Request i is served by rank i % world (no collective on the data path). Every
request goes through Scorer.score_tokens (host layout build, pinned H2D, graph replay, D2H of the scores); graphs are
captured per (N, S, L2) bucket on first use and that cost is reported separately from the per-request latency, which is
taken on a second pass over the same requests. Prints one JSON line on rank 0: p50 / p95 ms per request and aggregate
requests per second.
"""
import argparse
import json
import os
import sys
import time

import numpy as np
import torch


def _tree(rng, root_len, q_lens, leaf_lens, groups, vocab):
    """Token lists of a two-level tree (shared prefix, one stem per question, one tail per candidate); first tokens differ
    at every branching point so the packed tree has exactly this shape."""
    root = rng.integers(200, vocab, root_len).tolist()
    stems = [[8 + r] + rng.integers(200, vocab, ql - 1).tolist() for r, ql in enumerate(q_lens)]
    seqs, seen = [], {}
    for ll, r in zip(leaf_lens, groups):
        seen[r] = seen.get(r, 0) + 1
        seqs.append(root + stems[r] + [100 + seen[r]] + rng.integers(200, vocab, ll - 1).tolist())
    return seqs, list(groups)


def make_requests(n, seed, vocab, max_prefix):
    rng = np.random.default_rng(seed)
    reqs = []
    for _ in range(n):
        root = int(round(np.exp(rng.uniform(np.log(256), np.log(max_prefix)))))
        R = int(rng.integers(1, 4))
        S = int(rng.integers(max(2, R), 13))
        groups = sorted(int(g) for g in np.concatenate([np.arange(R), rng.integers(0, R, S - R)]))
        q_lens = [int(x) for x in rng.integers(4, 41, R)]
        leaf_lens = [int(x) for x in rng.integers(2, 41, S)]
        reqs.append(_tree(rng, root, q_lens, leaf_lens, groups, vocab))
    return reqs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--max-prefix", type=int, default=16384)
    ap.add_argument("--layers", type=int, default=64, help="debugging only")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "open-jev-fast_b200"))
from ojb200 import _lib, fastmodel as FM, modelgen as MG, server as SV
    kw = dict(MG.FULL)
    kw["num_hidden_layers"] = args.layers
    cfg = MG.make_config(**kw)
    fast = FM.FastQwen35(MG.build_core(cfg, device=dev, seed=0), free_original=True)
    W, b = MG.make_head(cfg.hidden_size, A=1, seed=1, device=dev)
    scorer = SV.Scorer(fast, W, b, pad_id=0, device=dev, max_graphs=4096)
    reqs = make_requests(args.requests, args.seed, cfg.vocab_size, args.max_prefix)
    mine = SV.shard_requests(len(reqs), rank, world)

    t0 = time.perf_counter()
    for i in mine:                                   # first pass: captures one graph per bucket
        scorer.score_tokens(*reqs[i]).cpu()
    capture_s = time.perf_counter() - t0
    _lib.check_status(dev)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    lat, rows = [], []
    t0 = time.perf_counter()
    for i in mine:                                   # second pass: steady state
        t = time.perf_counter()
        scorer.score_tokens(*reqs[i]).cpu()
        lat.append((time.perf_counter() - t) * 1e3)
        rows.append(scorer.last["rows"])
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    _lib.check_status(dev)
    stats = torch.tensor([wall, capture_s, float(len(mine))], dtype=torch.float64, device=dev)
    all_lat = torch.tensor(lat, dtype=torch.float64, device=dev)
    if world > 1:
        gathered = [torch.zeros(2 * (len(reqs) // world + 1), dtype=torch.float64, device=dev) for _ in range(world)]
        pad = torch.full((2 * (len(reqs) // world + 1),), -1.0, dtype=torch.float64, device=dev)
        pad[:len(lat)] = all_lat
        dist.all_gather(gathered, pad)
        all_lat = torch.cat([g[g >= 0] for g in gathered])
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        wall, capture_s = float(mx[0]), float(mx[1])
    if rank == 0:
        l = np.sort(all_lat.cpu().numpy())
        print(json.dumps({"sweep": "prefix 256..%d log-uniform, 1-3 questions, 2-12 leaves of 2-40 tokens" % args.max_prefix,
                          "requests": len(reqs), "n_gpus": world, "layers": args.layers,
                          "p50_ms": float(l[len(l) // 2]), "p95_ms": float(l[int(len(l) * 0.95)]), "mean_ms": float(l.mean()),
                          "requests_per_s": len(reqs) / wall, "rows_min_max": [int(min(rows)), int(max(rows))],
                          "graphs_captured_rank0": len(scorer.graphs), "capture_pass_s": capture_s}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
