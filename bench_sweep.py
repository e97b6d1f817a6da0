"""Length / width sweep of the full model: one stream of mixed-shape requests through the router onto 1 .. 8 GPUs of a node.

    python bench_sweep.py --gpus 1 --requests 256
    python bench_sweep.py --gpus 8 --requests 256

Requests are seeded synthetic trees: shared prefix length log-uniform in [256, 16384], 1-3 questions with stems of 4-40
tokens, 2-12 candidate leaves of 2-40 tokens. ojb200.router.Router in front of one ojb200.server.Scorer per GPU (full
weights, own graph cache, own stream; by default each in a child process of its own, fed over a pipe), shortest queue by
outstanding tokens; nothing is exchanged between GPUs.
Every request goes through Scorer.score_tokens (host layout build, pinned H2D, graph lookup or capture, replay, D2H of the
scores). The stream is served twice: the first pass captures one graph per (N, S, L2) key where a GPU meets the key for the
first time (reported as capture cost), the second pass is the steady state (with --capture-after 2: three times — eager at
first sight, capture at the second, steady state). One JSON line: service time per request (p50 /
p95 / mean, host clock around the worker's call), sojourn time with queueing, aggregate requests per second, host layout
time, graphs captured and requests served per GPU.
"""
import argparse
import json
import os
import sys
import threading
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


def scorer_worker(i, layers, tune, capture_after=1):
    """Builds the model and its Scorer on GPU i and returns the serve function of one worker: request -> record with the
    scores (numpy), the service time and what the scorer reports. Runs in the router's process (thread workers) or in a child
    process of its own (process workers)."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "open-jev-fast_b200"))
    from ojb200 import _lib, fastmodel as FM, modelgen as MG, server as SV
    if not tune:
        FM.FastQwen35.TUNE_MAX_ROWS = 0
    kw = dict(MG.FULL)
    kw["num_hidden_layers"] = layers
    cfg = MG.make_config(**kw)
    dev = torch.device("cuda", i)
    with torch.cuda.device(dev):
        fast = FM.FastQwen35(MG.build_core(cfg, device=dev, seed=0), free_original=True)
        W, b = MG.make_head(cfg.hidden_size, A=1, seed=1, device=dev)
        sc = SV.Scorer(fast, W, b, pad_id=0, device=dev, max_graphs=4096, capture_after=capture_after)

    def fn(req):
        t = time.perf_counter()
        out, info = sc.score_tokens(req[0], req[1], with_info=True)
        out = out.cpu().numpy()                              # the synchronisation point of this request
        _lib.check_status(sc.device)
        return dict(scores=out, ms=(time.perf_counter() - t) * 1e3, gpu=i, rows=info["rows"], build_ms=info["build_ms"],
                    captured=info["captured"])
    return fn


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--max-prefix", type=int, default=16384)
    ap.add_argument("--layers", type=int, default=64, help="debugging only")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--workers", choices=("process", "thread"), default="process",
                    help="one child process per GPU behind the router (own interpreter: layout builds and graph launches of "
                    "different GPUs never wait for each other), or all scorers in the router's process")
    ap.add_argument("--capture-after", type=int, default=1, help="capture a key's graph at its n-th request (1: at first sight, "
                    "as the reference does; 2: the first request of a key runs eagerly). The stream is served n + 1 times; "
                    "the last pass is the steady state")
    ap.add_argument("--verbose", action="store_true", help="per-request first pass / replay comparison on stderr")
    ap.add_argument("--tune", action="store_true", help="time the GEMM candidates per new row count (FastQwen35.tune) instead of "
                    "using the library's cost model: better kernels below 1024 rows, a much longer capture pass")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "open-jev-fast_b200"))
    from ojb200 import modelgen as MG, router as RT
    n_gpu = min(args.gpus, torch.cuda.device_count())
    vocab = MG.make_config(**MG.FULL).vocab_size
    t0 = time.perf_counter()
    if args.workers == "process":
        workers = [RT.ProcessWorker(scorer_worker, (i, args.layers, args.tune, args.capture_after)) for i in range(n_gpu)]
        for w in workers:
            w.wait_ready(1800)
    else:
        workers = [None] * n_gpu

        def build(i):
            workers[i] = scorer_worker(i, args.layers, args.tune, args.capture_after)
        ths = [threading.Thread(target=build, args=(i,)) for i in range(n_gpu)]
        for t in ths:
            t.start()
        for t in ths:
            t.join()
        assert all(w is not None for w in workers), "a model failed to build"
    build_s = time.perf_counter() - t0

    reqs = make_requests(args.requests, args.seed, vocab, args.max_prefix)
    router = RT.Router(workers)
    try:
        warm, warm_s = [], []
        for _ in range(max(1, args.capture_after)):           # graphs are captured in the last of these passes
            t0 = time.perf_counter()
            warm.append(router.map(reqs))
            warm_s.append(time.perf_counter() - t0)
        first, capture_s = warm[-1], warm_s[-1]
        t0 = time.perf_counter()
        futs = [router.submit(r) for r in reqs]
        second = [f.result() for f in futs]
        wall = time.perf_counter() - t0
    finally:
        router.close()
    lat = np.sort(np.array([r["ms"] for r in second]))
    rows = np.array([r["rows"] for r in second])
    same = all(np.array_equal(a["scores"], b["scores"]) for a, b in zip(first, second) if a["gpu"] == b["gpu"])
    if args.verbose:
        for i, (a, b) in enumerate(zip(first, second)):
            print("request", i, "rows", a["rows"], "gpu", a["gpu"], b["gpu"], "captured", a["captured"], "max diff",
                  float(np.abs(a["scores"] - b["scores"]).max()), file=sys.stderr)
    st = router.stats()
    print(json.dumps({"sweep": "prefix 256..%d log-uniform, 1-3 questions, 2-12 leaves of 2-40 tokens" % args.max_prefix,
                      "requests": len(reqs), "n_gpus": n_gpu, "workers": args.workers, "layers": args.layers, "tuned": bool(args.tune),
                      "p50_ms": float(lat[len(lat) // 2]), "p95_ms": float(lat[int(len(lat) * 0.95)]), "mean_ms": float(lat.mean()),
                      "requests_per_s": len(reqs) / wall, "steady_pass_s": wall, "capture_pass_s": capture_s,
                      "capture_after": args.capture_after, "eager_first_sight_pass_s": warm_s[0] if args.capture_after > 1 else None,
                      "eager_first_sight_ms_mean": float(np.mean([r["ms"] for r in warm[0]])) if args.capture_after > 1 else None,
                      "capture_ms_mean": float(np.mean([r["ms"] for r in first])),
                      "model_build_s": build_s, "graphs_captured": int(sum(r["captured"] for r in first)),
                      "recaptured_in_steady_pass": int(sum(r["captured"] for r in second)),
                      "host_layout_ms_mean": float(np.mean([r["build_ms"] for r in second])),
                      "host_layout_ms_max": float(np.max([r["build_ms"] for r in second])),
                      "rows_min": int(rows.min()), "rows_median": int(np.median(rows)), "rows_max": int(rows.max()),
                      "served_per_gpu": st["served"], "workers_alive": st["alive"], "requeued": st["requeued"],
                      "worker_errors": st["errors"], "replay_equals_first_pass": bool(same)}), flush=True)


if __name__ == "__main__":
    main()
