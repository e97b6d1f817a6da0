"""The reference's own forward on this GPU: open-jev-fast's unmodified FastQwen35.forward_gtree (src/fastmodel.py:400-482) with
its own CUDA operators rebuilt for sm_100a, cuBLAS / cuDNN for what it delegates to them, under a CUDA graph as its server
runs it (src/server.py:32-49 Entry).

TEST INFRASTRUCTURE ONLY: needs the built files of oracle/build_ref_kernels.py (oracle/_ref/ojref/) and is used by
tests/test_full_model_gpu.py (scores of the reference's kernels on the same weights) and by bench.py's reference-on-GPU leg
(milliseconds per request next to this library's). Every switch of the reference stays at its default: GDN_VER 6 (gdn_fused6),
FATTN 3 up to 384 rows and SDPA + gate_mul3 above, split-K 2 through torch.bmm, F.linear for the projections (its cuBLASLt
search extension is not built; F.linear is the fallback it names, src/fastmodel.py:65-69).

    python -m oracle.ref_forward --workload baseline --steps 30 --warmup 5      # one JSON line
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "open-jev-fast_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def load_model(core):
    """The reference's FastQwen35 around a Hugging Face Qwen3_5TextModel that lives on the GPU. None if the built files are
    missing."""
    from oracle import build_ref_kernels as B
    mod = B.load_fastmodel()
    if mod is None:
        return None, None
    return mod, mod.FastQwen35(core)


def scores(fast_ref, seqs, groups, W, b, pad_id=0):
    """fp32 [S, A] scores of one request through the reference's tree forward (eager, no graph)."""
    import torch
    with torch.inference_mode():
        ids, lay = fast_ref.gtree_build(seqs, groups, pad_id, NB=32, PB=16)
        h = fast_ref.forward_gtree(ids, lay).float()
        return (h @ W.float().t() + (b.float() if b is not None else 0.0)), lay.key


def timed_graph(fast_ref, seqs, groups, W, b, steps, warmup, pad_id=0):
    """src/server.py:32-49: two eager passes on a side stream, capture, then `steps` replays between CUDA events after
    `warmup` untimed ones. Returns (per-replay ms list, scores, key)."""
    import torch
    with torch.inference_mode():
        ids, lay = fast_ref.gtree_build(seqs, groups, pad_id, NB=32, PB=16)
        body = lambda: (fast_ref.forward_gtree(ids, lay).float() @ W.float().t() + b.float())
        st = torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            for _ in range(2):
                body()
        torch.cuda.current_stream().wait_stream(st)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = body()
        torch.cuda.synchronize()
        for _ in range(warmup):
            g.replay()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(True), torch.cuda.Event(True)) for _ in range(steps)]
        for a, c in ev:
            a.record()
            g.replay()
            c.record()
        torch.cuda.synchronize()
        return [a.elapsed_time(c) for a, c in ev], out.clone(), lay.key


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="baseline", choices=["baseline", "example"])
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--layers", type=int, default=64)
    args = ap.parse_args()
    import torch
    from ojb200 import modelgen as MG, trees
    try:
        kw = dict(MG.FULL)
        kw["num_hidden_layers"] = args.layers
        cfg = MG.make_config(**kw)
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        core = MG.build_core(cfg, device=dev, seed=0)
        mod, fast_ref = load_model(core)
        if fast_ref is None:
            print(json.dumps({"impl": "reference-gpu", "unavailable": "oracle/_ref/ojref is not built (oracle/build_ref_kernels.py)"}))
            return
        W, b = MG.make_head(cfg.hidden_size, A=1, seed=1, device=dev)
        seqs, groups = (trees.baseline_tree if args.workload == "baseline" else trees.example_tree)(0, cfg.vocab_size)
        from bench import ClockSampler
        with ClockSampler(0) as clocks:
            ms, out, key = timed_graph(fast_ref, seqs, groups, W, b, max(args.steps, 30), max(args.warmup, 5))
        ms.sort()
        print(json.dumps({"impl": "reference-gpu", "workload": args.workload, "key": list(key), "layers": args.layers,
                          "ms_per_request_p50": ms[len(ms) // 2], "ms_per_request_mean": sum(ms) / len(ms), "replays": len(ms),
                          "scores": [float(v) for v in out.flatten().cpu()], "clocks": clocks.summary(),
                          "what": "open-jev-fast FastQwen35.forward_gtree + fp32 head under a CUDA graph; its kernels.cu rebuilt "
                                  "for sm_100a, F.linear / torch.bmm projections, defaults of every switch"}), flush=True)
    except Exception as e:   # reported, never raised: the caller's own measurement must not depend on this leg
        print(json.dumps({"impl": "reference-gpu", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}), flush=True)


if __name__ == "__main__":
    main()
