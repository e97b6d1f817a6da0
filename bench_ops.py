"""Micro-benchmark of the non-GEMM kernels at the model's dimensions on one tree (for tuning and for ncu captures).

    python bench_ops.py [--tree baseline|example] [--reps 20] [--only gdn|attn|norm]

Prints one JSON line per op: microseconds per call (CUDA events over `reps` back-to-back calls after a warm-up).
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "open-jev-fast_b200"))
from ojb200 import ext as K
from ojb200 import layout as PL

bf16 = torch.bfloat16


def _time(fn, reps):
    """Microseconds per call with `reps` calls captured in one CUDA graph (no host launch cost in the number)."""
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(st)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(reps):
            fn()
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(True), torch.cuda.Event(True)
    a.record()
    g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / reps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tree", default="baseline")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--only", default=None)
    ap.add_argument("--hv", type=int, default=32)
    args = ap.parse_args()
    from ojb200 import trees
    if args.tree.startswith("root"):       # e.g. --tree root8192: one long shared root, two questions, four candidates
        seqs, groups = trees.make_tree(7, int(args.tree[4:]), [20, 22], [6, 9, 4, 12], [0, 0, 1, 1])
    else:
        seqs, groups = (trees.baseline_tree if args.tree == "baseline" else trees.example_tree)(0)
    ids, lay = PL.gtree_build(seqs, groups, 0, dev="cuda", dense=False)
    N, HK, HV, HD, H = lay.N, 16, args.hv, 128, 5120
    KD, VD = HK * HD, HV * HD
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g, device="cuda")
    out = lambda name, us: print(json.dumps({"op": name, "tree": args.tree, "N": N, "us": round(us, 2)}), flush=True)
    want = lambda n: args.only is None or args.only == n
    if want("gdn"):
        proj = rnd(N, 2 * KD + 2 * VD + 2 * HV).to(bf16)
        convw = (rnd(2 * KD + VD, 4) * 0.5).to(bf16)
        A_log = torch.log(torch.rand(HV, generator=g, device="cuda") * 16 + 1e-3).to(bf16)
        dt = torch.ones(HV, device="cuda", dtype=bf16)
        q, k, v, gg, beta = K.linattn_prep_rows(proj, lay.hist, convw, A_log, dt, KD, VD, HV, HK, HD)
        out("gdn_prep", _time(lambda: K.linattn_prep_rows(proj, lay.hist, convw, A_log, dt, KD, VD, HV, HK, HD), args.reps))
        o = torch.zeros(N, HV, HD, dtype=bf16, device="cuda")
        q3, k3, v3 = q.view(N, HK, HD), k.view(N, HK, HD), v.view(N, HV, HD)
        st = torch.empty(1 + lay.S, HV, HD, HD, device="cuda")
        out("gdn intra + depth-first state walk", _time(lambda: K.gdn_chunked(q3, k3, v3, gg, beta, HD ** -0.5, lay.chunks, lay.steps,
                                                                            lay.walk_ptr, 1, None, None, o), args.reps))
        out("gdn intra + level-parallel state pass", _time(lambda: K.gdn_tree_levels(q3, k3, v3, gg, beta, HD ** -0.5, lay, o, st), args.reps))
        normw = torch.ones(HD, device="cuda", dtype=bf16)
        out("gated_rmsnorm", _time(lambda: K.gated_rmsnorm(o, proj, normw, HV, HD, 2 * KD + VD, 1e-6), args.reps))
    if want("attn"):
        HQ, HKV, D = 24, 4, 256
        proj = rnd(N, 2 * HQ * D + 2 * HKV * D).to(bf16)
        w1 = torch.ones(D, device="cuda")
        ang = lay.pos.float()[:, None] * (1.0 / (10000 ** (torch.arange(0, 64, 2, device="cuda").float() / 64)))[None]
        cosb, sinb = torch.cat([ang.cos()] * 2, -1).to(bf16), torch.cat([ang.sin()] * 2, -1).to(bf16)
        qt, kt, vt, gate = K.fullattn_prep2(proj, w1, w1, cosb, sinb, 1, N, HQ, HKV, D, 1e-6)
        out("fullattn_prep", _time(lambda: K.fullattn_prep2(proj, w1, w1, cosb, sinb, 1, N, HQ, HKV, D, 1e-6), args.reps))
        for gq in ((6,) if N > 2048 else (3, 6)):
            out(f"tree_attn ranges gq={gq}", _time(lambda: K.fattn_tree_ranges(qt, kt, vt, gate, lay.krange, D ** -0.5, gq), args.reps))
        if N <= 2048:
            out("tree_attn bits gq=6", _time(lambda: K.fattn_tree(qt, kt, vt, gate, None, lay.vbits, D ** -0.5, 6), args.reps))
        vt_t = K.fullattn_prep2(proj, w1, w1, cosb, sinb, 1, N, HQ, HKV, D, 1e-6, with_vt_t=True)[4]
        out("fullattn_prep + transposed V", _time(lambda: K.fullattn_prep2(proj, w1, w1, cosb, sinb, 1, N, HQ, HKV, D, 1e-6, with_vt_t=True), args.reps))
        out("tree_attn tcgen05", _time(lambda: K.fattn_tree_tc(qt, kt, vt_t, gate, lay.krange, D ** -0.5), args.reps))
    if want("norm"):
        x, d = rnd(N, H).to(bf16), rnd(N, H).to(bf16)
        w1 = torch.ones(H, device="cuda")
        out("add_rmsnorm", _time(lambda: K.add_rmsnorm(x, d, w1, lay.rowmask, 1e-6), args.reps))


if __name__ == "__main__":
    main()
