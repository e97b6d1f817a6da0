"""Work-unit timelines of the block GEMM kernels (256-row block kernel and CTA-pair kernel) through ojb_gemm_set_trace.

    python bench_gemm_timeline.py --m 544 --shape 5120 34816 --kind swiglu --variant 3
    python bench_gemm_timeline.py --m 544 --shape 17408 5120 --kind splitk --splits 2 --variant 3 --detail 2

`--variant` is the library's variant code (3 block kernel, 4 all rows swapped, 16..256 forced w-tile width, 5 / 6 CTA-pair
kernel, 512 + width = pair kernel with forced width). One JSON line: the span of the launch, and per unit type the mean time
from the end of the previous epilogue to the completed accumulator ("main") and the mean epilogue time, in microseconds, plus
how many units each CTA ran, the spread of the main-loop time over the units of a type and of the finishing time over the CTAs. `--repeat` / `--knob` need a library built with -DOJB_GEMM_PROBES (MMAs of a stage issued r
times, pipeline depth capped, parts of the epilogue skipped): the shipped library has neither and the options are refused.
"""
import argparse
import json

import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "open-jev-fast_b200"))
from ojb200 import _lib  # noqa: E402
from ojb200 import lt_ext as LT  # noqa: E402
from ojb200._lib import call, i32, i64, ptr, stream_ptr  # noqa: E402

bf16 = torch.bfloat16
CAP = 8192


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=544)
    ap.add_argument("--shape", type=int, nargs=2, default=[5120, 34816], metavar=("K", "N"))
    ap.add_argument("--kind", default="plain", choices=["plain", "swiglu", "splitk"])
    ap.add_argument("--splits", type=int, default=1)
    ap.add_argument("--variant", type=int, default=3)
    ap.add_argument("--repeat", type=int, nargs="+", default=[1])
    ap.add_argument("--knob", type=int, nargs="+", default=[0])
    ap.add_argument("--detail", type=int, default=0, help="print the timelines of this many latest-finishing CTAs")
    args = ap.parse_args()
    dev = torch.device("cuda")
    probes = hasattr(_lib.lib(), "ojb_gemm_set_probe")
    if (args.repeat != [1] or args.knob != [0]) and not probes:
        raise SystemExit("--repeat / --knob need a library built with -DOJB_GEMM_PROBES")
    M, (K, N) = args.m, args.shape
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(M, K, generator=g, device=dev).to(bf16)
    ws = [(torch.randn(N, K, generator=g, device=dev) * 0.02).to(bf16) for _ in range(2)]
    if args.kind == "swiglu":
        blk = 64 if args.variant == 5 or args.variant >= 512 else 128
        ws = [LT.interleave_gate_up(w[:N // 2].contiguous(), w[N // 2:].contiguous(), blk) for w in ws]
    rec = torch.zeros(1 + 4 * CAP, dtype=torch.int64, device=dev)
    st = ptr(_lib.status_word(dev))

    def launch(w):
        if args.kind == "plain":
            out = torch.empty(M, N, dtype=bf16, device=dev)
            call("ojb_gemm_bf16", ptr(x), ptr(w), ptr(out), i64(M), i64(N), i64(K), i32(args.variant), st, stream_ptr())
        elif args.kind == "swiglu":
            out = torch.empty(M, N // 2, dtype=bf16, device=dev)
            call("ojb_gemm_bf16_swiglu_v", ptr(x), ptr(w), ptr(out), i64(M), i64(N), i64(K), i32(args.variant), st, stream_ptr())
        else:
            out = torch.empty(args.splits, M, N, dtype=torch.float32, device=dev)
            call("ojb_gemm_bf16_splitk", ptr(x), ptr(w), ptr(out), i64(M), i64(N), i64(K), i32(args.splits), i32(args.variant), st,
                 stream_ptr())
        return out

    try:
        for knob in args.knob:
            for rep in args.repeat:
                call("ojb_gemm_set_trace", None, i32(0))
                if probes:
                    call("ojb_gemm_set_probe", i32(rep), i32(knob))
                for w in ws:
                    launch(w)                               # warm-up, and the weights of the traced launch leave the L2
                torch.cuda.synchronize()
                rec.zero_()
                call("ojb_gemm_set_trace", ptr(rec), i32(CAP))
                launch(ws[0])
                torch.cuda.synchronize()
                t = rec.cpu().numpy()
                n = int(min(t[0], CAP))
                line = dict(M=M, K=K, N=N, kind=args.kind, splits=args.splits, variant=args.variant, repeat=rep, knob=knob, units=n)
                if n:
                    r = t[1:1 + 4 * n].reshape(n, 4)
                    cta = (r[:, 0] >> 32).astype(int)
                    tail = ((r[:, 0] >> 31) & 1).astype(bool)
                    t0 = r[:, 1].min()
                    beg, full, end = (r[:, 1] - t0) / 1e3, (r[:, 2] - t0) / 1e3, (r[:, 3] - t0) / 1e3
                    line["span_us"] = round(float(end.max()), 1)
                    for lab, m in (("block", ~tail), ("swapped", tail)):
                        if m.any():
                            d = (full - beg)[m]
                            line[lab] = dict(n=int(m.sum()), main_us=round(float(d.mean()), 2),
                                             main_min_med_max_us=[round(float(np.percentile(d, q)), 1) for q in (0, 50, 100)],
                                             epilogue_us=round(float((end - full)[m].mean()), 2))
                    ends_cta = np.array([end[cta == c].max() for c in np.unique(cta)])
                    line["cta_finish_min_med_max_us"] = [round(float(np.percentile(ends_cta, q)), 1) for q in (0, 50, 100)]
                    cnt = np.bincount(cta)
                    line["units_per_cta"] = {int(k): int(v) for k, v in zip(*np.unique(cnt[cnt > 0], return_counts=True))}
                    if args.detail:
                        ends = np.array([end[cta == c].max() if (cta == c).any() else 0.0 for c in range(cta.max() + 1)])
                        for c in np.argsort(ends)[::-1][:args.detail]:
                            m = cta == c
                            line.setdefault("timelines", {})[int(c)] = [
                                [("S" if tl else "B"), round(float(b), 1), round(float(f), 1), round(float(e), 1)]
                                for tl, b, f, e in sorted(zip(tail[m], beg[m], full[m], end[m]), key=lambda z: z[1])]
                print(json.dumps(line), flush=True)
    finally:
        call("ojb_gemm_set_trace", None, i32(0))
        if probes:
            call("ojb_gemm_set_probe", i32(1), i32(0))
    _lib.check_status(dev)


if __name__ == "__main__":
    main()
