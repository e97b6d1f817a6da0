"""GEMM sweep over the projection shapes of the model for every kernel variant.

    python bench_gemm_sweep.py [--m 64 288 544 1024 4096] [--quick]

For each (M, K, N): plain bf16 GEMM per tile variant, the SwiGLU-fused GEMM where N is a gate/up width, and split-K partial
GEMMs (with their reduce + residual + RMSNorm kernel) where N is the hidden size. Each case is timed with CUDA events over
launches that cycle through enough distinct weight copies to exceed the L2, checked against torch.matmul on fp32-upcast
operands, and printed as one JSON line: microseconds, TFLOP/s, fraction of the measured bf16 peak, weight-stream GB/s.
With --sustained SECS every case runs back to back for SECS seconds and the line also carries the board power, the SM clock
and the energy per call (NVML).
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "open-jev-fast_b200"))
from ojb200 import ext as K
from ojb200 import lt_ext as LT

bf16 = torch.bfloat16
SHAPES = [(5120, 12288), (5120, 12352), (5120, 14336), (5120, 34816), (17408, 5120), (6144, 5120), (4096, 5120)]


def _peak():
    p = os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")
    try:
        return json.load(open(p))["bf16_tflops"]
    except Exception:
        return 1590.0


SUSTAINED = 0.0      # --sustained: seconds of back-to-back launches per case, with board power and SM clock sampled
_LAST = {}           # power / clock / energy of the case timed last (sustained mode)


def _time_sustained(fns, secs):
    """Back-to-back launches for `secs` seconds (the GPU settles against its power cap, as inside a forward), NVML samples of
    board power and SM clock every 20 ms; the first third of the samples is dropped. Returns microseconds per call."""
    import threading
    import time
    import pynvml
    pynvml.nvmlInit()
    hd = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
    for f in fns[:2]:
        f()
    torch.cuda.synchronize()
    stop, samples = threading.Event(), []

    def sample():
        while not stop.is_set():
            samples.append((pynvml.nvmlDeviceGetPowerUsage(hd) / 1e3, pynvml.nvmlDeviceGetClockInfo(hd, pynvml.NVML_CLOCK_SM)))
            time.sleep(0.02)
    th = threading.Thread(target=sample)
    th.start()
    a, b = torch.cuda.Event(True), torch.cuda.Event(True)
    n, t0 = 0, time.perf_counter()
    a.record()
    while time.perf_counter() - t0 < secs:
        for _ in range(8):
            for f in fns:
                f()
        n += 8 * len(fns)
        torch.cuda.synchronize()
    b.record()
    torch.cuda.synchronize()
    stop.set()
    th.join()
    us = a.elapsed_time(b) * 1e3 / n
    samples = samples[len(samples) // 3:] or [(0.0, 0)]
    watts = sum(x[0] for x in samples) / len(samples)
    _LAST.clear()
    _LAST.update(watts=round(watts), sm_mhz=round(sum(x[1] for x in samples) / len(samples)), mj_per_call=round(watts * us / 1e3, 1))
    return us


def _time(fns, reps=3):
    """fns: list of closures over distinct weight copies; returns microseconds per call (best of reps passes)."""
    if SUSTAINED > 0:
        return _time_sustained(fns, SUSTAINED)
    for f in fns[:2]:
        f()
    best = float("inf")
    for _ in range(reps):
        a, b = torch.cuda.Event(True), torch.cuda.Event(True)
        a.record()
        for f in fns:
            f()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) * 1e3 / len(fns))
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, nargs="+", default=[64, 288, 539, 544, 1024, 4096])
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--shape", type=int, nargs=2, default=None, metavar=("K", "N"), help="only this weight shape")
    ap.add_argument("--only", default=None, help="only kernels whose name starts with this (plain, swiglu, splitk)")
    ap.add_argument("--library", action="store_true",
                    help="also time torch.nn.functional.linear (cuBLASLt, the GEMM path of the reference) on the same operands: a comparator only")
    ap.add_argument("--e4m3", action="store_true",
                    help="also time the 8-bit form (ojb_gemm_e4m3: bf16 out, SwiGLU where N is a gate/up width, fp32 partials where N is "
                         "the hidden size) and the row quantisation kernel")
    ap.add_argument("--sustained", type=float, default=0.0, metavar="SECS",
                    help="time every case over SECS seconds of back-to-back launches and report board power, SM clock and "
                    "energy per call (the GPU runs against its power cap, as it does inside a forward)")
    ap.add_argument("--copies", type=int, default=0, help="distinct weight copies to cycle through (default: enough to exceed L2)")
    args = ap.parse_args()
    global SUSTAINED
    SUSTAINED = args.sustained
    dev = torch.device("cuda")
    peak = _peak()
    g = torch.Generator(device=dev).manual_seed(0)
    want = lambda name: args.only is None or name.startswith(args.only)
    for Kd, N in ([tuple(args.shape)] if args.shape else SHAPES):
        copies = args.copies or max(2, min(8, int(300e6 // (N * Kd * 2)) + 1))      # > 126 MB of distinct weights in flight
        ws = [(torch.randn(N, Kd, generator=g, device=dev) * 0.02).to(bf16) for _ in range(copies)]
        for M in args.m:
            x = torch.randn(M, Kd, generator=g, device=dev).to(bf16)
            ref = x.float() @ ws[0].float().t()
            flops = 2.0 * M * N * Kd

            def report(name, us, err):
                print(json.dumps({"M": M, "K": Kd, "N": N, "kernel": name, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                                  "frac_of_peak": round(flops / us / 1e6 / peak, 3), "weight_gbs": round(N * Kd * 2 / us / 1e3, 1),
                                  "max_err": err, **_LAST}), flush=True)
            for v in ((0, 1, 2, 3, 7, 8, 9) if want("plain") else ()):
                if v == 7 and M > 2048:
                    continue
                out = LT.lt_matmul(x, ws[0], v)
                err = (out.float() - ref).abs().max().item()
                report(f"plain v{v}", _time([lambda w=w, v=v: LT.lt_matmul(x, w, v) for w in ws]), err)
            if args.library:
                out = torch.nn.functional.linear(x, ws[0])
                report("library F.linear", _time([lambda w=w: torch.nn.functional.linear(x, w) for w in ws]),
                       (out.float() - ref).abs().max().item())
            if args.e4m3 and want("e4m3"):
                xq, sx = LT.quantize_rows_e4m3(x)
                q8 = [LT.quantize_weight_e4m3(w) for w in ws]
                deq = xq.view(torch.float8_e4m3fn).float() * sx[:, None]
                ref8 = deq @ (q8[0][0].view(torch.float8_e4m3fn).float() * q8[0][1][:, None]).t()
                out = LT.gemm_e4m3(xq, sx, q8[0][0], q8[0][1], 0)
                report("e4m3 plain", _time([lambda q=q: LT.gemm_e4m3(xq, sx, q[0], q[1], 0) for q in q8]),
                       (out.float() - ref8).abs().max().item())
                if N == 5120:
                    for S in (2, 3, 4):
                        parts = LT.gemm_e4m3(xq, sx, q8[0][0], q8[0][1], 2, S)
                        report(f"e4m3 splitk S{S}", _time([lambda q=q, S=S: LT.gemm_e4m3(xq, sx, q[0], q[1], 2, S) for q in q8]),
                               (parts.sum(0) - ref8).abs().max().item())
                if N % 256 == 0 and Kd == 5120 and N > 20000:
                    # (timing only: the rows are not interleaved here; tests/test_gemm_gpu.py checks the SwiGLU values)
                    report("e4m3 swiglu", _time([lambda q=q: LT.gemm_e4m3(xq, sx, q[0], q[1], 1) for q in q8]), None)
                report("e4m3 quantize rows", _time([lambda: LT.quantize_rows_e4m3(x) for _ in range(8)]), None)
                del q8, deq, ref8
            if N % 256 == 0 and Kd == 5120 and N > 20000 and want("swiglu"):
                I = N // 2
                wb = [LT.interleave_gate_up(w[:I], w[I:]) for w in ws]
                out = LT.gemm_swiglu(x, wb[0])
                gg, uu = ref[:, :I].to(bf16).float(), ref[:, I:].to(bf16).float()
                err = (out.float() - torch.nn.functional.silu(gg).to(bf16).float() * uu).abs().max().item()
                report("swiglu", _time([lambda w=w: LT.gemm_swiglu(x, w) for w in wb]), err)
                for v in (1, 3, 7):
                    if v == 7 and M > 2048:
                        continue
                    report(f"swiglu v{v}", _time([lambda w=w, v=v: LT.gemm_swiglu(x, w, v) for w in wb]), err)
                wb64 = [LT.interleave_gate_up(w[:I], w[I:], 64) for w in ws]      # layout of the CTA-pair kernel
                err64 = (LT.gemm_swiglu(x, wb64[0], 8).float() - torch.nn.functional.silu(gg).to(bf16).float() * uu).abs().max().item()
                report("swiglu v8", _time([lambda w=w: LT.gemm_swiglu(x, w, 8) for w in wb64]), err64)
                del wb64
                err9 = (LT.gemm_swiglu(x, wb[0], 9).float() - torch.nn.functional.silu(gg).to(bf16).float() * uu).abs().max().item()
                report("swiglu v9", _time([lambda w=w: LT.gemm_swiglu(x, w, 9) for w in wb]), err9)
            if N == 5120 and not args.quick and want("splitk"):
                h = torch.randn(M, N, generator=g, device=dev).to(bf16)
                w1 = torch.ones(N, device=dev)
                plan = LT.plan_splitk(M, N, Kd)
                for S in sorted({1, 2, 3, 4, 6, plan}):
                    for v in (0, 1, 3, 7, 8, 9):
                        if v == 7 and M > 2048:
                            continue
                        parts = LT.gemm_splitk(x, ws[0], S, v)
                        err = (parts.sum(0) - ref).abs().max().item()
                        report(f"splitk S{S}{'*' if S == plan else ''} v{v}", _time([lambda w=w, S=S, v=v: LT.gemm_splitk(x, w, S, v) for w in ws]), err)
                        report(f"splitk S{S}{'*' if S == plan else ''} v{v} + reduce/norm",
                               _time([lambda w=w, S=S, v=v: K.add_rmsnorm_sk2(h, LT.gemm_splitk(x, w, S, v), w1, None, 1e-6) for w in ws]), err)
        del ws
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
