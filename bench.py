"""Benchmark of the prefix-tree scoring forward (64-layer hybrid 27B-scale model, random-init weights, synthetic trees).

    python bench.py --gpus 1 --steps 100 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...
    python bench.py --impl reference          # the reference's PyTorch path on the host cores (bounded sample)
    python bench.py --no-reference-gpu        # skip the leg that times the reference's own CUDA forward on this GPU

A step = one request: the 539-row, 7-candidate tree pushed through the forward + scoring head. Data
parallel: every rank owns a full copy of the weights and its own requests; nothing is exchanged on the data path, the
process group only provides the barrier and the max over ranks of the timed region. Prints one JSON line on rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "open-jev-fast_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

METRIC = "requests/s (539-row 7-candidate tree forward + scoring head, data parallel); ms_per_step = ms/request"
METRIC_OTHER = "requests/s (one tree forward + scoring head per request, tree named in config.workload, data parallel); ms_per_step = ms/request"


def peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def matmul_params(cfg):
    """Matmul weights of one forward (embedding and head excluded): P, and the per-layer-type split."""
    H, I = cfg.hidden_size, cfg.intermediate_size
    KD = cfg.linear_num_key_heads * cfg.linear_key_head_dim
    VD = cfg.linear_num_value_heads * cfg.linear_value_head_dim
    HV = cfg.linear_num_value_heads
    qd = cfg.num_attention_heads * cfg.head_dim
    kvd = cfg.num_key_value_heads * cfg.head_dim
    lin = H * (2 * KD + 2 * VD + 2 * HV) + VD * H
    full = H * (2 * qd + 2 * kvd) + qd * H
    n_lin = sum(t == "linear_attention" for t in cfg.layer_types)
    n_full = len(cfg.layer_types) - n_lin
    return (n_lin + n_full) * 3 * H * I + n_lin * lin + n_full * full


class ClockSampler:
    """nvidia-smi polled every 200 ms while the timed region runs (read-only queries)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm = sorted(float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit())
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[3 + i].lower().startswith("active") for r in self.rows)]
        mx = max(float(r[1]) for r in self.rows if len(r) >= 7)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": mx, "reasons": reasons, "samples": len(sm)}


_CPU_CORE = {}


def cpu_reference_sample(cfg_kwargs, seqs, threads, reps=0):
    """The reference's PyTorch path on the host: one linear-attention decoder layer and one full-attention decoder layer
    (each with its MLP) at full width, bf16 weights, over every candidate path; a forward costs n_lin * t_lin + n_full *
    t_full (the layers of one type do identical work). Returns (t_lin, t_full) in seconds."""
    from ojb200 import modelgen as MG
    from oracle import hf_path as OH
    torch.set_num_threads(threads)
    if "core" not in _CPU_CORE:
        kw = dict(cfg_kwargs)
        kw.update(num_hidden_layers=2, layer_types=["linear_attention", "full_attention"])
        _CPU_CORE["core"] = MG.build_core(MG.make_config(**kw), device="cpu", seed=0, draw_on="cpu")
    return OH.time_layers(_CPU_CORE["core"], seqs, reps=reps)


def workload_name(name, seqs, groups):
    """The same string in both arms: what tree, which graph key (from the host layout builder; no GPU needed)."""
    from ojb200 import layout as PL
    d = PL.gtree_host(seqs, groups, 0, 32, 16, vbits=False)[0]
    return (f"{name} tree: key (N,S,L2)=({d['N']}, {d['S']}, {d['L2']}), real rows {d['Nreal']}, 64-layer hybrid "
            "(48 GDN + 16 gated GQA), hidden 5120, MLP 17408, HV=32")


def reference_on_gpu(args):
    """The reference's own forward_gtree (its CUDA operators rebuilt for sm_100a + cuBLAS) timed on this GPU in a child
    process, before this library's model is built: a fault or a missing build there cannot touch the numbers below."""
    cmd = [sys.executable, "-m", "oracle.ref_forward", "--workload", args.workload, "--steps", "30", "--warmup", "5",
           "--layers", str(args.layers)]
    try:
        r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
        for line in reversed(r.stdout.strip().splitlines()):
            if line.startswith("{"):
                return json.loads(line)
        return {"impl": "reference-gpu", "unavailable": f"no result line (exit code {r.returncode}): {r.stderr[-200:]}"}
    except Exception as e:
        return {"impl": "reference-gpu", "unavailable": f"{type(e).__name__}: {e}"}


def run_reference(args, cfg_kwargs, seqs, groups, n_lin, n_full):
    """`--impl reference`: K timed samples (after W untimed ones) of the reference's PyTorch path on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    times = []
    for i in range(args.warmup + args.steps):
        t_lin, t_full = cpu_reference_sample(cfg_kwargs, seqs, threads)
        if i >= args.warmup:
            times.append(n_lin * t_lin + n_full * t_full)
    sec = sum(times) / len(times)
    v = 1.0 / sec
    sample = (f"Hugging Face qwen3_5 torch path, bf16 weights, {threads} threads: per step 1 linear-attention + 1 full-attention "
              f"decoder layer (with MLP) at full width over the {len(seqs)} candidate paths ({sum(map(len, seqs))} tokens), "
              f"scaled by ({n_lin},{n_full}) layers")
    line = {"metric": METRIC if args.workload == "baseline" else METRIC_OTHER, "value": v, "unit": "requests/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "impl": "reference", "extrapolated": True,
            "config": {"workload": workload_name(args.workload, seqs, groups),
                       "timed": "host cores; one layer of each type timed, scaled to 64 layers"},
            "cpu_baseline": {"value": v, "unit": "requests/s", "cores": threads, "kind": "reference", "sample": sample},
            "e2e": {"value": v, "unit": "requests/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the gate/up GEMM at M = 544, from one ncu capture of the same
# kernel and shape (bytes). Not measured by this run: the line says so in `traffic_source`. The algorithmic bytes are
# weights + x + out = 381.0 MB at M = 544.
TRAFFIC_NCU = {("gemm_block256", 544): 395.3e6, ("gemm_tile128", 544): 389.1e6}


def gemm_roofline(fast, M, pk, pk_kind, dev):
    """Times the dominant kernel — the gate/up GEMM with the SwiGLU epilogue, 64 launches per forward, each streaming its own
    356 MB weight (larger than L2, so no flush is needed between launches) — with CUDA events on the launching stream."""
    from ojb200 import lt_ext as LT
    H = fast.H
    x = torch.randn(M, H, device=dev).to(torch.bfloat16)
    layers = [d for d in fast.L if getattr(d, "fused_mlp", False)]
    for d in layers[:4]:
        fast._mlp_in(x, d)
    best = float("inf")
    for _ in range(3):
        a, b = torch.cuda.Event(True), torch.cuda.Event(True)
        a.record()
        for d in layers:
            fast._mlp_in(x, d)               # the kernel variant the model uses for this row count (FastQwen35.tune)
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) / len(layers))
    N2, Kd = layers[0].w_gu_blk.shape
    flops = 2.0 * M * N2 * Kd
    ach = flops / (best * 1e-3) / 1e12
    peak = pk["bf16_tflops"]
    w_gbs = N2 * Kd * 2 / (best * 1e-3) / 1e9
    N2_, Kd_ = layers[0].w_gu_blk.shape
    idx = fast._plan.get(("gu", M, N2_, Kd_), 0)
    code = LT.VARIANT_BN[idx] if idx else LT.gemm_plan(M, N2_, Kd_, 1)[0]
    kern = {1: "gemm_tile128_kernel<256,4,swiglu>", 2: "gemm_tile128_kernel<128,6,swiglu>"}.get(code, "gemm_block256_kernel<swiglu>")
    return {"bound": "tensor", "kernel": kern + " (gate/up GEMM + SwiGLU, 64 launches per forward)", "achieved": ach, "peak": peak,
            "unit": "TFLOP/s", "frac": ach / peak, "traffic": TRAFFIC_NCU.get((kern.split("_kernel")[0], M)),
            "traffic_source": "one ncu capture of this kernel at this shape (committed summary), not this run", "peak_source": f"{pk_kind} burst bf16", "us_per_launch": best * 1e3,
            "algorithmic_flops_per_launch": flops, "weight_stream_gbs": w_gbs, "hbm_peak_gbs": pk["hbm_gbs"]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="baseline", choices=["baseline", "example"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip timing the reference's own CUDA forward on this GPU")
    ap.add_argument("--profile", type=int, default=0, help="run this many eager (graph-free) forwards between "
                    "cudaProfilerStart/Stop and exit: for `ncu --profile-from-start off`")
    ap.add_argument("--pack", type=int, default=0, help="also time this many requests packed into one forward (extra key "
                    "`packed` of the JSON line; the headline numbers stay one request per forward)")
    ap.add_argument("--fp8", action="store_true", help="run the projections on e4m3 operands (ojb_gemm_e4m3): not the parity "
                    "path, reported with its own dtype and without a roofline entry")
    ap.add_argument("--layers", type=int, default=64, help="debugging only: a run with fewer than 64 layers is not a result")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    from ojb200 import trees
    from ojb200 import modelgen as MG
    cfg_kwargs = dict(MG.FULL)
    cfg_kwargs["num_hidden_layers"] = args.layers
    cfg = MG.make_config(**cfg_kwargs)
    n_lin = sum(t == "linear_attention" for t in cfg.layer_types)
    n_full = args.layers - n_lin
    mk = trees.baseline_tree if args.workload == "baseline" else trees.example_tree
    if args.impl == "reference":
        seqs, groups = mk(0, cfg.vocab_size)
        return run_reference(args, cfg_kwargs, seqs, groups, n_lin, n_full)

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from ojb200 import _lib, fastmodel as FM, server as SV
    pk, pk_kind = peaks()
    ref_gpu = None
    if rank == 0 and world == 1 and not args.no_reference_gpu and not args.profile and not args.fp8:
        ref_gpu = reference_on_gpu(args)

    core = MG.build_core(cfg, device=dev, seed=0)
    fast = FM.FastQwen35(core, free_original=True, fp8=args.fp8)
    W, b = MG.make_head(cfg.hidden_size, A=1, seed=1, device=dev)
    scorer = SV.Scorer(fast, W, b, pad_id=0, device=dev)
    # every rank serves its own requests: different seeds, same shape (weak scaling: fixed work per GPU)
    reqs = [mk(1000 * rank + i, cfg.vocab_size) for i in range(4)]
    out = scorer.score_tokens(*reqs[0])          # captures the graph for this key (not timed)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    assert bool(torch.isfinite(out).all()), "non-finite scores"
    # scores of the tree the reference-on-GPU leg runs (seed 0), for the cross-check in the result line
    ref_scores_ours = scorer.score_tokens(*mk(0, cfg.vocab_size)).float().cpu() if ref_gpu is not None else None
    key = scorer.last["key"]
    ent = scorer.graphs[key]

    if args.profile > 0:
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for _ in range(args.profile):
            fast.score_gtree(ent.ids, ent.lay, W, b)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled_forwards": args.profile, "key": key}), flush=True)
        return

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed: inputs resident in HBM, K graph replays between two events
    for _ in range(args.warmup):
        ent.replay()
    barrier()
    with ClockSampler(local) as clocks:
        e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
        per = []
        e0.record()
        for _ in range(args.steps):
            a, c = torch.cuda.Event(True), torch.cuda.Event(True)
            a.record(); ent.replay(); c.record()
            per.append((a, c))
        e1.record()
        barrier()
        total_ms = e0.elapsed_time(e1)
        # ---- end to end through Scorer.forward-level API: host layout build + pinned H2D + replay + D2H of the scores
        for i in range(args.warmup):
            scorer.score_tokens(*reqs[i % len(reqs)]).cpu()
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            s_host = scorer.score_tokens(*reqs[i % len(reqs)]).cpu()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
    _lib.check_status(dev)
    steps_ms = sorted(a.elapsed_time(c) for a, c in per)
    if world > 1:
        t = torch.tensor([total_ms, e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_s = float(t[0]), float(t[1])
    ms_per_step = total_ms / args.steps

    packed = None
    if args.pack > 1 and rank == 0:
        # several requests per forward (Scorer.score_packed): end to end, host layout + H2D + replay + D2H inside the region
        group = [reqs[i % len(reqs)] for i in range(args.pack)]
        for _ in range(max(args.warmup, 2)):
            [o.cpu() for o in scorer.score_packed(group)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            outs = [o.cpu() for o in scorer.score_packed(group)]
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        packed = {"requests_per_forward": args.pack, "rows": scorer.last["rows"], "ms_per_forward": dt / args.steps * 1e3,
                  "value": args.pack * args.steps / dt, "unit": "requests/s", "h2d_bytes_per_forward": scorer.last["h2d_bytes"]}
        _lib.check_status(dev)

    roof = gemm_roofline(fast, key[0], pk, pk_kind, dev) if rank == 0 and not args.fp8 else None
    P = matmul_params(cfg)
    line = {"metric": METRIC if args.workload == "baseline" else METRIC_OTHER, "value": world * 1e3 / ms_per_step, "unit": "requests/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "e4m3 projections with per-row scales, bf16 elsewhere (outside the bf16 parity tolerance)" if args.fp8 else "bf16",
            "data": "synthetic",
            "config": {"workload": workload_name(args.workload, *mk(0, cfg.vocab_size)),
                       "layers": args.layers, "parallelism": f"dp{world}", "l2": "inputs larger than L2 (46 GB of weights per step)",
                       "timing": "CUDA events around K graph replays, max over ranks"},
            "ms_per_request_p50": steps_ms[len(steps_ms) // 2],
            "e2e": {"value": world * args.steps / e2e_s, "unit": "requests/s", "ms_per_request": e2e_s / args.steps * 1e3,
                    "h2d_bytes_per_step": scorer.last["h2d_bytes"], "d2h_bytes_per_step": int(s_host.numel() * 4),
                    "host_layout_ms": scorer.last["build_ms"]},
            "gpu_launches": ent.launches * args.steps, "launches_per_step": ent.launches,
            "clocks": clocks.summary(), "roofline": roof,
            "model": {"matmul_params": P, "gemm_tflop_per_step": 2.0 * key[0] * P / 1e12,
                      "gemm_floor_ms_at_peak": 2.0 * key[0] * P / (pk["bf16_tflops"] * 1e12) * 1e3,
                      "weight_floor_ms": 2.0 * P / (pk["hbm_gbs"] * 1e9) * 1e3}}
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            t_lin, t_full = cpu_reference_sample(cfg_kwargs, reqs[0][0], threads, reps=1)
            sec = n_lin * t_lin + n_full * t_full
            line["cpu_baseline"] = {"value": 1.0 / sec, "unit": "requests/s", "cores": threads, "kind": "reference",
                                    "sample": f"Hugging Face qwen3_5 torch path (bf16, {threads} threads): 1 linear-attention + 1 "
                                              f"full-attention decoder layer over the {len(reqs[0][0])} candidate paths, "
                                              f"x({n_lin},{n_full}); {sec:.1f} s per request"}
        else:
            line["cpu_baseline"] = None
        if packed is not None:
            line["packed"] = packed
        if ref_gpu is not None:
            # the reference's own forward (its CUDA operators + cuBLAS) on this GPU, same weights, same tree, CUDA graph replay
            line["reference_gpu"] = ref_gpu
            line["reference_gpu_ms"] = ref_gpu.get("ms_per_request_p50")
            if ref_gpu.get("scores") is not None:
                line["reference_gpu"]["max_abs_score_diff_vs_ours"] = float(
                    (torch.tensor(ref_gpu["scores"]) - ref_scores_ours.flatten()).abs().max())
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
