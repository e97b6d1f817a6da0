"""GEMM surface of open-jev-fast's src/lt_ext.py / src/lt.cpp, backed by the tcgen05 GEMM of libojb200.so.

The reference enumerates cuBLASLt algorithms per shape (lt_setup) and runs one by index (lt_matmul); split-K plans go
through lt2_*. Here an "algorithm" is one of the library's GEMM variants: index 0 lets the library choose, 1 / 2 force the
128-row tile kernel with 256 / 128-wide tiles, 3 the 256-row block kernel with automatic w-tile width, 4..6 that kernel
with w-tile width 256, 192, 128, 7 that kernel with all of x in swapped-operand units (M <= 2048), 8 / 9 the CTA-pair
kernel (tcgen05.mma.cta_group::2) with automatic width / all of x in swapped-operand units, 10 the block kernel with
block units for all but the last full block of x and two swapped-operand chunks for the remaining 257..511 rows.
Two entry points have no counterpart in the reference: gemm_swiglu (SwiGLU fused into the epilogue) and gemm_splitk
(fp32 partial sums from the un-split [N, K] weight).
"""
import ctypes
import sys

import torch

from . import _lib
from ._lib import call, i32, i64, ptr, stream_ptr

bf16 = torch.bfloat16
VARIANT_BN = [0, 1, 2, 3, 256, 192, 128, 4, 5, 6, 7]
N_VARIANTS = len(VARIANT_BN)
SM_COUNT = 148
_plans = []          # lt2 plans: dicts
_wl1_cache = {}      # data_ptr of a [S, K/S, N] weight -> its [N, K] re-layout


def load():
    """Counterpart of src/lt_ext.py:5 load()."""
    _lib.lib()
    return sys.modules[__name__]


def _check(x, w):
    if not (x.is_cuda and w.is_cuda and x.is_contiguous() and w.is_contiguous() and x.dtype == bf16 and w.dtype == bf16):
        raise RuntimeError("lt_matmul: x and w must be contiguous CUDA bf16 tensors")
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise RuntimeError("lt_matmul: x [M, K] and w [N, K] expected")


def lt_setup(M, N, K, max_algos):
    """src/lt.cpp:15 — number of candidate algorithms for (M, N, K)."""
    return min(int(max_algos), N_VARIANTS)


def lt_matmul(x, w, idx):
    """src/lt.cpp:43 — out[M, N] = x[M, K] @ w[N, K]^T (bf16, fp32 accumulate)."""
    _check(x, w)
    if not 0 <= idx < N_VARIANTS:
        raise RuntimeError("lt_matmul: algorithm index out of range")
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty(M, N, dtype=bf16, device=x.device)
    call("ojb_gemm_bf16", ptr(x), ptr(w), ptr(out), i64(M), i64(N), i64(K), i32(VARIANT_BN[idx]), ptr(_lib.status_word(x.device)),
         stream_ptr())
    return out


def gemm_swiglu(x, w_blk, idx=0):
    """out[M, I] = silu(x @ gate^T) * (x @ up^T) with w_blk = block-interleaved [2I, K] weight (see interleave_gate_up)."""
    _check(x, w_blk)
    M, K = x.shape
    N = w_blk.shape[0]
    out = torch.empty(M, N // 2, dtype=bf16, device=x.device)
    call("ojb_gemm_bf16_swiglu_v", ptr(x), ptr(w_blk), ptr(out), i64(M), i64(N), i64(K), i32(VARIANT_BN[idx]),
         ptr(_lib.status_word(x.device)), stream_ptr())
    return out


def interleave_gate_up(w_gate, w_up, block=128):
    """[I, K] gate and up weights -> [2I, K] in blocks of `block` gate rows followed by their up rows (I % 128 == 0)."""
    I, K = w_gate.shape
    if I % 128:
        raise RuntimeError("interleave_gate_up: I must be a multiple of 128")
    return torch.stack([w_gate.view(I // block, block, K), w_up.view(I // block, block, K)], 1).reshape(2 * I, K).contiguous()


def gemm_plan(M, N, K, kind, max_splits=16):
    """(variant code, K ranges, modelled microseconds) that the library's cost model picks for a shape; kind = 0 bf16
    output, 1 SwiGLU-fused, 2 fp32 split-K partials. Host arithmetic only."""
    v, s, us = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_float()
    call("ojb_gemm_plan", i64(M), i64(N), i64(K), i32(kind), i32(max_splits), ctypes.byref(v), ctypes.byref(s), ctypes.byref(us))
    return v.value, s.value, us.value


def plan_splitk(M, N, K, sms=SM_COUNT):
    """Number of K ranges for a projection whose output goes through the partial-sum reduction (residual + RMSNorm kernel)."""
    return gemm_plan(M, N, K, 2)[1]


def gemm_splitk(x, w, S, idx=0):
    """fp32 partials [S, M, N] of x @ w^T over S K ranges of ceil(K/64/S) k-blocks; w stays [N, K]."""
    _check(x, w)
    M, K = x.shape
    N = w.shape[0]
    parts = torch.empty(S, M, N, dtype=torch.float32, device=x.device)
    call("ojb_gemm_bf16_splitk", ptr(x), ptr(w), ptr(parts), i64(M), i64(N), i64(K), i32(S), i32(VARIANT_BN[idx]),
         ptr(_lib.status_word(x.device)), stream_ptr())
    return parts


# ---------------------------------------------------------------------------------------------- lt2_* (src/lt.cpp:64-190)
def quantize_weight_e4m3(w):
    """Offline weight preparation of the 8-bit path: w [N, K] bf16 -> (e4m3 bytes [N, K] as uint8, fp32 scale per row), scale =
    max|row| / 448. Plain torch: this runs once per weight, not in the forward."""
    wf = w.float()
    s = wf.abs().amax(dim=1).clamp_min(1e-30) / 448.0
    q = (wf / s[:, None]).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).contiguous(), s.contiguous()


def quantize_rows_e4m3(x):
    """x [M, K] bf16 -> (e4m3 bytes [M, K] uint8, fp32 scale [M]) through ojb_quantize_rows_e4m3 (one kernel)."""
    if not (x.is_cuda and x.is_contiguous() and x.dtype == bf16 and x.dim() == 2):
        raise RuntimeError("quantize_rows_e4m3: contiguous CUDA bf16 [M, K] expected")
    M, K = x.shape
    q = torch.empty(M, K, dtype=torch.uint8, device=x.device)
    s = torch.empty(M, dtype=torch.float32, device=x.device)
    call("ojb_quantize_rows_e4m3", ptr(x), ptr(q), ptr(s), i64(M), i64(K), stream_ptr())
    return q, s


def gemm_e4m3(xq, sx, wq, sw, kind=0, splits=1):
    """out = (xq @ wq^T) * sx[:, None] * sw[None, :] on e4m3 operands (ojb_gemm_e4m3). kind 0: bf16 [M, N]; 1: SwiGLU on the
    re-laid gate/up weight -> bf16 [M, N/2]; 2: fp32 partials [splits, M, N]."""
    for t, dt in ((xq, torch.uint8), (wq, torch.uint8), (sx, torch.float32), (sw, torch.float32)):
        if not (t.is_cuda and t.is_contiguous() and t.dtype == dt):
            raise RuntimeError("gemm_e4m3: contiguous CUDA uint8 operands and fp32 scales expected")
    M, K = xq.shape
    N = wq.shape[0]
    if wq.shape[1] != K or sx.numel() != M or sw.numel() != N:
        raise RuntimeError("gemm_e4m3: shapes do not match")
    if kind == 0:
        out = torch.empty(M, N, dtype=bf16, device=xq.device)
    elif kind == 1:
        out = torch.empty(M, N // 2, dtype=bf16, device=xq.device)
    else:
        out = torch.empty(splits, M, N, dtype=torch.float32, device=xq.device)
    call("ojb_gemm_e4m3", ptr(xq), ptr(sx), ptr(wq), ptr(sw), ptr(out), i64(M), i64(N), i64(K), i32(kind), i32(splits),
         ptr(_lib.status_word(xq.device)), stream_ptr())
    return out


def lt2_plan(M, N, K, S, f32, wl):
    """src/lt.cpp:64 — plan handle. wl = 0: w [N, K]; wl = 1: w [S, K/S, N] (the reference's pre-split layout)."""
    if wl not in (0, 1) or (wl == 0 and S != 1 and False):
        raise RuntimeError("lt2_plan: wl must be 0 or 1")
    _plans.append(dict(M=M, N=N, K=K, S=S, f32=bool(f32), wl=wl))
    return len(_plans) - 1


def lt2_search(h, max_cands, min_waves):
    """src/lt.cpp:93 — number of candidates of plan h."""
    return N_VARIANTS


def lt2_info(h, i):
    """src/lt.cpp:170 — description of candidate i."""
    return f"tcgen05 GEMM variant code {VARIANT_BN[i]}, plan {_plans[h]}"


def lt2_run(h, x, w, i):
    """src/lt.cpp:160 — [S, M, N] partial products (fp32 if the plan says so, else bf16)."""
    p = _plans[h]
    if p["wl"] == 1:
        key = (w.data_ptr(), tuple(w.shape))
        w2 = _wl1_cache.get(key)
        if w2 is None:
            S, Ks, N = w.shape
            w2 = _wl1_cache[key] = w.permute(2, 0, 1).reshape(N, S * Ks).contiguous()
        w = w2
    parts = gemm_splitk(x, w, p["S"], i)
    return parts if p["f32"] else parts.to(bf16)


def lt2_raw(h, i):
    """src/lt.cpp:179 — opaque algorithm bytes; here the variant index."""
    return [int(i)]


def lt2_add_raw(h, raw):
    """src/lt.cpp:183 — register an algorithm from lt2_raw; returns its index."""
    return int(raw[0])
