"""Operator surface of open-jev-fast's src/ext.py, backed by libojb200.so through the C ABI.

Names, positional argument order, dtypes and returned shapes follow the prototypes in the reference's src/ext.py:6-45,
so code written against `K = ext.load()` keeps working. Outputs are allocated here with torch.empty on the inputs' device
(the C layer allocates nothing) and every launch goes to torch's current stream, so the ops can be captured in CUDA graphs.
Variants that the reference keeps for history (v1 / map / dedup / fused3..9) map onto the one implementation that honours
their layout contract.
"""
import sys

import torch

from . import _lib
from ._lib import call, f32, i32, i64, ptr, stream_ptr

bf16 = torch.bfloat16


def load(verbose=False):
    """Counterpart of src/ext.py:47 load(): returns the op namespace (this module). Raises if the library is missing."""
    _lib.lib()
    return sys.modules[__name__]


def _chk(*ts):
    _lib.need_cuda_bf16(*ts)


# ------------------------------------------------------------------------------------------------ norms / activations
def add_rmsnorm(x, delta, w1, rowmask, eps):
    """src/ext.py:6 — returns [h, hn]; without delta, h is x itself (src/kernels.cu:761)."""
    _chk(x, delta, w1, rowmask)
    N, H = x.shape
    hn = torch.empty_like(x)
    h = x if delta is None else torch.empty_like(x)
    call("ojb_add_rmsnorm", ptr(x), ptr(delta), ptr(w1), ptr(rowmask), ptr(None if delta is None else h), ptr(hn),
         i64(N), i64(H), f32(eps), stream_ptr())
    return [h, hn]


def add_rmsnorm_sk(x, parts, w1, rowmask, eps):
    """src/ext.py:15 / :29 — parts fp32 [S, N, H] (bf16 partials are widened first), returns [h, hn]."""
    if parts.dtype != torch.float32:
        parts = parts.float()
    _chk(x, parts, w1, rowmask)
    N, H = x.shape
    S = parts.shape[0]
    if tuple(parts.shape[1:]) != (N, H):
        raise RuntimeError("add_rmsnorm_sk: parts must be [S, N, H]")
    h, hn = torch.empty_like(x), torch.empty_like(x)
    call("ojb_add_rmsnorm_sk", ptr(x), ptr(parts), i32(S), ptr(w1), ptr(rowmask), ptr(h), ptr(hn), i64(N), i64(H),
         f32(eps), stream_ptr())
    return [h, hn]


add_rmsnorm_sk2 = add_rmsnorm_sk


def act_tables(like):
    """src/ext.py:23 — [silu_tab bf16[65536], sig_tab f32[65536]] on like's device."""
    silu_tab = torch.empty(65536, dtype=bf16, device=like.device)
    sig_tab = torch.empty(65536, dtype=torch.float32, device=like.device)
    call("ojb_act_tables", ptr(silu_tab), ptr(sig_tab), stream_ptr())
    return [silu_tab, sig_tab]


def silu_mul(gu):
    """src/ext.py:7 — gu [N, 2I] -> [N, I]."""
    _chk(gu)
    N, I2 = gu.shape
    out = torch.empty(N, I2 // 2, dtype=bf16, device=gu.device)
    call("ojb_silu_mul", ptr(gu), ptr(None), ptr(out), i64(N), i64(I2 // 2), stream_ptr())
    return out


def silu_mul_lut(gu, tab):
    """src/ext.py:24 — same through the 65536-entry table of act_tables (bit-identical)."""
    _chk(gu, tab)
    N, I2 = gu.shape
    out = torch.empty(N, I2 // 2, dtype=bf16, device=gu.device)
    call("ojb_silu_mul", ptr(gu), ptr(tab), ptr(out), i64(N), i64(I2 // 2), stream_ptr())
    return out


def _gate_mul(att, gate, T, HQ, D):
    # att [B, HQ, T, D] with unit stride in D; gate [B*T, HQ*D]
    if att.dim() != 4 or att.stride(3) != 1 or att.shape[1] != HQ or att.shape[2] != T or att.shape[3] != D:
        raise RuntimeError("gate_mul: att must be [B, HQ, T, D] with unit stride along D")
    _chk(gate)
    out = torch.empty_like(gate)
    B = att.shape[0]
    es = att.element_size()
    for b in range(B):
        a_ptr = _lib.ctypes.c_void_p(att.data_ptr() + b * att.stride(0) * es)
        g_ptr = _lib.ctypes.c_void_p(gate.data_ptr() + b * T * HQ * D * es)
        o_ptr = _lib.ctypes.c_void_p(out.data_ptr() + b * T * HQ * D * es)
        call("ojb_gate_mul", a_ptr, i64(att.stride(2)), i64(att.stride(1)), g_ptr, o_ptr, i64(T), i64(HQ), i64(D),
             stream_ptr())
    return out


def gate_mul(att, gate, T, HQ, D):
    """src/ext.py:11."""
    return _gate_mul(att, gate, T, HQ, D)


def gate_mul2(att, gate, T, HQ, D):
    """src/ext.py:14."""
    return _gate_mul(att, gate, T, HQ, D)


def gate_mul3(att, gate, sig, T, HQ, D):
    """src/ext.py:28 — strided att; the sigmoid is computed (same bits as the table)."""
    return _gate_mul(att, gate, T, HQ, D)


def pack_bits(vis):
    """src/ext.py:40 — bool [N, N] -> int32 [N, N/32]."""
    _chk(vis)
    N = vis.shape[0]
    if vis.dtype not in (torch.bool, torch.uint8) or vis.shape[1] != N or N % 32:
        raise RuntimeError("pack_bits: vis must be bool [N, N] with N % 32 == 0")
    out = torch.empty(N, N // 32, dtype=torch.int32, device=vis.device)
    call("ojb_pack_bits", ptr(vis), ptr(out), i64(N), stream_ptr())
    return out


# ------------------------------------------------------------------------------------------------ full attention
def fullattn_prep2(proj, qw1, kw1, cosb, sinb, B, T, HQ, HKV, D, eps):
    """src/ext.py:13 — returns [qt [B,HQ,T,D], kt [B,HKV,T,D], vt [B,HKV,T,D], gate [B*T, HQ*D]]."""
    _chk(proj, qw1, kw1, cosb, sinb)
    N = B * T
    RD = cosb.shape[-1]
    if proj.shape != (N, HQ * 2 * D + 2 * HKV * D):
        raise RuntimeError("fullattn_prep: proj must be [B*T, 2*HQ*D + 2*HKV*D]")
    dev = proj.device
    qt = torch.empty(B, HQ, T, D, dtype=bf16, device=dev)
    kt = torch.empty(B, HKV, T, D, dtype=bf16, device=dev)
    vt = torch.empty(B, HKV, T, D, dtype=bf16, device=dev)
    gate = torch.empty(N, HQ * D, dtype=bf16, device=dev)
    cosb = cosb.reshape(N, RD)
    sinb = sinb.reshape(N, RD)
    for b in range(B):
        sl = slice(b * T, (b + 1) * T)
        call("ojb_fullattn_prep", ptr(proj[sl]), ptr(qw1), ptr(kw1), ptr(cosb[sl]), ptr(sinb[sl]), ptr(qt[b]), ptr(kt[b]),
             ptr(vt[b]), ptr(gate[sl]), i64(T), i64(HQ), i64(HKV), i64(D), i64(RD), f32(eps), stream_ptr())
    return [qt, kt, vt, gate]


fullattn_prep = fullattn_prep2   # src/ext.py:10 — same contract
