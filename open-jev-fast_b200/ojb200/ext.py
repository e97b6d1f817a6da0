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


def resnorm_f32(h, x_init, delta, parts, w1, rowmask, eps):
    """Residual add + RMSNorm on an fp32 residual stream (ojb_resnorm_f32): h fp32 [N, H] is updated in place with
    x_init (bf16 rows that start the stream), the sum of the fp32 partial planes `parts` [S, N, H] or a bf16 `delta`
    (at most one of the three), and the bf16 norm output hn is returned. Same place in the forward as the reference's
    add_rmsnorm / add_rmsnorm_sk2 (src/fastmodel.py:196-203), without their bf16 roundings of the stream."""
    _chk(h, x_init, delta, parts, w1, rowmask)
    N, H = h.shape
    if h.dtype != torch.float32 or (parts is not None and (parts.dtype != torch.float32 or tuple(parts.shape[1:]) != (N, H))):
        raise RuntimeError("resnorm_f32: h must be fp32 [N, H] and parts fp32 [S, N, H]")
    hn = torch.empty(N, H, dtype=bf16, device=h.device)
    call("ojb_resnorm_f32", ptr(h), ptr(x_init), ptr(delta), ptr(parts), i32(0 if parts is None else parts.shape[0]), ptr(w1),
         ptr(rowmask), ptr(hn), i64(N), i64(H), f32(eps), stream_ptr())
    return hn


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
def fullattn_prep2(proj, qw1, kw1, cosb, sinb, B, T, HQ, HKV, D, eps, with_vt_t=False):
    """src/ext.py:13 — returns [qt [B,HQ,T,D], kt [B,HKV,T,D], vt [B,HKV,T,D], gate [B*T, HQ*D]]; with_vt_t=True appends V with
    keys contiguous, [B, HKV, D, T] (operand layout of fattn_tree_tc)."""
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
    vt_t = torch.empty(B, HKV, D, T, dtype=bf16, device=dev) if with_vt_t else None
    cosb = cosb.reshape(N, RD)
    sinb = sinb.reshape(N, RD)
    for b in range(B):
        sl = slice(b * T, (b + 1) * T)
        call("ojb_fullattn_prep", ptr(proj[sl]), ptr(qw1), ptr(kw1), ptr(cosb[sl]), ptr(sinb[sl]), ptr(qt[b]), ptr(kt[b]),
             ptr(vt[b]), ptr(None if vt_t is None else vt_t[b]), ptr(gate[sl]), i64(T), i64(HQ), i64(HKV), i64(D), i64(RD),
             f32(eps), stream_ptr())
    return [qt, kt, vt, gate] + ([vt_t] if with_vt_t else [])


fullattn_prep = fullattn_prep2   # src/ext.py:10 — same contract


# ------------------------------------------------------------------------------------------------ Gated DeltaNet
def _prep(proj, hist, rep_ptr, rep_pos, n_out, convw, A_log, dt_bias, KD, VD, HV, HK, HD, l2norm=True):
    _chk(proj, hist, rep_ptr, rep_pos, convw, A_log, dt_bias)
    if HD != 128 or HK * HD != KD or HV * HD != VD or convw.shape[1] != 4:
        raise RuntimeError("linattn_prep: head dim must be 128 and the conv width 4")
    if any(t.dtype != bf16 for t in (proj, convw, A_log, dt_bias)) or A_log.numel() != HV or dt_bias.numel() != HV:
        # the reference reads these through bf16 pointers without a check (src/kernels.cu:1173-1283); fp32 parameters would
        # be misread silently
        raise RuntimeError("linattn_prep: proj, convw, A_log [HV] and dt_bias [HV] must be bf16")
    N = proj.shape[0]
    if proj.shape[1] != 2 * KD + 2 * VD + 2 * HV or hist.shape != (N + 1, 4) or hist.dtype != torch.int32:
        raise RuntimeError("linattn_prep: proj must be [N, 2KD+2VD+2HV] and hist int32 [N+1, 4]")
    dev = proj.device
    q = torch.empty(n_out, KD, dtype=bf16, device=dev)
    k = torch.empty(n_out, KD, dtype=bf16, device=dev)
    v = torch.empty(n_out, VD, dtype=bf16, device=dev)
    g = torch.empty(n_out, HV, dtype=torch.float32, device=dev)
    beta = torch.empty(n_out, HV, dtype=bf16, device=dev)
    call("ojb_gdn_prep", ptr(proj), ptr(hist), ptr(rep_ptr), ptr(rep_pos), i64(0 if rep_pos is None else rep_pos.numel()),
         ptr(convw), ptr(A_log), ptr(dt_bias), ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), i64(N), i64(KD), i64(VD),
         i64(HV), i64(HK), i32(1 if l2norm else 0), stream_ptr())
    return q, k, v, g, beta


def _expand(x, HK, HV, HD):
    return x.view(-1, HK, 1, HD).expand(-1, HK, HV // HK, HD).reshape(-1, HV * HD).contiguous()


def linattn_prep_rows(proj, hist, convw, A_log, dt_bias, KD, VD, HV, HK, HD):
    """One output row per packed row (no replication): [q [N,KD], k [N,KD], v [N,VD], g f32 [N,HV], beta [N,HV]].
    Not in the reference; the tree-native Gated DeltaNet pass consumes this layout."""
    return list(_prep(proj, hist, None, None, proj.shape[0], convw, A_log, dt_bias, KD, VD, HV, HK, HD))


def linattn_prep_dedup2(proj, hist, rep_ptr, rep_pos, L2, convw, A_log, dt_bias, KD, VD, HV, HK, HD, rep_qk):
    """src/ext.py:22 — replicated slots [S*L2, ...]; rep_qk expands q / k to the value heads."""
    R = rep_pos.numel()
    if rep_ptr.numel() != proj.shape[0] + 2 or R % L2:
        raise RuntimeError("linattn_prep_dedup2: rep_ptr must have N+2 entries and rep_pos a multiple of L2")
    q, k, v, g, beta = _prep(proj, hist, rep_ptr, rep_pos, R, convw, A_log, dt_bias, KD, VD, HV, HK, HD)
    if rep_qk:
        q, k = _expand(q, HK, HV, HD), _expand(k, HK, HV, HD)
    return [q, k, v, g, beta]


# ---- the reference's older prep variants (src/ext.py:8,12,16-21,45): same arithmetic, other row layouts. Each is the one prep
# kernel above with the history table (and, where the output is replicated, the slot tables) of its layout; the tables are
# small integer arrays built on the host and cached per layout.
_hist_cache = {}


def _np():
    import numpy as np
    return np


def _dev_i32(a, device):
    return torch.as_tensor(_np().ascontiguousarray(a, dtype=_np().int32)).to(device)


def _hist_seq(B, T, device):
    """hist for B sequences of T rows laid back to back: row b*T+t sees rows t-3..t of its own sequence."""
    key = ("seq", B, T, str(device))
    if key not in _hist_cache:
        np = _np()
        t = np.arange(B * T) % T
        h = np.arange(B * T)[:, None] - 3 + np.arange(4)[None, :]
        h = np.where(t[:, None] - 3 + np.arange(4)[None, :] >= 0, h, -1)
        _hist_cache[key] = _dev_i32(np.concatenate([h, np.full((1, 4), -1)]), device)
    return _hist_cache[key]


def _hist_tree1(Lp, S, Ls, device):
    """hist for [prefix (Lp) | S suffix blocks of Ls rows]: a suffix row continues the prefix."""
    key = ("tree1", Lp, S, Ls, str(device))
    if key not in _hist_cache:
        np = _np()
        N = Lp + S * Ls
        h = np.full((N + 1, 4), -1, np.int64)
        for n in range(N):
            if n < Lp:
                path = list(range(max(0, n - 3), n + 1))
            else:
                s, t = divmod(n - Lp, Ls)
                path = (list(range(max(0, Lp - 3), Lp)) + list(range(Lp + s * Ls, n + 1)))[-4:]
            h[n, 4 - len(path):] = path
        _hist_cache[key] = _dev_i32(h, device)
    return _hist_cache[key]


def _slots_from_src(src_np, N):
    """CSR (rep_ptr [N+2], rep_pos [S*L2]) of the slots that hold each packed row; group N = pad slots; plus hist from src."""
    np = _np()
    S, L2 = src_np.shape
    flat = src_np.reshape(-1)
    order = np.argsort(np.where(flat >= 0, flat, N), kind="stable")
    counts = np.bincount(np.where(flat >= 0, flat, N), minlength=N + 1)
    rep_ptr = np.concatenate([[0], np.cumsum(counts)])
    hist = np.full((N + 1, 4), -1, np.int64)
    for s in range(S):
        row = src_np[s]
        for t in range(L2):
            n = row[t]
            if n >= 0 and hist[n, 3] < 0:
                path = row[max(0, t - 3): t + 1]
                hist[n, 4 - len(path):] = path
    return rep_ptr, order, hist


def linattn_prep(proj, convw, A_log, dt_bias, T, KD, VD, HV, HK, HD):
    """src/ext.py:8 — rows are sequences of T tokens back to back; q and k are NOT normalised (the caller's attention kernel
    does it) and are expanded to the value heads: [q [N, HV*HD], k [N, HV*HD], v [N, VD], g f32 [N, HV], beta [N, HV]]."""
    N = proj.shape[0]
    q, k, v, g, beta = _prep(proj, _hist_seq(N // T, T, proj.device), None, None, N, convw, A_log, dt_bias, KD, VD, HV, HK, HD, False)
    return [_expand(q, HK, HV, HD), _expand(k, HK, HV, HD), v, g, beta]


def linattn_prep2(proj, convw, A_log, dt_bias, B, T, KD, VD, HV, HK, HD, do_l2):
    """src/ext.py:12 — as linattn_prep for a [B, T] batch, with the L2 norm of q and k optional (what the reference's
    non-tree forward calls, src/fastmodel.py:223)."""
    N = proj.shape[0]
    q, k, v, g, beta = _prep(proj, _hist_seq(B, T, proj.device), None, None, N, convw, A_log, dt_bias, KD, VD, HV, HK, HD, bool(do_l2))
    return [_expand(q, HK, HV, HD), _expand(k, HK, HV, HD), v, g, beta]


def linattn_prep_tree(proj, convw, A_log, dt_bias, Lp, S, Ls, KD, VD, HV, HK, HD):
    """src/ext.py:45 — single-level tree [prefix | S suffixes], one output row per packed row, q / k on the value heads."""
    N = proj.shape[0]
    if N != Lp + S * Ls:
        raise RuntimeError("linattn_prep_tree: proj must have Lp + S*Ls rows")
    q, k, v, g, beta = _prep(proj, _hist_tree1(Lp, S, Ls, proj.device), None, None, N, convw, A_log, dt_bias, KD, VD, HV, HK, HD)
    return [_expand(q, HK, HV, HD), _expand(k, HK, HV, HD), v, g, beta]


def linattn_prep_rep(proj, convw, A_log, dt_bias, Lp, S, Ls, KD, VD, HV, HK, HD):
    """src/ext.py:16 — as linattn_prep_tree, written in replicated form: S sequences of Lp + Ls rows (the prefix in front of
    every suffix), q / k on the value heads."""
    N = proj.shape[0]
    if N != Lp + S * Ls:
        raise RuntimeError("linattn_prep_rep: proj must have Lp + S*Ls rows")
    key = ("rep", Lp, S, Ls, str(proj.device))
    if key not in _hist_cache:
        np = _np()
        L2 = Lp + Ls
        src = np.concatenate([np.tile(np.arange(Lp), (S, 1)), Lp + np.arange(S * Ls).reshape(S, Ls)], 1)
        rep_ptr, rep_pos, _ = _slots_from_src(src, N)
        _hist_cache[key] = (_dev_i32(rep_ptr, proj.device), _dev_i32(rep_pos, proj.device))
    rep_ptr, rep_pos = _hist_cache[key]
    q, k, v, g, beta = _prep(proj, _hist_tree1(Lp, S, Ls, proj.device), rep_ptr, rep_pos, S * (Lp + Ls), convw, A_log, dt_bias,
                             KD, VD, HV, HK, HD)
    return [_expand(q, HK, HV, HD), _expand(k, HK, HV, HD), v, g, beta]


def _prep_src(proj, src, convw, A_log, dt_bias, KD, VD, HV, HK, HD):
    if src.dim() != 2 or src.dtype != torch.int32:
        raise RuntimeError("linattn_prep_map: src must be int32 [S, L2]")
    N = proj.shape[0]
    rep_ptr, rep_pos, hist = _slots_from_src(src.detach().cpu().numpy(), N)      # host round trip: not a graph-capturable path
    dev = proj.device
    return _prep(proj, _dev_i32(hist, dev), _dev_i32(rep_ptr, dev), _dev_i32(rep_pos, dev), src.numel(), convw, A_log, dt_bias,
                 KD, VD, HV, HK, HD)


def linattn_prep_map(proj, src, convw, A_log, dt_bias, KD, VD, HV, HK, HD):
    """src/ext.py:18 — slot (s, t) holds packed row src[s, t] (-1: pad slot, zeros); q / k on the value heads."""
    q, k, v, g, beta = _prep_src(proj, src, convw, A_log, dt_bias, KD, VD, HV, HK, HD)
    return [_expand(q, HK, HV, HD), _expand(k, HK, HV, HD), v, g, beta]


def linattn_prep_map2(proj, src, convw, A_log, dt_bias, KD, VD, HV, HK, HD, tch):
    """src/ext.py:20 — as linattn_prep_map with q / k on the key heads (grouped value attention); tch (tokens per thread in
    the reference's schedule) has no meaning here."""
    return list(_prep_src(proj, src, convw, A_log, dt_bias, KD, VD, HV, HK, HD))


def linattn_prep_dedup(proj, src, rep_ptr, rep_pos, convw, A_log, dt_bias, KD, VD, HV, HK, HD):
    """src/ext.py:21 — as linattn_prep_dedup2 with the history taken from src [S, L2] instead of a hist table."""
    N = proj.shape[0]
    if rep_ptr.numel() != N + 2 or rep_pos.numel() != src.numel():
        raise RuntimeError("linattn_prep_dedup: rep_ptr must have N+2 entries and rep_pos S*L2")
    hist = _slots_from_src(src.detach().cpu().numpy(), N)[2]
    return list(_prep(proj, _dev_i32(hist, proj.device), rep_ptr, rep_pos, rep_pos.numel(), convw, A_log, dt_bias, KD, VD, HV, HK, HD))


def linattn_prep_dedup3(proj, hist, rep_ptr, rep_pos, L2, convw, A_log, dt_bias, KD, VD, HV, HK, HD):
    """src/ext.py:27 — as dedup2 plus a copy of k expanded to the value heads: [q, k, krep, v, g, beta]."""
    q, k, v, g, beta = linattn_prep_dedup2(proj, hist, rep_ptr, rep_pos, L2, convw, A_log, dt_bias, KD, VD, HV, HK, HD, False)
    return [q, k, _expand(k, HK, HV, HD), v, g, beta]


_table_cache = {}


def _seq_tables(B, T, device):
    """chunk / step / walk tables for B independent sequences of T rows laid out back to back."""
    key = (B, T, str(device))
    t = _table_cache.get(key)
    if t is None:
        nc = (T + 63) // 64
        chunks = torch.zeros(B * nc, 4, dtype=torch.int32)
        steps = torch.zeros(B * nc, 4, dtype=torch.int32)
        for b in range(B):
            for j in range(nc):
                i = b * nc + j
                chunks[i, 0], chunks[i, 1] = b * T + j * 64, min(64, T - j * 64)
                steps[i, 0], steps[i, 1] = i, 1 if j == 0 else 0
        walks = torch.arange(0, (B + 1) * nc, nc, dtype=torch.int32)
        t = _table_cache[key] = tuple(x.to(device) for x in (chunks, steps, walks))
    return t


def gdn_chunked(q, k, v, g, beta, scale, chunks, steps, walk_ptr, n_walks, init_state=None, final_state=None, out=None):
    """Table-driven chunked gated delta rule (see include/ojb200.h ojb_gdn_chunked). q, k [rows, HK, 128],
    v [rows, HV, 128], g f32 / beta bf16 [rows, HV]. Returns out bf16 [rows, HV, 128]."""
    _chk(q, k, v, g, beta, chunks, steps, walk_ptr, init_state, final_state)
    rows, HV, HD = v.shape[-3], v.shape[-2], v.shape[-1]
    HK = k.shape[-2]
    if HD != 128 or k.shape[-1] != 128 or g.dtype != torch.float32 or beta.dtype != bf16:
        raise RuntimeError("gdn: head dim must be 128, g fp32 and beta bf16")
    nch = chunks.shape[0]
    nbytes = _lib.lib().ojb_gdn_scratch_bytes
    nbytes.restype = _lib.ctypes.c_int64
    scratch = torch.empty(nbytes(i64(nch), i64(HV)), dtype=torch.uint8, device=v.device)
    if out is None:
        out = torch.empty(v.shape, dtype=bf16, device=v.device)
    call("ojb_gdn_chunked", ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(chunks), i64(nch), ptr(steps), ptr(walk_ptr),
         i64(n_walks), ptr(init_state), ptr(final_state), ptr(scratch), ptr(out), i64(HK), i64(HV), f32(scale),
         ptr(_lib.status_word(v.device)), stream_ptr())
    return out


def gdn_chunked_proj(proj, hist, convw, A_log, dt_bias, KD, VD, HV, HK, scale, chunks, steps, walk_ptr, n_walks, init_state=None,
                     final_state=None, out=None):
    """gdn_chunked with the preparation fused into its first launch (ojb_gdn_chunked_proj): reads the in-projection output
    `proj` [N, 2KD+2VD+2HV] and the history table directly — linattn_prep_rows + gdn_chunked in two launches instead of three,
    same bits. Chunks must be runs of consecutive packed rows of one tree node (the layout builder's tables).
    Returns out bf16 [N, HV, 128] (rows outside every chunk are left as they are)."""
    _chk(proj, hist, convw, A_log, dt_bias, chunks, steps, walk_ptr, init_state, final_state)
    N = proj.shape[0]
    if any(t.dtype != bf16 for t in (proj, convw, A_log, dt_bias)) or proj.shape[1] != 2 * KD + 2 * VD + 2 * HV \
            or hist.shape != (N + 1, 4) or hist.dtype != torch.int32 or convw.shape != (2 * KD + VD, 4):
        raise RuntimeError("gdn_chunked_proj: proj [N, 2KD+2VD+2HV], convw [2KD+VD, 4], A_log / dt_bias bf16 and hist int32 [N+1, 4]")
    nch = chunks.shape[0]
    nbytes = _lib.lib().ojb_gdn_scratch_bytes
    nbytes.restype = _lib.ctypes.c_int64
    scratch = torch.empty(nbytes(i64(nch), i64(HV)), dtype=torch.uint8, device=proj.device)
    if out is None:
        out = torch.zeros(N, HV, 128, dtype=bf16, device=proj.device)
    call("ojb_gdn_chunked_proj", ptr(proj), ptr(hist), ptr(convw), ptr(A_log), ptr(dt_bias), ptr(chunks), i64(nch), ptr(steps),
         ptr(walk_ptr), i64(n_walks), ptr(init_state), ptr(final_state), ptr(scratch), ptr(out), i64(KD), i64(VD), i64(HK), i64(HV),
         f32(scale), ptr(_lib.status_word(proj.device)), stream_ptr())
    return out


def gdn_tree_levels(q, k, v, g, beta, scale, lay, out, states=None):
    """Tree-native pass with the state recurrence run level by level (root, question stems, leaves as three launches whose
    walks run side by side). q, k [N, HK, 128], v [N, HV, 128]; `out` [N, HV, 128] is written for real rows only; `states`
    fp32 [1 + S, HV, 128, 128] receives the end state of the root (slot 0) and of question r (slot 1 + r)."""
    _chk(q, k, v, g, beta, out, states)
    N, HV = v.shape[0], v.shape[1]
    HK, S = k.shape[1], lay.S
    if states is None:
        states = torch.empty(1 + S, HV, 128, 128, dtype=torch.float32, device=v.device)
    nch = lay.chunks.shape[0]
    nbytes = _lib.lib().ojb_gdn_scratch_bytes
    nbytes.restype = _lib.ctypes.c_int64
    scratch = torch.empty(nbytes(i64(nch), i64(HV)), dtype=torch.uint8, device=v.device)
    levels = (_lib.ctypes.c_int32 * 4)(0, 1, 1 + S, 1 + 2 * S)
    call("ojb_gdn_chunked_levels", ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(lay.chunks), i64(nch), ptr(lay.lsteps),
         ptr(lay.lwalks), levels, i64(3), ptr(states), ptr(scratch), ptr(out), i64(HK), i64(HV), f32(scale),
         ptr(_lib.status_word(v.device)), stream_ptr())
    return out, states


def gdn_fused6(q, k, v, g, beta, scale):
    """src/ext.py:34 — q, k [B,T,HK,128], v [B,T,HV,128], g f32 / beta [B,T,HV] -> o [B,T,HV,128]; zero initial state,
    rows of the last partial chunk beyond T do not exist, pad slots inside T produce zeros only if their inputs are."""
    B, T = v.shape[0], v.shape[1]
    chunks, steps, walks = _seq_tables(B, T, v.device)
    return gdn_chunked(q, k, v, g, beta, scale, chunks, steps, walks, B)


gdn_fused = gdn_fused2 = gdn_fused3 = gdn_fused4 = gdn_fused8 = gdn_fused9 = gdn_fused6   # src/ext.py:30-33,41-42


def gdn_fused5(q, k, v, g, beta, scale, proj, zoff, normw, sig, canon, rowmask, neps):
    """src/ext.py:44 — gdn_fused6 followed by the gated RMSNorm, written per packed row: [N, HV*128]; packed row n reads the
    Gated DeltaNet output at its canonical slot (canon[slot] = n), rows with rowmask 0 are zero. Two launches plus the index
    arithmetic here; the reference fuses them into one kernel and rejected that form as slower."""
    B, T, HV, HD = v.shape
    N = proj.shape[0]
    if canon.numel() != B * T or rowmask.numel() != N:
        raise RuntimeError("gdn_fused5: canon must have B*T entries and rowmask N")
    o = gdn_fused6(q, k, v, g, beta, scale)
    c = canon.reshape(-1).long()
    ok = c >= 0
    inv = torch.zeros(N, dtype=torch.int32, device=proj.device)
    inv[c[ok]] = torch.arange(B * T, device=proj.device, dtype=torch.int32)[ok]
    y = _gated_norm(o.view(B * T, HV, HD), inv, proj, normw, HV, HD, zoff, neps)
    return y * (rowmask != 0).to(y.dtype)[:, None]


gdn_fused7 = gdn_fused5   # src/ext.py:35 — same contract (the reference's persistent-CTA schedule of it)


def gdn_fused6ts(q, k, v, g, beta, scale):
    """src/ext.py:36 — the reference's instrumented build of gdn_fused6 returns int64 [B*HV, 16] clock stamps instead of the
    output. The kernels here are instrumented through ojb_gdn_set_trace instead; this name runs the operator and returns
    a zero tensor of the reference's shape."""
    gdn_fused6(q, k, v, g, beta, scale)
    return torch.zeros(v.shape[0] * v.shape[2], 16, dtype=torch.int64, device=v.device)


def gdn_tree(q, k, v, g, beta, scale, lay, final_state=None):
    """Tree-native pass over packed rows: q, k [N, HK*128], v [N, HV*128] from linattn_prep_rows; the chunk / walk tables
    come from the layout (lay.chunks, lay.steps, lay.meta). Shared nodes are computed once. Returns o [N, HV, 128]; rows
    that belong to no node (end padding) are zero."""
    N = v.shape[0]
    HV = g.shape[1]
    HK = q.shape[1] // 128
    out = torch.zeros(N, HV, 128, dtype=bf16, device=v.device)
    return gdn_chunked(q.view(N, HK, 128), k.view(N, HK, 128), v.view(N, HV, 128), g, beta, scale, lay.chunks, lay.steps,
                       lay.meta[6:8], 1, None, final_state, out)


def gated_rmsnorm_map(x, proj, w, HV, HD, zoff, eps, Lp, Ls):
    """src/ext.py:17 — x is the Gated DeltaNet output in replicated form [S, Lp + Ls, HV, HD] (linattn_prep_rep); packed row n
    of [prefix | S suffixes] reads slot (0, n) for a prefix row and (s, Lp + t) for row t of suffix s."""
    N = proj.shape[0]
    key = ("gmap", N, Lp, Ls, str(proj.device))
    if key not in _hist_cache:
        np = _np()
        n = np.arange(N)
        s_, t_ = np.divmod(np.maximum(n - Lp, 0), max(Ls, 1))
        _hist_cache[key] = _dev_i32(np.where(n < Lp, n, s_ * (Lp + Ls) + Lp + t_), proj.device)
    return _gated_norm(x, _hist_cache[key], proj, w, HV, HD, zoff, eps)


def _gated_norm(x, inv, proj, w, HV, HD, zoff, eps):
    _chk(x, inv, proj, w)
    N, P = proj.shape
    out = torch.empty(N, HV * HD, dtype=bf16, device=proj.device)
    call("ojb_gated_rmsnorm", ptr(x), ptr(inv), ptr(proj), ptr(w), ptr(out), i64(N), i64(HV), i64(HD), i64(zoff), i64(P),
         f32(eps), stream_ptr())
    return out


def gated_rmsnorm(x, proj, w, HV, HD, zoff, eps):
    """src/ext.py:9 — x [N, HV, HD] in packed-row order."""
    return _gated_norm(x, None, proj, w, HV, HD, zoff, eps)


def gated_rmsnorm_inv(x, inv, proj, w, HV, HD, zoff, eps):
    """src/ext.py:19 — x read at slot inv[n]."""
    return _gated_norm(x, inv, proj, w, HV, HD, zoff, eps)


def gated_rmsnorm_inv2(x, inv, proj, w, sig, HV, HD, zoff, eps):
    """src/ext.py:25 — as gated_rmsnorm_inv; the sigmoid is computed (same bits as the table)."""
    return _gated_norm(x, inv, proj, w, HV, HD, zoff, eps)


# ------------------------------------------------------------------------------------------------ tree attention
def _tree_attn(qt, kt, vt, gate, vbits, krange, scale, gq):
    _chk(qt, kt, vt, gate, vbits, krange)
    if qt.dim() != 4 or qt.shape[0] != 1:
        raise RuntimeError("fattn_tree: qt must be [1, HQ, N, D]")
    _, HQ, N, D = qt.shape
    HKV = kt.shape[1]
    if N % 32 or (HQ // HKV) % gq or D not in (64, 128, 256):
        raise RuntimeError("fattn_tree: N % 32 == 0, gq | HQ/HKV and D in {64,128,256} required")
    y = torch.empty(N, HQ * D, dtype=bf16, device=qt.device)
    call("ojb_tree_attn", ptr(qt), ptr(kt), ptr(vt), ptr(gate), ptr(vbits), ptr(krange), ptr(y), i64(N), i64(HQ), i64(HKV),
         i64(D), i64(gq), f32(scale), stream_ptr())
    return y


def fattn_tree(qt, kt, vt, gate, sig, vbits, scale, gq):
    """src/ext.py:37 — ancestor-masked attention + gate from the packed visibility words; gq in {3, 6} heads per CTA."""
    return _tree_attn(qt, kt, vt, gate, vbits, None, scale, gq)


def fattn_tree3(qt, kt, vt, gate, sig, vbits, scale):
    """src/ext.py:39 — the reference's two-warps-per-head schedule; same result, served by the 3-heads-per-CTA launch."""
    G = qt.shape[1] // kt.shape[1]
    return _tree_attn(qt, kt, vt, gate, vbits, None, scale, 3 if G % 3 == 0 else 1)


def fattn_tree_ranges(qt, kt, vt, gate, krange, scale, gq):
    """Same attention with the mask given as three key ranges per row (lay.krange): no N x N structure anywhere."""
    return _tree_attn(qt, kt, vt, gate, None, krange, scale, gq)


def fattn_tree_tc(qt, kt, vt_t, gate, krange, scale):
    """Tree attention + gate on the tcgen05 tensor cores (ojb_tree_attn_tc): head dim 256, at most 6 query heads per kv head,
    mask from the three key ranges per row. qt [1, HQ, N, 256], kt [1, HKV, N, 256], vt_t [1, HKV, 256, N] (fullattn_prep2 with
    with_vt_t=True), gate [N, HQ*256] -> y [N, HQ*256]."""
    _chk(qt, kt, vt_t, gate, krange)
    _, HQ, N, D = qt.shape
    HKV = kt.shape[1]
    if D != 256 or N % 32 or HQ % HKV or HQ // HKV > 6 or tuple(vt_t.shape) != (1, HKV, D, N):
        raise RuntimeError("fattn_tree_tc: head dim 256, N % 32 == 0, HQ/HKV <= 6 and vt_t [1, HKV, 256, N] required")
    y = torch.empty(N, HQ * D, dtype=bf16, device=qt.device)
    call("ojb_tree_attn_tc", ptr(qt), ptr(kt), ptr(vt_t), ptr(gate), ptr(krange), ptr(y), i64(N), i64(HQ), i64(HKV), i64(D),
         f32(scale), ptr(_lib.status_word(qt.device)), stream_ptr())
    return y


def fattn_tree2(proj, qw1, kw1, cosb, sinb, sig, vbits, HQ, HKV, scale, eps):
    """src/ext.py:38 — q/k preparation + attention + gate from the in-projection output (two launches here)."""
    N = proj.shape[0]
    D = qw1.shape[0]
    qt, kt, vt, gate = fullattn_prep2(proj, qw1, kw1, cosb, sinb, 1, N, HQ, HKV, D, eps)
    G = HQ // HKV
    return _tree_attn(qt, kt, vt, gate, vbits, None, scale, 3 if G % 3 == 0 else 1)


def fattn_tree2_ts(proj, qw1, kw1, cosb, sinb, sig, vbits, HQ, HKV, scale, eps):
    """src/ext.py:38 (instrumented fattn_tree2) — int64 [CTAs, 16] clock stamps in the reference; here the operator runs and a
    zero tensor of that shape (CTAs of the reference's grid: HKV * (HQ/HKV/3) * N/16) is returned."""
    fattn_tree2(proj, qw1, kw1, cosb, sinb, sig, vbits, HQ, HKV, scale, eps)
    return torch.zeros(HKV * max(HQ // HKV // 3, 1) * (proj.shape[0] // 16), 16, dtype=torch.int64, device=proj.device)


def l2_prefetch(t, chunk):
    """src/ext.py:26 — bulk L2 prefetch of a contiguous CUDA tensor in slices of `chunk` bytes (a multiple of 16)."""
    if not (t.is_cuda and t.is_contiguous()) or chunk % 16:
        raise RuntimeError("l2_prefetch: contiguous CUDA tensor and chunk % 16 == 0 required")
    call("ojb_l2_prefetch", ptr(t), i64(t.numel() * t.element_size()), i64(min(int(chunk), 1 << 20)), stream_ptr())


def embed_rope(ids, table, pos, inv_freq, scaling=1.0):
    """ids, pos int64 [N]; table bf16 [vocab, H]; inv_freq f32 [R2] -> (x bf16 [N, H], cos bf16 [N, 2*R2], sin): the
    embedding rows and the rotary tables of a packed tree in one launch (the reference calls torch's embedding and the
    backbone's rotary module, src/fastmodel.py:404-405)."""
    _chk(ids, table, pos, inv_freq)
    if ids.dtype != torch.int64 or pos.dtype != torch.int64 or table.dtype != bf16 or inv_freq.dtype != torch.float32:
        raise RuntimeError("embed_rope: int64 ids / pos, bf16 table and fp32 inv_freq required")
    N, (V, H), R2 = ids.numel(), table.shape, inv_freq.numel()
    x = torch.empty(N, H, dtype=bf16, device=table.device)
    cos = torch.empty(N, 2 * R2, dtype=bf16, device=table.device)
    sin = torch.empty_like(cos)
    call("ojb_embed_rope", ptr(ids), ptr(table), i64(V), ptr(pos), ptr(inv_freq), f32(scaling), ptr(x), ptr(cos), ptr(sin),
         i64(N), i64(H), i64(R2), stream_ptr())
    return x, cos, sin


# ------------------------------------------------------------------------------------------------ scoring head
def score_head(hn, rows, W, bias):
    """hn bf16 [N, H], rows int64 [S], W f32 [A, H], bias f32 [A] or None -> f32 [S, A] (gather + fp32 linear in one
    launch; the reference does `head(hn[lastidx].float())` with torch, src/server.py:37)."""
    _chk(hn, rows, W, bias)
    S, (A, H) = rows.numel(), W.shape
    out = torch.empty(S, A, dtype=torch.float32, device=hn.device)
    call("ojb_score_head", ptr(hn), ptr(rows), ptr(W), ptr(bias), ptr(out), i64(S), i64(A), i64(H), stream_ptr())
    return out
