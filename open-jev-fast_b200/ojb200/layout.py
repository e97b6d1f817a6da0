"""Prefix-tree layout: host builder (C++ in libojb200.so) + upload. Mirrors FastQwen35.gtree_build of open-jev-fast
(src/fastmodel.py:321-398): same arguments, same returned (ids, lay) with the same field names, shapes and dtypes."""
import ctypes
from types import SimpleNamespace

import numpy as np
import torch

from . import _lib

_I64P = ctypes.POINTER(ctypes.c_int64)
_I32P = ctypes.POINTER(ctypes.c_int32)


def _pad8(n):
    return n + (-n) % 8


def _flatten(seqs, groups):
    S = len(seqs)
    off = np.zeros(S + 1, np.int64)
    np.cumsum([len(s) for s in seqs], out=off[1:])
    tok = np.fromiter((t for s in seqs for t in s), np.int64, count=int(off[-1]))
    return tok, off, np.asarray(groups, np.int32)


def gtree_host(seqs, groups, pad_id, NB=32, PB=16, pin=False, vbits=True):
    """Runs the host builder. Returns (dims dict, buf64, buf32, ext32) as CPU torch tensors (pinned if asked). With
    vbits=False the N x N/32 visibility words (last field of buf32) are not computed; dims["n32_used"] is the number of
    int32 elements of buf32 that carry data."""
    if len(seqs) == 0 or len(groups) != len(seqs):
        raise RuntimeError("gtree_build: need one group index per candidate and at least one candidate")
    tok, off, grp = _flatten(seqs, groups)
    dims = np.zeros(10, np.int64)
    L = _lib.lib()
    args = (tok.ctypes.data_as(_I64P), off.ctypes.data_as(_I64P), grp.ctypes.data_as(_I32P), ctypes.c_int64(len(seqs)))
    rc = L.ojb_gtree_dims(*args, ctypes.c_int64(NB), ctypes.c_int64(PB), dims.ctypes.data_as(_I64P))
    if rc != 0:
        raise RuntimeError("gtree_build: invalid request (empty candidate, unused question index, or row bucket not a "
                           "multiple of 32)")
    N, S, R, L2, Lr, Nreal, n64, n32, next_, cap = (int(v) for v in dims)
    buf64 = torch.empty(n64, dtype=torch.int64, pin_memory=pin)
    buf32 = torch.empty(n32, dtype=torch.int32, pin_memory=pin)
    ext32 = torch.empty(next_, dtype=torch.int32, pin_memory=pin)
    rc = L.ojb_gtree_fill(*args, ctypes.c_int64(pad_id), ctypes.c_int64(NB), ctypes.c_int64(PB),
                          ctypes.cast(buf64.data_ptr(), _I64P), ctypes.cast(buf32.data_ptr(), _I32P),
                          ctypes.cast(ext32.data_ptr(), _I32P), ctypes.c_int32(0 if vbits else 1))
    if rc != 0:
        raise RuntimeError("gtree_build: layout fill failed")
    d = dict(N=N, S=S, R=R, L2=L2, Lr=Lr, Nreal=Nreal, cap=cap)
    d["n32_used"] = n32 if vbits else n32 - _pad8(N * (N // 32))
    return d, buf64, buf32, ext32


def field_views(d, g64, g32, e32):
    """Named views into the three packed buffers (host or device)."""
    N, S, L2, cap = d["N"], d["S"], d["L2"], d["cap"]
    n64 = N + (-N) % 4
    sizes = [S * L2, N, N + 2, S * L2, (N + 1) * 4, S * L2, N, N * (N // 32)]
    o = np.cumsum([0] + [_pad8(x) for x in sizes])
    v = lambda k: g32[o[k]:o[k] + sizes[k]]
    eo = np.cumsum([0, N * 8, (1 + 2 * S) * 4, cap * 4, cap * 4, 8, cap * 4, _pad8(2 + 2 * S)])
    e = lambda k: e32[eo[k]:eo[k + 1]]
    return dict(ids=g64[:N], pos=g64[n64:n64 + N], lastidx=g64[2 * n64:2 * n64 + S],
                src=v(0).view(S, L2), inv=v(1), rep_ptr=v(2), rep_pos=v(3), hist=v(4).view(N + 1, 4), canon=v(5),
                rowmask=v(6), vbits=v(7).view(N, N // 32),
                krange=e(0).view(N, 8), nodes=e(1).view(1 + 2 * S, 4), chunks=e(2).view(cap, 4), steps=e(3).view(cap, 4),
                meta=e(4), lsteps=e(5).view(cap, 4), lwalks=e(6)[:2 + 2 * S])


def dense_masks(vbits):
    """amask bool [1,1,N,N] and amask_add bf16 (0 / -inf) from the packed visibility words (device-side torch ops)."""
    N = vbits.shape[0]
    sh = torch.arange(32, device=vbits.device, dtype=torch.int32)
    vis = ((vbits.unsqueeze(-1) >> sh) & 1).bool().view(N, N)
    add = torch.zeros((N, N), dtype=torch.bfloat16, device=vbits.device).masked_fill_(~vis, float("-inf"))
    return vis[None, None], add[None, None]


def gtree_build(seqs, groups, pad_id, NB=32, PB=16, dev="cuda", dense=True):
    """Drop-in for FastQwen35.gtree_build: returns (ids, lay). Three host-to-device copies (int64 fields, int32 fields,
    extension tables); the dense masks, which only the SDPA-style paths of the reference read, are expanded on the device
    from the packed bits instead of being copied (skip them with dense=False)."""
    on_gpu = torch.device(dev).type == "cuda"
    d, b64, b32, e32 = gtree_host(seqs, groups, pad_id, NB, PB, pin=on_gpu)
    g64 = b64.to(dev, non_blocking=True)
    g32 = b32.to(dev, non_blocking=True)
    ge = e32.to(dev, non_blocking=True)
    f = field_views(d, g64, g32, ge)
    lay = SimpleNamespace(N=d["N"], S=d["S"], R=d["R"], L2=d["L2"], Lr=d["Lr"], Nreal=d["Nreal"], key=(d["N"], d["S"], d["L2"]),
                          cap=d["cap"], _host=(b64, b32, e32), _dev=(g64, g32, ge))
    ids = f.pop("ids")
    for k, v in f.items():
        setattr(lay, k, v)
    lay.walk_ptr, lay.n_walks = lay.meta[6:8], 1
    if dense:
        lay.amask, lay.amask_add = dense_masks(lay.vbits)
    return ids, lay


def pack_requests(requests, pad_id=0, NB=32, PB=16, dev="cuda", pin=False):
    """Several requests in one forward (not in the reference, which scores one request at a time): every request keeps
    its own packed tree, the trees follow one another in the row dimension, and every table of the tree kernels is shifted
    accordingly — history and key ranges by the row offset of the request, walk steps by its chunk offset; each tree is
    one walk of the state pass. `requests` = list of (seqs, groups). Returns (ids, lay, host) where lay has the fields the
    tree forward reads (pos, rowmask, hist, krange, chunks, steps, walk_ptr, n_walks, lastidx, N, S) and `host` is the
    dict of host tensors behind them (for re-upload into static buffers), plus `counts` = candidates per request."""
    ids, pos, rowmask, hist, krange, chunks, steps, last, walks, counts, keys = [], [], [], [], [], [], [], [], [0], [], []
    base = cbase = 0
    for seqs, groups in requests:
        d, b64, b32, e32 = gtree_host(seqs, groups, pad_id, NB, PB, vbits=False)
        f = {k: v.numpy() for k, v in field_views(d, b64, b32, e32).items() if k != "vbits"}
        N = d["N"]
        ids.append(f["ids"]); pos.append(f["pos"]); rowmask.append(f["rowmask"])
        h = f["hist"][:N].copy()
        h[h >= 0] += base
        hist.append(h)
        kr = f["krange"].copy()
        kr[:, 5] = np.where(kr[:, 0] > 0, base, 0)
        kr[:, 0] = np.where(kr[:, 0] > 0, kr[:, 0] + base, 0)
        kr[:, 1:5] += base
        krange.append(kr)
        ch = f["chunks"].copy()
        ch[:, 0] += base
        chunks.append(ch)
        w0, w1 = int(f["meta"][6]), int(f["meta"][7])
        st = f["steps"][w0:w1].copy()
        st[:, 0] += cbase
        steps.append(st)
        walks.append(walks[-1] + (w1 - w0))
        last.append(f["lastidx"] + base)
        counts.append(d["S"])
        keys.append((d["N"], d["S"], d["L2"]))
        base += N
        cbase += ch.shape[0]
    hist.append(np.full((1, 4), -1, np.int32))
    host = dict(ids=np.concatenate(ids), pos=np.concatenate(pos), rowmask=np.concatenate(rowmask), hist=np.concatenate(hist),
                krange=np.concatenate(krange), chunks=np.concatenate(chunks), steps=np.concatenate(steps),
                walk_ptr=np.asarray(walks, np.int32), lastidx=np.concatenate(last))
    host = {k: (torch.as_tensor(np.ascontiguousarray(v)).pin_memory() if pin else torch.as_tensor(np.ascontiguousarray(v)))
            for k, v in host.items()}
    lay = SimpleNamespace(N=base, S=int(sum(counts)), L2=max(k[2] for k in keys), n_walks=len(requests), counts=counts,
                          key=tuple(keys), **{k: v.to(dev) for k, v in host.items() if k != "ids"})
    return host["ids"].to(dev), lay, host


def batch_layout(attention_mask, dev):
    """Layout of a right-padded batch [B, T] of independent sequences (the non-tree forward of src/fastmodel.py:205-241)
    in the vocabulary of the tree kernels: every sequence is its own path, rows are b*T + t, padded up to a multiple of 32
    rows. Returns a namespace with pos, rowmask, hist, krange, chunks, steps, walk_ptr, n_walks, lastidx, N."""
    m = attention_mask.detach().cpu().numpy().astype(bool)
    B, T = m.shape
    N = -(-(B * T) // 32) * 32
    lens = m.sum(1)
    pos = np.zeros(N, np.int64)
    rowmask = np.zeros(N, np.int32)
    hist = np.full((N + 1, 4), -1, np.int32)
    krange = np.zeros((N, 8), np.int32)
    chunks, steps, walks = [], [], [0]
    for b in range(B):
        L = int(lens[b])
        for t in range(T):
            n = b * T + t
            krange[n, 3], krange[n, 4] = (b * T, n + 1) if t < L else (n, n + 1)
            if t < L:
                pos[n], rowmask[n] = t, 1
                for i in range(4):
                    if t - 3 + i >= 0:
                        hist[n, i] = n - 3 + i
        for j in range(0, L, 64):
            steps.append([len(chunks), 1 if j == 0 else 0, 0, 0])
            chunks.append([b * T + j, min(64, L - j), 0, 0])
        walks.append(len(steps))
    for n in range(B * T, N):
        krange[n, 3], krange[n, 4] = n, n + 1
    if not chunks:
        chunks, steps = [[0, 0, 0, 0]], [[0, 1, 0, 0]]
    t32 = lambda a: torch.as_tensor(np.asarray(a, np.int32)).to(dev)
    last = np.array([b * T + max(int(lens[b]) - 1, 0) for b in range(B)], np.int64)
    return SimpleNamespace(N=N, S=B, L2=T, pos=torch.as_tensor(pos).to(dev), rowmask=t32(rowmask), hist=t32(hist),
                           krange=t32(krange), chunks=t32(chunks), steps=t32(steps), walk_ptr=t32(walks), n_walks=B,
                           lastidx=torch.as_tensor(last).to(dev))


def tree_layout(pre_ids, suf_ids, suf_mask, pad=0, dense=True, cap=None):
    """Single-level tree [prefix | S suffixes of Ls rows] of FastQwen35.tree_layout (src/fastmodel.py:247-264): the same
    fields (Lp, S, Ls, N, pos, amask, rowmask, lastidx, repidx) plus the tables the kernels here consume (hist, krange,
    chunks, steps, walk_ptr). The first `pad` prefix rows are left padding. Rows are padded up to a multiple of 32 (N32).
    dense=False leaves out the O(N^2) mask and the replication index (the kernels do not read them); cap pads the chunk and
    step tables to a fixed number of entries so that one CUDA graph serves every request of a (Lp, S, Ls) key."""
    dev = suf_ids.device
    Lp = int(pre_ids.shape[0])
    S, Ls = (int(x) for x in suf_ids.shape)
    m = suf_mask.detach().cpu().numpy().astype(bool)
    N = Lp + S * Ls
    N32 = -(-N // 32) * 32
    pos = np.zeros(N32, np.int64)
    rowmask = np.zeros(N32, np.int32)
    hist = np.full((N32 + 1, 4), -1, np.int32)
    krange = np.zeros((N32, 8), np.int32)
    for n in range(N32):
        krange[n, 3], krange[n, 4] = n, n + 1                      # default: a row sees only itself
    # positions follow the reference for every row, padding included: prefix t - pad, suffix t + (Lp - pad)
    pos[:Lp] = np.arange(Lp) - pad
    for s in range(S):
        pos[Lp + s * Ls: Lp + (s + 1) * Ls] = np.arange(Ls) + (Lp - pad)
    if Lp > pad:
        pr = np.arange(pad, Lp)
        rowmask[pad:Lp] = 1
        krange[pad:Lp, 3], krange[pad:Lp, 4] = pad, pr + 1
        hp = pr[:, None] - 3 + np.arange(4)[None, :]
        hist[pad:Lp] = np.where(hp >= pad, hp, -1)
    lens = m.sum(1)
    for s in range(S):
        for t in range(int(lens[s])):
            n = Lp + s * Ls + t
            rowmask[n] = 1
            krange[n, 1], krange[n, 2] = pad, Lp
            krange[n, 3], krange[n, 4] = Lp + s * Ls, n + 1
            tail = list(range(max(pad, Lp - 3), Lp)) + list(range(Lp + s * Ls, n + 1))     # the last rows of this path
            for i in range(4):
                if len(tail) - 4 + i >= 0:
                    hist[n, i] = tail[len(tail) - 4 + i]
    chunks, steps, walks = [], [], [0]
    for j in range(pad, Lp, 64):
        steps.append([len(chunks), 1 if j == pad else 0, 0, 0])
        chunks.append([j, min(64, Lp - j), 0, 0])
    if steps:
        steps[-1][2] = 1                                            # park the prefix state in slot A
    for s in range(S):
        for j in range(0, int(lens[s]), 64):
            steps.append([len(chunks), (2 if Lp > pad else 1) if j == 0 else 0, 0, 0])
            chunks.append([Lp + s * Ls + j, min(64, int(lens[s]) - j), 0, 0])
    walks.append(len(steps))
    if not chunks:
        chunks, steps = [[0, 0, 0, 0]], [[0, 1, 0, 0]]
    if cap is not None:
        if len(chunks) > cap:
            raise RuntimeError("tree_layout: more chunks than the table capacity")
        chunks += [[0, 0, 0, 0]] * (cap - len(chunks))
        steps += [[0, 0, 0, 0]] * (cap - len(steps))
    t32 = lambda a: torch.as_tensor(np.asarray(a, np.int32)).to(dev)
    lastidx = np.array([Lp + s * Ls + max(int(lens[s]) - 1, 0) for s in range(S)], np.int64)
    if not dense:
        return SimpleNamespace(Lp=Lp, S=S, Ls=Ls, N=N, N32=N32, pos=torch.as_tensor(pos[:N]).to(dev), pos32=torch.as_tensor(pos).to(dev),
                               rowmask=t32(rowmask[:N]), rowmask32=t32(rowmask), lastidx=torch.as_tensor(lastidx).to(dev),
                               hist=t32(hist), krange=t32(krange), chunks=t32(chunks), steps=t32(steps), walk_ptr=t32(walks), n_walks=1)
    # dense mask with the reference's semantics for every row (rows that are padding still see valid earlier keys of their
    # own segment and of the prefix); the kernels read krange, where padding rows see only themselves
    seg = np.concatenate([np.zeros(Lp, np.int64), np.repeat(np.arange(1, S + 1), Ls)])
    tp = np.concatenate([np.arange(Lp), np.tile(np.arange(Ls), S)])
    valid = np.concatenate([np.arange(Lp) >= pad, m.reshape(-1)])
    earlier = tp[None, :] <= tp[:, None]
    from_prefix = (seg[None, :] == 0) & ((seg[:, None] != 0) | earlier)
    same_suffix = (seg[None, :] == seg[:, None]) & (seg[:, None] != 0) & earlier
    vis = ((from_prefix | same_suffix) & valid[None, :]) | np.eye(N, dtype=bool)
    repidx = np.array([[p if p < Lp else Lp + s * Ls + (p - Lp) for p in range(Lp + Ls)] for s in range(S)], np.int64)
    return SimpleNamespace(Lp=Lp, S=S, Ls=Ls, N=N, N32=N32, pos=torch.as_tensor(pos[:N]).to(dev), pos32=torch.as_tensor(pos).to(dev),
                           amask=torch.as_tensor(vis).to(dev)[None, None], rowmask=t32(rowmask[:N]), rowmask32=t32(rowmask),
                           lastidx=torch.as_tensor(lastidx).to(dev), repidx=torch.as_tensor(repidx).to(dev), hist=t32(hist),
                           krange=t32(krange), chunks=t32(chunks), steps=t32(steps), walk_ptr=t32(walks), n_walks=1)
