"""CPU restatement (numpy, explicit loops) of open-jev-fast's prefix-tree layouts.

TEST INFRASTRUCTURE ONLY (see oracle/ops.py). `gtree_layout` follows FastQwen35.gtree_build (src/fastmodel.py:321-398),
`state_layout` follows FastQwen35.tree_layout (src/fastmodel.py:247-264). Pinned bit-exactly against the outputs of the
reference's own functions stored in tests/golden/layout_golden.npz (made by tests/golden/make_layout_golden.py).
"""
import numpy as np


def _lcp(seqs, start, lim):
    """First index in [start, lim) where the sequences disagree, else lim (src/fastmodel.py:328)."""
    for i in range(start, lim):
        if any(s[i] != seqs[0][i] for s in seqs):
            return i
    return lim


def gtree_layout(seqs, groups, pad_id, NB=32, PB=16):
    """Returns a dict of numpy arrays with the reference's field names (plus scalars N, S, R, L2, Lr, Nreal and the dense
    bool `vis`)."""
    S = len(seqs)
    R = max(groups) + 1
    Lr = _lcp(seqs, 0, min(len(s) for s in seqs) - 1)                                  # :329
    q_len = []
    for r in range(R):                                                                 # :331-333
        gs = [seqs[c] for c in range(S) if groups[c] == r]
        q_len.append(_lcp(gs, Lr, min(len(s) for s in gs) - 1) - Lr)
    l_len = [len(seqs[c]) - Lr - q_len[groups[c]] for c in range(S)]                   # :334
    Nreal = Lr + sum(q_len) + sum(l_len)
    N = -(-Nreal // NB) * NB
    L2 = -(-max(len(s) for s in seqs) // PB) * PB                                      # :337
    q_begin, l_begin, off = [], [], Lr
    for r in range(R):
        q_begin.append(off)
        off += q_len[r]
    for c in range(S):
        l_begin.append(off)
        off += l_len[c]
    ids = np.full(N, pad_id, np.int64)
    pos = np.zeros(N, np.int64)
    valid = np.zeros(N, bool)
    node = np.full(N, 1 + R + S, np.int64)            # end padding = last node (:357-358)
    inv = np.zeros(N, np.int32)
    src = np.full((S, L2), -1, np.int32)
    last = np.zeros(S, np.int64)
    for i in range(Lr):                                                                # :344
        ids[i], pos[i], valid[i], node[i], inv[i] = seqs[0][i], i, True, 0, i
    first = {}
    for c in range(S):                                                                 # :346-351
        r = groups[c]
        first.setdefault(r, c)
        a = Lr + q_len[r]
        for i in range(Lr):
            src[c, i] = i
        for i in range(q_len[r]):
            src[c, Lr + i] = q_begin[r] + i
        for i in range(l_len[c]):
            n = l_begin[c] + i
            src[c, a + i] = n
            ids[n], pos[n], valid[n], node[n], inv[n] = seqs[c][a + i], a + i, True, 1 + R + c, c * L2 + a + i
        last[c] = l_begin[c] + l_len[c] - 1
    for r in range(R):                                                                 # :352-356
        c = first[r]
        for i in range(q_len[r]):
            n = q_begin[r] + i
            ids[n], pos[n], valid[n], node[n], inv[n] = seqs[c][Lr + i], Lr + i, True, 1 + r, c * L2 + Lr + i
    # CSR packed row -> slots, group N = pad slots (:364-366)
    buckets = [[] for _ in range(N + 1)]
    for slot, n in enumerate(src.reshape(-1)):
        buckets[n if n >= 0 else N].append(slot)
    rep_ptr = np.zeros(N + 2, np.int32)
    rep_pos = np.zeros(S * L2, np.int32)
    k = 0
    for n in range(N + 1):
        rep_ptr[n] = k
        for slot in buckets[n]:
            rep_pos[k] = slot
            k += 1
    rep_ptr[N + 1] = k
    hist = np.full((N + 1, 4), -1, np.int32)                                            # :368-373
    for n in range(N):
        if buckets[n]:
            sc, tc = divmod(buckets[n][0], L2)
            for i in range(4):
                if tc - 3 + i >= 0:
                    hist[n, i] = src[sc, tc - 3 + i]
    canon = np.full(S * L2, -1, np.int32)                                               # :375
    for n in range(N):
        if valid[n]:
            canon[inv[n]] = n
    parent = {0: -1}
    for r in range(R):
        parent[1 + r] = 0
    for c in range(S):
        parent[1 + R + c] = 1 + groups[c]
    parent[1 + R + S] = -1
    vis = np.zeros((N, N), bool)                                                        # :377-379
    for n in range(N):
        anc = set()
        p = parent[int(node[n])]
        while p >= 0:
            anc.add(p)
            p = parent[p]
        for m in range(N):
            v = (int(node[m]) in anc) or (node[m] == node[n] and m <= n)
            vis[n, m] = (v and valid[m]) or m == n
    vbits = np.packbits(vis, axis=1, bitorder="little").view("<i4").reshape(N, N // 32)  # :380
    return dict(N=N, S=S, R=R, L2=L2, Lr=Lr, Nreal=Nreal, ids=ids, pos=pos, lastidx=last, src=src, inv=inv, rep_ptr=rep_ptr,
                rep_pos=rep_pos, hist=hist, canon=canon, rowmask=valid.astype(np.int32), vbits=vbits, vis=vis,
                q_len=q_len, l_len=l_len, q_begin=q_begin, l_begin=l_begin)


def state_layout(Lp, suf_mask, pad=0):
    """Single-level tree [prefix | S suffixes of Ls rows] of src/fastmodel.py:247-264. suf_mask int [S, Ls]. The first
    `pad` prefix rows are left padding. Returns dict(pos, vis, rowmask, lastidx, repidx)."""
    suf_mask = np.asarray(suf_mask)
    S, Ls = suf_mask.shape
    N = Lp + S * Ls
    seg = np.zeros(N, np.int64)
    tpos = np.zeros(N, np.int64)
    valid = np.zeros(N, bool)
    for n in range(Lp):
        tpos[n], valid[n] = n, n >= pad
    for s in range(S):
        for t in range(Ls):
            n = Lp + s * Ls + t
            seg[n], tpos[n], valid[n] = s + 1, t, bool(suf_mask[s, t])
    pos = np.where(seg == 0, tpos - pad, tpos + (Lp - pad))
    vis = np.zeros((N, N), bool)
    for n in range(N):
        for m in range(N):
            if seg[m] == 0:
                v = seg[n] != 0 or tpos[m] <= tpos[n]
            else:
                v = seg[m] == seg[n] and tpos[m] <= tpos[n]
            vis[n, m] = (v and valid[m]) or n == m
    lastidx = np.array([Lp + s * Ls + int(suf_mask[s].sum()) - 1 for s in range(S)], np.int64)
    repidx = np.zeros((S, Lp + Ls), np.int64)
    for s in range(S):
        for p in range(Lp + Ls):
            repidx[s, p] = p if p < Lp else Lp + s * Ls + (p - Lp)
    return dict(Lp=Lp, S=S, Ls=Ls, N=N, pos=pos, vis=vis, rowmask=valid.astype(np.int32), lastidx=lastidx, repidx=repidx)
