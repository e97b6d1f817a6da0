"""Prefix-tree layout: oracle restatement and the C++ host builder against the reference's own outputs (golden file),
bit-exact. Runs without a GPU."""
import os

import numpy as np
import pytest
import torch

from ojb200 import trees
from oracle import layout as OL

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "layout_golden.npz"))
FIELDS = ("pos", "rowmask", "vbits", "src", "inv", "lastidx", "rep_ptr", "rep_pos", "hist", "canon")
CASES = trees.layout_cases()


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_reference_golden(name):
    seqs, groups, pad_id, NB, PB = CASES[name]
    lay = OL.gtree_layout(seqs, groups, pad_id, NB, PB)
    N, S, R, L2, Lr, Nreal = GOLD[f"{name}/meta"]
    assert (lay["N"], lay["S"], lay["R"], lay["L2"], lay["Lr"], lay["Nreal"]) == (N, S, R, L2, Lr, Nreal)
    assert np.array_equal(lay["ids"], GOLD[f"{name}/ids"])
    for f in FIELDS:
        a, b = lay[f], GOLD[f"{name}/{f}"]
        assert a.dtype == b.dtype and a.shape == b.shape and np.array_equal(a, b), f
    assert np.array_equal(np.packbits(lay["vis"], axis=1, bitorder="little"), GOLD[f"{name}/amask"])


@pytest.mark.parametrize("name", list(CASES))
def test_host_builder_matches_reference_golden(name):
    from ojb200 import layout as PL
    seqs, groups, pad_id, NB, PB = CASES[name]
    d, b64, b32, e32 = PL.gtree_host(seqs, groups, pad_id, NB, PB)
    N, S, R, L2, Lr, Nreal = GOLD[f"{name}/meta"]
    assert (d["N"], d["S"], d["R"], d["L2"], d["Lr"], d["Nreal"]) == (N, S, R, L2, Lr, Nreal)
    f = PL.field_views(d, b64, b32, e32)
    assert np.array_equal(f["ids"].numpy(), GOLD[f"{name}/ids"])
    for k in FIELDS:
        a, b = f[k].numpy(), GOLD[f"{name}/{k}"]
        assert a.dtype == b.dtype and a.shape == b.shape and np.array_equal(a, b), k
    # the packed buffers themselves are laid out as the reference's (32-byte aligned fields, zero padding)
    ref = OL.gtree_layout(seqs, groups, pad_id, NB, PB)
    parts = [ref[k].reshape(-1) for k in ("src", "inv", "rep_ptr", "rep_pos", "hist", "canon", "rowmask", "vbits")]
    want = np.concatenate([np.concatenate([p.astype(np.int32), np.zeros((-len(p)) % 8, np.int32)]) for p in parts])
    assert np.array_equal(b32.numpy(), want)


@pytest.mark.parametrize("name", list(CASES))
def test_extension_tables(name):
    """krange reproduces the visibility bits; chunks tile every node; the walk visits each chunk once, parents first."""
    from ojb200 import layout as PL
    seqs, groups, pad_id, NB, PB = CASES[name]
    d, b64, b32, e32 = PL.gtree_host(seqs, groups, pad_id, NB, PB)
    f = {k: v.numpy() for k, v in PL.field_views(d, b64, b32, e32).items()}
    ref = OL.gtree_layout(seqs, groups, pad_id, NB, PB)
    N = d["N"]
    vis = np.zeros((N, N), bool)
    for n in range(N):
        k = f["krange"][n]
        vis[n, 0:k[0]] = True
        vis[n, k[1]:k[2]] = True
        vis[n, k[3]:k[4]] = True
    assert np.array_equal(vis, ref["vis"])
    nc, ns = f["meta"][0], f["meta"][1]
    assert nc <= d["cap"] and ns == nc
    covered = np.zeros(N, int)
    for row0, rows, node, _ in f["chunks"][:nc]:
        assert 0 < rows <= 64
        n0, nl = f["nodes"][node][:2]
        assert n0 <= row0 and row0 + rows <= n0 + nl
        covered[row0:row0 + rows] += 1
    assert np.array_equal(covered, ref["rowmask"])
    seen, done_nodes = set(), set()
    for chunk, load, save, _ in f["steps"][:ns]:
        assert chunk not in seen
        seen.add(chunk)
        node = f["chunks"][chunk][2]
        parent = f["nodes"][node][2]
        if load in (2, 3):
            assert parent >= 0
        done_nodes.add(node)
    assert len(seen) == nc
    # level tables: every chunk once; a walk that loads a slot finds it exported by a walk of an earlier level
    S = d["S"]
    lw = f["lwalks"]
    assert lw[0] == 0 and lw[1 + 2 * S] == nc and all(lw[i] <= lw[i + 1] for i in range(1 + 2 * S))
    exported, seen = set(), set()
    for lo, hi in ((0, 1), (1, 1 + S), (1 + S, 1 + 2 * S)):
        new = set()
        for w in range(lo, hi):
            for s_ in range(lw[w], lw[w + 1]):
                chunk, load, save, aux = f["lsteps"][s_]
                assert chunk not in seen and save == 0
                seen.add(chunk)
                first = s_ == lw[w]
                assert load == (0 if not first else (4 if (aux >> 16) else 1))
                if aux >> 16:
                    assert (aux >> 16) - 1 in exported
                if aux & 0xffff:
                    new.add((aux & 0xffff) - 1)
        exported |= new
    assert len(seen) == nc


def test_rejects_bad_requests():
    from ojb200 import layout as PL
    with pytest.raises(RuntimeError):
        PL.gtree_host([[1, 2], []], [0, 0], 0)          # empty candidate
    with pytest.raises(RuntimeError):
        PL.gtree_host([[1, 2], [1, 3]], [0, 2], 0)      # question 1 has no candidate
    with pytest.raises(RuntimeError):
        PL.gtree_host([[1, 2]], [0], 0, NB=8)           # 8 rows: not a whole 32-key word
    with pytest.raises(RuntimeError):
        PL.gtree_host([], [], 0)


@pytest.mark.parametrize("name", list(trees.state_cases()))
def test_state_layout_oracle_matches_reference_golden(name):
    pre, suf, msk, pad = trees.state_cases()[name]
    lay = OL.state_layout(len(pre), msk, pad)
    Lp, S, Ls, N = GOLD[f"{name}/meta"]
    assert (lay["Lp"], lay["S"], lay["Ls"], lay["N"]) == (Lp, S, Ls, N)
    for f in ("pos", "rowmask", "lastidx", "repidx"):
        assert np.array_equal(lay[f], GOLD[f"{name}/{f}"]), f
    assert np.array_equal(np.packbits(lay["vis"], axis=1, bitorder="little"), GOLD[f"{name}/amask"])


@pytest.mark.parametrize("name", list(CASES))
def test_build_without_visibility_words(name):
    """OJB_LAYOUT_NO_VBITS: every other field and both other buffers are identical, the N x N/32 words are left untouched
    (the scorer neither builds nor uploads them: the attention kernel works from the O(N) key ranges)."""
    from ojb200 import layout as PL
    seqs, groups, pad_id, NB, PB = CASES[name]
    d1, a64, a32, ae = PL.gtree_host(seqs, groups, pad_id, NB, PB)
    d0, b64, b32, be = PL.gtree_host(seqs, groups, pad_id, NB, PB, vbits=False)
    N = d1["N"]
    assert d1["n32_used"] == a32.numel() and d0["n32_used"] == a32.numel() - (N * (N // 32) + 7) // 8 * 8
    assert {k: v for k, v in d0.items() if k != "n32_used"} == {k: v for k, v in d1.items() if k != "n32_used"}
    assert torch.equal(a64, b64) and torch.equal(ae, be)
    assert torch.equal(a32[:d0["n32_used"]], b32[:d0["n32_used"]])


def test_long_prefix_layout_is_linear_in_rows():
    """A 16 384-token shared prefix (the top of the length sweep): the O(N) build succeeds and its key ranges are causal."""
    from ojb200 import layout as PL
    seqs, groups = trees.make_tree(7, 16384, [12, 9], [5, 8, 3, 6], [0, 0, 1, 1], 4096)
    d, b64, b32, e32 = PL.gtree_host(seqs, groups, 0, 32, 16, vbits=False)
    assert d["N"] % 32 == 0 and d["Nreal"] == 16384 + 21 + 22 and d["n32_used"] < 40 * d["N"]
    f = PL.field_views(d, b64, b32, e32)
    kr = f["krange"].numpy()
    n = np.arange(d["Nreal"])
    assert np.all(kr[:16384, 0] == n[:16384] + 1)          # root rows: causal prefix
    assert np.all(kr[16384:d["Nreal"], 0] == 16384)        # every other row sees the whole root


def test_packed_requests_tables():
    """layout.pack_requests: the visibility implied by the shifted key ranges is block diagonal with each request's own
    visibility on the diagonal; histories, chunks and walk steps point into the request's own rows; one walk per request."""
    from ojb200 import layout as PL
    names = ["example", "doc", "ragged"]
    reqs = [(CASES[n][0], CASES[n][1]) for n in names]
    ids, lay, host = PL.pack_requests(reqs, 0, 32, 16, dev="cpu")
    refs = [OL.gtree_layout(s, g, 0, 32, 16) for s, g in reqs]
    assert lay.N == sum(r["N"] for r in refs) and lay.n_walks == 3 and lay.counts == [r["S"] for r in refs]
    kr = host["krange"].numpy()
    N = lay.N
    vis = np.zeros((N, N), bool)
    for n in range(N):
        a0, e0, a1, e1, a2, e2 = kr[n, 5], kr[n, 0], kr[n, 1], kr[n, 2], kr[n, 3], kr[n, 4]
        vis[n, a0:e0] = True
        vis[n, a1:e1] = True
        vis[n, a2:e2] = True
    base = 0
    hist, chunks, steps, walks = host["hist"].numpy(), host["chunks"].numpy(), host["steps"].numpy(), host["walk_ptr"].numpy()
    for i, r in enumerate(refs):
        n = r["N"]
        blk = vis[base:base + n, base:base + n]
        real = r["rowmask"].astype(bool)
        assert np.array_equal(blk[real], r["vis"][real])
        assert not vis[base:base + n, :base].any() and not vis[base:base + n, base + n:].any()
        h = hist[base:base + n]
        assert ((h == -1) | ((h >= base) & (h < base + n))).all()
        assert np.array_equal(np.where(h >= 0, h - base, -1), r["hist"][:n])
        st = steps[walks[i]:walks[i + 1]]
        rows = chunks[st[:, 0]]
        assert ((rows[:, 0] >= base) & (rows[:, 0] + rows[:, 1] <= base + n)).all()
        assert rows[:, 1].sum() == real.sum()                     # the walk of a request covers each of its real rows once
        assert np.array_equal(host["lastidx"].numpy()[sum(lay.counts[:i]):sum(lay.counts[:i + 1])], r["lastidx"] + base)
        base += n
