"""Order of the work units of the block GEMM kernels (host side of csrc/gemm_units.cuh through ojb_gemm_unit_order): every
(x block or chunk, K range, w tile) occurs exactly once, the units of one w tile are adjacent, and with bands — x larger than
the L2 — every unit of a band comes before the units of the next band. No GPU."""
import ctypes

import numpy as np
import pytest

from ojb200 import _lib


def _order(n_xblk, tail_rows, n_xchunk, BN, N, splits, kb_total, band):
    lib = _lib.lib()
    fn = lib.ojb_gemm_unit_order
    fn.restype = ctypes.c_int64
    cap = 200000
    out = np.zeros((cap, 5), np.int32)
    n = fn(ctypes.c_int32(n_xblk), ctypes.c_int32(tail_rows), ctypes.c_int32(n_xchunk), ctypes.c_int32(BN), ctypes.c_int64(N),
           ctypes.c_int32(splits), ctypes.c_int32(kb_total), ctypes.c_int32(band), out.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
           ctypes.c_int64(cap))
    assert n >= 0, n
    return out[:n]


@pytest.mark.parametrize("n_xblk,tail_rows,n_xchunk,BN,N,splits,band", [
    (2, 32, 1, 256, 34816, 1, 0),        # the 544-row gate/up shape
    (2, 32, 1, 240, 12352, 1, 0),        # a w tile width that does not divide 256
    (2, 32, 1, 256, 5120, 2, 0),         # two K ranges
    (0, 288, 2, 256, 34816, 1, 0),       # every row in swapped-operand chunks
    (1, 288, 2, 256, 5120, 3, 0),        # block units plus two exact chunks
    (64, 0, 1, 256, 34816, 1, 13),       # 16 384 rows in five bands
    (64, 32, 1, 256, 34816, 1, 13),      # the same with a 32-row remainder
    (26, 0, 1, 192, 12352, 1, 9),        # bands of unequal size (9, 9, 8), narrower w tiles
    (64, 32, 1, 256, 5120, 2, 4),        # bands, K ranges and a remainder together
])
def test_every_unit_once_and_band_after_band(n_xblk, tail_rows, n_xchunk, BN, N, splits, band):
    kb_total = 80
    u = _order(n_xblk, tail_rows, n_xchunk, BN, N, splits, kb_total, band)
    n_wtile, n_wtile256 = -(-N // BN), -(-N // 256)
    blocks = u[u[:, 0] == 0]
    tails = u[u[:, 0] == 1]
    assert len(blocks) == n_xblk * n_wtile * splits
    assert len(tails) == (n_wtile256 * splits * n_xchunk if tail_rows else 0)
    assert len({(int(a), int(b), int(c)) for _, a, b, c, _ in blocks}) == len(blocks)          # (x block, K range, w tile) unique
    assert len({(int(b), int(c), int(d)) for _, _, b, c, d in tails}) == len(tails)             # (K range, w tile, x chunk) unique
    if len(blocks):
        assert blocks[:, 1].min() == 0 and blocks[:, 1].max() == n_xblk - 1 and blocks[:, 3].max() == n_wtile - 1
    if len(tails):
        assert tails[:, 3].max() == n_wtile256 - 1 and tails[:, 4].max() == n_xchunk - 1 and (tails[:, 1] == n_xblk).all()
    if band:
        b_of = blocks[:, 1] // band
        pos = np.flatnonzero(u[:, 0] == 0)
        assert (np.diff(b_of) >= 0).all()                                   # band after band
        if len(tails):
            assert np.flatnonzero(u[:, 0] == 1).min() > pos[b_of < b_of.max()].max()      # remainder units only in the last band
        for b in np.unique(b_of):                                            # inside a band: w tile after w tile
            assert (np.diff(blocks[b_of == b][:, 3]) >= 0).all()
    else:
        assert (np.diff(blocks[:, 3]) >= 0).all() if len(blocks) else True
    # a remainder unit follows block units of a w tile that overlaps its 256 w rows (its weight rows are in L2 by then)
    if len(blocks) and len(tails):
        for i in np.flatnonzero(u[:, 0] == 1)[:50]:
            prev = u[:i]
            prev = prev[prev[:, 0] == 0]
            t = int(u[i, 3])
            assert ((prev[:, 3] * BN < (t + 1) * 256) & ((prev[:, 3] + 1) * BN > t * 256 - BN)).any()


def test_rejects_bad_geometry():
    lib = _lib.lib()
    fn = lib.ojb_gemm_unit_order
    fn.restype = ctypes.c_int64
    out = np.zeros((4, 5), np.int32)
    p = out.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))
    assert fn(ctypes.c_int32(2), ctypes.c_int32(0), ctypes.c_int32(1), ctypes.c_int32(250), ctypes.c_int64(1024), ctypes.c_int32(1),
              ctypes.c_int32(8), ctypes.c_int32(0), p, ctypes.c_int64(4)) == -1                 # BN not a multiple of 16
    assert fn(ctypes.c_int32(2), ctypes.c_int32(0), ctypes.c_int32(1), ctypes.c_int32(256), ctypes.c_int64(1024), ctypes.c_int32(1),
              ctypes.c_int32(8), ctypes.c_int32(0), p, ctypes.c_int64(4)) == -4                 # more units than the buffer holds
