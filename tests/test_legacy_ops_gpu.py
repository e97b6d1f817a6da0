"""Older operator variants of the reference's op list (src/ext.py:8-45) served by the production kernels: each one under the
layout contract of its name — which rows its convolution history follows, whether q / k come on the key heads or expanded to
the value heads, replicated slots or packed rows."""
import pytest
import torch

from ojb200 import trees
from oracle import ops as O

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16
KD, VD, HV, HK, HD = 256, 512, 4, 2, 128


def _weights(seed=0):
    g = torch.Generator().manual_seed(seed)
    convw = (torch.randn(2 * KD + VD, 4, generator=g) * 0.3).to(bf16).cuda()
    A_log = torch.log(torch.rand(HV, generator=g) * 16 + 1e-3).to(bf16).cuda()
    dt_bias = torch.ones(HV).to(bf16).cuda()
    return convw, A_log, dt_bias, g


def _expand(x):
    return x.view(-1, HK, 1, HD).expand(-1, HK, HV // HK, HD).reshape(-1, HV * HD)


def _close(a, b, tol=2 ** -7):
    assert a.shape == b.shape, (a.shape, b.shape)
    assert (a.float() - b.float()).abs().max().item() <= tol * max(1.0, b.float().abs().max().item())


def test_sequence_preps_follow_each_sequence_and_the_l2_switch():
    from ojb200 import ext as K
    convw, A_log, dt_bias, g = _weights()
    B, T = 3, 37
    proj = torch.randn(B * T, 2 * KD + 2 * VD + 2 * HV, generator=g).to(bf16).cuda()
    hist = torch.full((B * T + 1, 4), -1, dtype=torch.int32)
    for n in range(B * T):
        for i in range(4):
            if n % T - 3 + i >= 0:
                hist[n, i] = n - 3 + i
    rq, rk, rv, rg, rb = O.linattn_prep(proj.cpu(), hist, convw.cpu(), A_log.cpu(), dt_bias.cpu(), KD, VD, HV, HK, HD)
    q, k, v, gg, beta = K.linattn_prep2(proj, convw, A_log, dt_bias, B, T, KD, VD, HV, HK, HD, True)
    _close(q.cpu(), _expand(rq)), _close(k.cpu(), _expand(rk)), _close(v.cpu(), rv), _close(beta.cpu(), rb)
    assert torch.allclose(gg.cpu(), rg, rtol=1e-4, atol=1e-5)
    q0, k0, v0, _, _ = K.linattn_prep(proj, convw, A_log, dt_bias, T, KD, VD, HV, HK, HD)          # no L2 norm
    assert q0.shape == (B * T, HV * HD) and torch.equal(v0, v)
    qn = torch.nn.functional.normalize(q0.float().view(-1, HV, HD), dim=-1).reshape(B * T, -1)
    _close(qn.cpu(), _expand(rq), tol=2 ** -6)
    q1 = K.linattn_prep2(proj, convw, A_log, dt_bias, B, T, KD, VD, HV, HK, HD, False)[0]
    assert torch.equal(q1, q0)


def test_single_level_tree_preps_and_the_row_map_of_the_gated_norm():
    from ojb200 import ext as K
    convw, A_log, dt_bias, g = _weights(1)
    Lp, S, Ls = 21, 3, 8
    N = Lp + S * Ls
    proj = torch.randn(N, 2 * KD + 2 * VD + 2 * HV, generator=g).to(bf16).cuda()
    q, k, v, gg, beta = K.linattn_prep_tree(proj, convw, A_log, dt_bias, Lp, S, Ls, KD, VD, HV, HK, HD)
    # oracle: every suffix as the continuation of the prefix
    for s in range(S):
        rows = list(range(Lp)) + list(range(Lp + s * Ls, Lp + (s + 1) * Ls))
        sub = proj[rows].cpu()
        hist = torch.full((len(rows) + 1, 4), -1, dtype=torch.int32)
        for n in range(len(rows)):
            for i in range(4):
                if n - 3 + i >= 0:
                    hist[n, i] = n - 3 + i
        rq, rk, rv, rg, rb = O.linattn_prep(sub, hist, convw.cpu(), A_log.cpu(), dt_bias.cpu(), KD, VD, HV, HK, HD)
        _close(q[rows].cpu(), _expand(rq)), _close(v[rows].cpu(), rv), _close(k[rows].cpu(), _expand(rk))
    qr, kr, vr, gr, br = K.linattn_prep_rep(proj, convw, A_log, dt_bias, Lp, S, Ls, KD, VD, HV, HK, HD)
    assert qr.shape == (S * (Lp + Ls), HV * HD) and vr.shape == (S * (Lp + Ls), VD)
    for s in range(S):
        rows = list(range(Lp)) + list(range(Lp + s * Ls, Lp + (s + 1) * Ls))
        sl = slice(s * (Lp + Ls), (s + 1) * (Lp + Ls))
        assert torch.equal(qr[sl], q[rows]) and torch.equal(vr[sl], v[rows]) and torch.equal(gr[sl], gg[rows])
    # gated norm reading the replicated output back through the row map == gated norm of the packed rows
    x_rep = torch.randn(S * (Lp + Ls), HV, HD, generator=g).to(bf16).cuda()
    w = (1 + 0.02 * torch.randn(HD, generator=g)).to(bf16).cuda()
    zoff = 2 * KD + VD
    got = K.gated_rmsnorm_map(x_rep, proj, w, HV, HD, zoff, 1e-6, Lp, Ls)
    idx = [n if n < Lp else ((n - Lp) // Ls) * (Lp + Ls) + Lp + (n - Lp) % Ls for n in range(N)]
    want = K.gated_rmsnorm(x_rep[idx].contiguous(), proj, w, HV, HD, zoff, 1e-6)
    assert torch.equal(got, want)


def test_src_mapped_preps_equal_the_production_prep_and_fused5_equals_its_two_halves():
    from ojb200 import ext as K, layout as PL
    convw, A_log, dt_bias, g = _weights(2)
    seqs, groups, pad_id, NB, PB = trees.layout_cases()["ragged"]
    ids, lay = PL.gtree_build(seqs, groups, pad_id, NB, PB, dev="cuda", dense=False)
    N, S, L2 = lay.N, lay.S, lay.L2
    proj = torch.randn(N, 2 * KD + 2 * VD + 2 * HV, generator=g).to(bf16).cuda()
    want = K.linattn_prep_dedup2(proj, lay.hist, lay.rep_ptr, lay.rep_pos, L2, convw, A_log, dt_bias, KD, VD, HV, HK, HD, False)
    got2 = K.linattn_prep_map2(proj, lay.src, convw, A_log, dt_bias, KD, VD, HV, HK, HD, 4)
    gotd = K.linattn_prep_dedup(proj, lay.src, lay.rep_ptr, lay.rep_pos, convw, A_log, dt_bias, KD, VD, HV, HK, HD)
    for a, b, c in zip(want, got2, gotd):
        assert torch.equal(a, b) and torch.equal(a, c)
    got1 = K.linattn_prep_map(proj, lay.src, convw, A_log, dt_bias, KD, VD, HV, HK, HD)
    assert torch.equal(got1[0], _expand(want[0])) and torch.equal(got1[2], want[2])
    q, k, v, gg, beta = want
    args = (q.view(S, L2, HK, HD), k.view(S, L2, HK, HD), v.view(S, L2, HV, HD), gg.view(S, L2, HV), beta.view(S, L2, HV), HD ** -0.5)
    w = (1 + 0.02 * torch.randn(HD, generator=g)).to(bf16).cuda()
    zoff = 2 * KD + VD
    y5 = K.gdn_fused5(*args, proj, zoff, w, None, lay.canon, lay.rowmask, 1e-6)
    o = K.gdn_fused6(*args)
    y2 = K.gated_rmsnorm_inv2(o, lay.inv, proj, w, None, HV, HD, zoff, 1e-6)
    assert y5.shape == (N, VD)
    real = lay.rowmask.bool()
    assert torch.equal(y5[real], y2[real]) and float(y5[~real].abs().max()) == 0.0
    assert torch.equal(K.gdn_fused7(*args, proj, zoff, w, None, lay.canon, lay.rowmask, 1e-6), y5)
    ts = K.gdn_fused6ts(*args)
    assert ts.shape == (S * HV, 16) and ts.dtype == torch.int64
    K.l2_prefetch(proj, 65536)
    torch.cuda.synchronize()
    from ojb200 import _lib
    _lib.check_status()
