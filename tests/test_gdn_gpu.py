"""Gated DeltaNet kernels (prep, chunked core in replicated and tree-native form, gated norm) against the CPU oracle."""
import numpy as np
import pytest
import torch

from ojb200 import trees
from oracle import gdn as OG
from oracle import layout as OL
from oracle import ops as O

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def _inputs(T, HK, HV, seed):
    """Input distributions of the single-layer benchmark configuration: q/k unit-norm per head, v ~ N(0,1), g = logsigmoid(N(0,1)), beta = sigmoid(N(0,1))."""
    g_ = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(T, HK, 128, generator=g_), dim=-1).to(bf16)
    k = torch.nn.functional.normalize(torch.randn(T, HK, 128, generator=g_), dim=-1).to(bf16)
    v = torch.randn(T, HV, 128, generator=g_).to(bf16)
    g = torch.nn.functional.logsigmoid(torch.randn(T, HV, generator=g_))
    beta = torch.sigmoid(torch.randn(T, HV, generator=g_)).to(bf16)
    return q, k, v, g, beta


def _rel(a, b):
    return ((a.float().cpu() - b).norm() / b.norm()).item()


# bf16 operands of the chunk products (u, w, v', state copy) bound the error: the reference reports rel-L2 1-2e-3 against
# FLA for its own kernel; the acceptance bound for the final state is 1e-2 relative.
@pytest.mark.parametrize("B,T,HK,HV", [(1, 64, 1, 1), (2, 96, 2, 4), (3, 40, 1, 2), (1, 539, 2, 4), (7, 112, 2, 6)])
def test_gdn_replicated_vs_recurrent(B, T, HK, HV):
    from ojb200 import ext as K
    scale = 128 ** -0.5
    ins = [_inputs(T, HK, HV, 10 + b) for b in range(B)]
    q, k, v, g, beta = (torch.stack([x[i] for x in ins]).cuda() for i in range(5))
    o = K.gdn_fused6(q, k, v, g, beta, scale)
    torch.cuda.synchronize()
    assert o.shape == (B, T, HV, 128)
    for b in range(B):
        ref, _ = OG.recurrent(*ins[b], scale)
        assert _rel(o[b], ref) < 4e-3, (b, _rel(o[b], ref))
        assert (o[b].float().cpu() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()


def test_gdn_final_state_and_initial_state():
    """Prefix run exporting its final state, then suffixes started from it (the long-prefix hand-off of
    src/fastmodel.py:296-302), against one recurrent pass over prefix+suffix."""
    from ojb200 import ext as K
    HK, HV, Lp, Ls, S = 2, 4, 200, 48, 3
    scale = 128 ** -0.5
    pre = _inputs(Lp, HK, HV, 1)
    sufs = [_inputs(Ls, HK, HV, 2 + s) for s in range(S)]
    dev = "cuda"
    nc = (Lp + 63) // 64
    chunks = torch.tensor([[j * 64, min(64, Lp - j * 64), 0, 0] for j in range(nc)], dtype=torch.int32, device=dev)
    steps = torch.tensor([[j, 1 if j == 0 else 0, 0, 1 if j == nc - 1 else 0] for j in range(nc)], dtype=torch.int32, device=dev)
    walks = torch.tensor([0, nc], dtype=torch.int32, device=dev)
    fin = torch.zeros(1, HV, 128, 128, device=dev)
    o_pre = K.gdn_chunked(*(x.cuda() for x in pre), scale, chunks, steps, walks, 1, None, fin)
    ref_pre, ref_state = OG.recurrent(*pre, scale)
    assert _rel(o_pre, ref_pre) < 4e-3
    assert _rel(fin[0], ref_state) < 1e-2          # required: GDN final state within 1e-2 relative
    # suffixes: one chunk each, all starting from initial state 0
    cat = [torch.cat([s[i] for s in sufs]).cuda() for i in range(5)]
    chunks = torch.tensor([[s * Ls, Ls, 0, 0] for s in range(S)], dtype=torch.int32, device=dev)
    steps = torch.tensor([[s, 4, 0, 1 << 16] for s in range(S)], dtype=torch.int32, device=dev)
    walks = torch.arange(S + 1, dtype=torch.int32, device=dev)
    o_suf = K.gdn_chunked(*cat, scale, chunks, steps, walks, S, fin, None)
    for s in range(S):
        ref, _ = OG.recurrent(*sufs[s], scale, init=ref_state)
        assert _rel(o_suf[s * Ls:(s + 1) * Ls], ref) < 4e-3


@pytest.mark.parametrize("name", ["doc", "example", "baseline", "nostem", "ragged", "prefix_of"])
def test_gdn_tree_native_matches_per_path_recurrence(name):
    from ojb200 import ext as K
    from ojb200 import layout as PL
    seqs, groups, pad_id, NB, PB = trees.layout_cases()[name]
    ids, lay = PL.gtree_build(seqs, groups, pad_id, NB, PB, dev="cuda", dense=False)
    N, HK, HV = lay.N, 2, 4
    q, k, v, g, beta = _inputs(N, HK, HV, 5)
    scale = 128 ** -0.5
    o = K.gdn_tree(q.cuda().view(N, -1), k.cuda().view(N, -1), v.cuda().view(N, -1), g.cuda(), beta.cuda(), scale, lay)
    torch.cuda.synchronize()
    ref, _ = OG.tree(q, k, v, g, beta, scale, lay.src.cpu())
    real = lay.rowmask.cpu().bool()
    assert _rel(o[real.cuda()], ref[real]) < 4e-3
    assert float(o[~real.cuda()].float().abs().max()) == 0.0 if (~real).any() else True
    # the level-parallel state pass (root | stems | leaves, three launches) gives the same rows, and exports the root state
    o_lv = torch.zeros_like(o)
    _, states = K.gdn_tree_levels(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), scale, lay, o_lv)
    torch.cuda.synchronize()
    assert torch.equal(o_lv, o)
    if lay.Lr > 0:
        root = slice(0, lay.Lr)
        _, ref_root = OG.recurrent(q[root], k[root], v[root], g[root], beta[root], scale)
        assert _rel(states[0], ref_root) < 1e-2
    # the replicated-layout op on the same tree gives the same rows (two routes to one result)
    src = lay.src.cpu()
    rep = [O.scatter_slots(x, src) for x in (q, k, v, g, beta)]
    S, L2 = src.shape
    o_rep = K.gdn_fused6(*(x.cuda().view(S, L2, *x.shape[1:]) for x in rep), scale)
    o_rows = o_rep.view(S * L2, HV, 128)[lay.inv.long()]
    assert _rel(o_rows[real.cuda()], ref[real]) < 4e-3


@pytest.mark.parametrize("name", ["doc", "example"])
def test_prep_rows_and_scatter(name):
    from ojb200 import ext as K
    from ojb200 import layout as PL
    seqs, groups, pad_id, NB, PB = trees.layout_cases()[name]
    ids, lay = PL.gtree_build(seqs, groups, pad_id, NB, PB, dev="cuda", dense=False)
    N, HK, HV, HD = lay.N, 2, 4, 128
    KD, VD = HK * HD, HV * HD
    gen = torch.Generator().manual_seed(3)
    proj = torch.randn(N, 2 * KD + 2 * VD + 2 * HV, generator=gen).to(bf16)
    convw = (torch.randn(2 * KD + VD, 4, generator=gen) * 0.5).to(bf16)
    A_log = torch.log(torch.rand(HV, generator=gen) * 16).to(bf16)
    dt_bias = torch.ones(HV).to(bf16)
    rq, rk, rv, rg, rb = O.linattn_prep(proj, lay.hist.cpu(), convw, A_log, dt_bias, KD, VD, HV, HK, HD)
    real = lay.rowmask.cpu().bool()
    dq, dk, dv, dg, db = K.linattn_prep_rows(proj.cuda(), lay.hist, convw.cuda(), A_log.cuda(), dt_bias.cuda(), KD, VD, HV, HK, HD)

    def close(a, b, frac):
        a, b = a.float().cpu()[real], b.float()[real]
        assert bool(((a - b).abs() <= b.abs() * 2 ** -7 + 1e-6).all())
        assert (a == b).float().mean().item() >= frac
    close(dq, rq, 0.97); close(dk, rk, 0.97); close(dv, rv, 0.98); close(db, rb, 0.98)
    assert torch.allclose(dg.cpu()[real], rg[real], rtol=1e-5, atol=1e-6)
    # scattered form = the unreplicated rows placed at every slot, pad slots zero
    sq, sk, sv, sg, sb = K.linattn_prep_dedup2(proj.cuda(), lay.hist, lay.rep_ptr, lay.rep_pos, lay.L2, convw.cuda(), A_log.cuda(),
                                               dt_bias.cuda(), KD, VD, HV, HK, HD, False)
    src = lay.src.cpu()
    for got, rows in ((sq, dq), (sk, dk), (sv, dv), (sg, dg), (sb, db)):
        assert torch.equal(got.cpu(), O.scatter_slots(rows.cpu(), src))


def test_state_pass_bounded_wait_runs_out_and_reports_through_the_status_word():
    """The state pass waits for the bulk copies of each step's operands on an mbarrier, with the library's wait limit. With the
    limit at 50 ms and the host-side failure switch on, the copies of the second step are announced but never issued: the wait
    runs out, every CTA leaves its walk, the status word says so, and the next call on the same context is correct."""
    import ctypes
    import time
    from ojb200 import ext as K, _lib
    lib = _lib.lib()
    B, T, HK, HV = 2, 150, 2, 4
    g_ = torch.Generator().manual_seed(12)
    q = torch.nn.functional.normalize(torch.randn(B * T, HK, 128, generator=g_), dim=-1).to(bf16).cuda()
    k = torch.nn.functional.normalize(torch.randn(B * T, HK, 128, generator=g_), dim=-1).to(bf16).cuda()
    v = torch.randn(B * T, HV, 128, generator=g_).to(bf16).cuda()
    g = torch.nn.functional.logsigmoid(torch.randn(B * T, HV, generator=g_)).cuda()
    beta = torch.sigmoid(torch.randn(B * T, HV, generator=g_)).to(bf16).cuda()
    chunks, steps, walks = K._seq_tables(B, T, torch.device("cuda"))
    good = K.gdn_chunked(q, k, v, g, beta, 128 ** -0.5, chunks, steps, walks, B)
    torch.cuda.synchronize()
    _lib.check_status()
    try:
        assert lib.ojb_gemm_set_wait_limit_ms(ctypes.c_int32(50)) == 0
        assert lib.ojb_gemm_test_drop_copy(ctypes.c_int32(1)) == 0
        t0 = time.perf_counter()
        K.gdn_chunked(q, k, v, g, beta, 128 ** -0.5, chunks, steps, walks, B)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    finally:
        lib.ojb_gemm_test_drop_copy(ctypes.c_int32(0))
        lib.ojb_gemm_set_wait_limit_ms(ctypes.c_int32(0))
    assert dt < 1.5, dt                             # gave up after the 50 ms limit, not after the default 2 s
    with pytest.raises(RuntimeError, match="wait ran out"):
        _lib.check_status()
    again = K.gdn_chunked(q, k, v, g, beta, 128 ** -0.5, chunks, steps, walks, B)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(again, good)


def test_gated_rmsnorm():
    from ojb200 import ext as K
    N, HV, HD = 37, 4, 128
    gen = torch.Generator().manual_seed(4)
    x = torch.randn(50, HV, HD, generator=gen).to(bf16)
    P = 2 * 256 + 2 * HV * HD + 2 * HV
    proj = torch.randn(N, P, generator=gen).to(bf16)
    w = (1 + 0.02 * torch.randn(HD, generator=gen)).to(bf16)
    inv = torch.randint(0, 50, (N,), generator=gen).to(torch.int32)
    zoff = 2 * 256 + HV * HD
    y = K.gated_rmsnorm_inv2(x.cuda(), inv.cuda(), proj.cuda(), w.cuda(), None, HV, HD, zoff, 1e-6)
    ref = O.gated_rmsnorm(x[inv.long()], proj[:, zoff:zoff + HV * HD].view(N, HV, HD), w, 1e-6)
    a, b = y.float().cpu(), ref.float()
    assert bool(((a - b).abs() <= b.abs() * 2 ** -7 + 1e-6).all())
    assert (a == b).float().mean().item() > 0.98


@pytest.mark.parametrize("name,HK,HV", [(n, hk, hv) for n in ("doc", "baseline", "example", "nostem", "wide", "single", "ragged",
                                                               "prefix_of", "long") for hk, hv in ((2, 4), (4, 4))] +
                         [("baseline", 16, 32), ("wide", 16, 32)])     # model width: short chunks run two to a CTA there
def test_prep_fused_into_the_intra_pass_gives_the_same_bits(name, HK, HV):
    """ojb_gdn_chunked_proj (conv + SiLU + L2 norm + gates inside the first Gated DeltaNet launch) against ojb_gdn_prep followed
    by ojb_gdn_chunked on the same in-projection output: same arithmetic, so the same bits — outputs and exported final state,
    on every tree shape of the layout cases (single-row nodes, empty stems, nodes longer than a chunk, paired short chunks)."""
    from ojb200 import ext as K
    from ojb200 import layout as PL
    seqs, groups, pad_id, NB, PB = trees.layout_cases()[name]
    ids, lay = PL.gtree_build(seqs, groups, pad_id, NB, PB, dev="cuda", dense=False)
    N, HD = lay.N, 128
    KD, VD = HK * HD, HV * HD
    gen = torch.Generator().manual_seed(17)
    proj = torch.randn(N, 2 * KD + 2 * VD + 2 * HV, generator=gen).to(bf16).cuda()
    convw = (torch.randn(2 * KD + VD, 4, generator=gen) * 0.3).to(bf16).cuda()
    A_log = torch.log(torch.rand(HV, generator=gen) * 16 + 1e-3).to(bf16).cuda()
    dt_bias = torch.ones(HV).to(bf16).cuda()
    scale = HD ** -0.5
    q, k, v, g, beta = K.linattn_prep_rows(proj, lay.hist, convw, A_log, dt_bias, KD, VD, HV, HK, HD)
    fin_a = torch.zeros(1, HV, HD, HD, device="cuda")
    fin_b = torch.zeros(1, HV, HD, HD, device="cuda")
    steps = lay.steps.clone()
    w0, w1 = int(lay.walk_ptr[0]), int(lay.walk_ptr[1])
    steps[w1 - 1, 3] = steps[w1 - 1, 3] | 1                       # export the state after the last step of the walk
    want = torch.zeros(N, HV, HD, dtype=bf16, device="cuda")
    K.gdn_chunked(q.view(N, HK, HD), k.view(N, HK, HD), v.view(N, HV, HD), g, beta, scale, lay.chunks, steps, lay.walk_ptr, 1,
                  None, fin_a, want)
    got = torch.zeros(N, HV, HD, dtype=bf16, device="cuda")
    K.gdn_chunked_proj(proj, lay.hist, convw, A_log, dt_bias, KD, VD, HV, HK, scale, lay.chunks, steps, lay.walk_ptr, 1, None,
                       fin_b, got)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert torch.equal(fin_a, fin_b)
    assert float(want.float().abs().max()) > 0


def test_prep_refuses_projection_rows_that_are_not_16_byte_aligned():
    """The prep kernels read rows of proj 16 bytes at a time: a row length that is not a multiple of 8 elements (HV % 4 != 0)
    is refused by the entry points instead of being launched."""
    from ojb200 import ext as K
    HK = HV = 1
    N = 32
    proj = torch.zeros(N, 2 * 128 + 2 * 128 + 2, dtype=bf16, device="cuda")
    hist = torch.full((N + 1, 4), -1, dtype=torch.int32, device="cuda")
    convw = torch.zeros(3 * 128, 4, dtype=bf16, device="cuda")
    one = torch.ones(HV, dtype=bf16, device="cuda")
    with pytest.raises(RuntimeError):
        K.linattn_prep_rows(proj, hist, convw, one, one, 128, 128, HV, HK, 128)
