"""Row-wise / element-wise CUDA kernels against the CPU oracle (oracle/ops.py), through the reference's op names."""
import pytest
import torch

from oracle import ops as O

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def _randn(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(bf16)


def _same(a, b, frac=0.995, atol_ulps=2):
    """bf16 outputs: at least `frac` bit-identical, the rest within a couple of bf16 ulps (reduction-order noise)."""
    a, b = a.float().cpu(), b.float().cpu()
    assert a.shape == b.shape
    if a.numel() == 0:
        return
    eq = (a == b).float().mean().item()
    err = (a - b).abs()
    tol = b.abs() * 2 ** -8 * atol_ulps + 1e-6
    assert bool((err <= tol).all()), (err.max().item(), eq)
    assert eq >= frac, eq


@pytest.mark.parametrize("N,H", [(5, 64), (33, 5120), (7, 8192), (0, 64)])
@pytest.mark.parametrize("with_delta,with_mask", [(False, False), (True, True), (True, False), (False, True)])
def test_add_rmsnorm(N, H, with_delta, with_mask):
    from ojb200 import ext as K
    x = _randn(N, H, seed=1)
    d = _randn(N, H, seed=2) if with_delta else None
    w1 = 1.0 + torch.randn(H, generator=torch.Generator().manual_seed(3)) * 0.02
    m = (torch.arange(N) % 3 != 0).to(torch.int32) if with_mask else None
    h, hn = K.add_rmsnorm(x.cuda(), None if d is None else d.cuda(), w1.cuda(), None if m is None else m.cuda(), 1e-6)
    rh, rhn = O.add_rmsnorm(x, d, w1, m, 1e-6)
    assert torch.equal(h.cpu(), rh)
    _same(hn, rhn)


@pytest.mark.parametrize("S", [1, 2, 3, 4])
def test_add_rmsnorm_sk(S):
    from ojb200 import ext as K
    N, H = 37, 5120
    x = _randn(N, H, seed=4)
    parts = torch.randn(S, N, H, generator=torch.Generator().manual_seed(5))
    w1 = 1.0 + torch.randn(H, generator=torch.Generator().manual_seed(6)) * 0.02
    m = (torch.arange(N) % 4 != 1).to(torch.int32)
    h, hn = K.add_rmsnorm_sk2(x.cuda(), parts.cuda(), w1.cuda(), m.cuda(), 1e-6)
    rh, rhn = O.add_rmsnorm_sk(x, parts, w1, m, 1e-6)
    assert torch.equal(h.cpu(), rh)
    _same(hn, rhn)


def test_act_tables_and_silu():
    from ojb200 import ext as K
    like = torch.zeros(1, device="cuda", dtype=bf16)
    st, sg = K.act_tables(like)
    rst, rsg = O.act_tables()
    fin = torch.isfinite(rst.float())
    # expf differs by <= 2 ulp between the CPU and the GPU: the bf16 table is compared bit-exactly where it can be
    _same(st.cpu()[fin], rst[fin], frac=0.99)
    assert torch.allclose(sg.cpu()[fin], rsg[fin], rtol=1e-6, atol=1e-7)
    gu = _randn(19, 2 * 1024, seed=7, scale=2.0)
    a = K.silu_mul(gu.cuda())
    b = K.silu_mul_lut(gu.cuda(), st)
    assert torch.equal(a, b)                 # table lookups are bit-identical to the computed kernel
    _same(a, O.silu_mul(gu), frac=0.99)


def test_gate_mul_strided():
    from ojb200 import ext as K
    T, HQ, D = 21, 6, 256
    att = _randn(1, HQ, T, D, seed=8)
    gate = _randn(T, HQ * D, seed=9)
    y = K.gate_mul2(att.cuda(), gate.cuda(), T, HQ, D)
    _same(y, O.gate_mul(att[0], gate), frac=0.99)
    # a transposed (strided) attention output, as SDPA returns it
    att_t = att.permute(0, 2, 1, 3).contiguous().cuda().permute(0, 2, 1, 3)
    sig = torch.zeros(65536, device="cuda")
    y2 = K.gate_mul3(att_t, gate.cuda(), sig, T, HQ, D)
    assert torch.equal(y, y2)


def test_pack_bits():
    from ojb200 import ext as K
    N = 96
    vis = torch.rand(N, N, generator=torch.Generator().manual_seed(10)) < 0.3
    out = K.pack_bits(vis.cuda())
    assert torch.equal(out.cpu(), O.pack_bits(vis))


@pytest.mark.parametrize("N,HQ,HKV,D,RD", [(45, 24, 4, 256, 64), (17, 4, 2, 128, 32), (9, 2, 1, 64, 16)])
def test_fullattn_prep(N, HQ, HKV, D, RD):
    from ojb200 import ext as K
    proj = _randn(N, 2 * HQ * D + 2 * HKV * D, seed=11)
    g = torch.Generator().manual_seed(12)
    qw1 = 1.0 + torch.randn(D, generator=g) * 0.02
    kw1 = 1.0 + torch.randn(D, generator=g) * 0.02
    ang = torch.rand(N, RD // 2, generator=g) * 6.28
    cosb = torch.cat([ang.cos(), ang.cos()], -1).to(bf16)
    sinb = torch.cat([ang.sin(), ang.sin()], -1).to(bf16)
    qt, kt, vt, gate = K.fullattn_prep2(proj.cuda(), qw1.cuda(), kw1.cuda(), cosb.cuda(), sinb.cuda(), 1, N, HQ, HKV, D, 1e-6)
    rq, rk, rv, rg = O.fullattn_prep(proj, qw1, kw1, cosb, sinb, HQ, HKV, D, 1e-6)
    assert torch.equal(vt[0].cpu(), rv) and torch.equal(gate.cpu(), rg)
    _same(qt[0], rq, frac=0.98)
    _same(kt[0], rk, frac=0.98)


def test_embed_rope_matches_torch_embedding_and_the_backbone_rotary_module():
    """ojb_embed_rope against what the reference's forward calls (src/fastmodel.py:404-405): torch's embedding lookup and the
    Hugging Face rotary module on text positions — bit for bit, including positions in the tens of thousands."""
    from ojb200 import ext as K, modelgen as MG
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5TextRotaryEmbedding
    cfg = MG.make_config(**dict(MG.SMALL, head_dim=256))
    rot = Qwen3_5TextRotaryEmbedding(cfg).cuda()
    g = torch.Generator().manual_seed(3)
    N, V, H = 96, 512, 256
    table = torch.randn(V, H, generator=g).to(torch.bfloat16).cuda()
    ids = torch.randint(0, V, (N,), generator=g).cuda()
    pos = torch.cat([torch.arange(40), torch.randint(0, 40000, (N - 40,), generator=g)]).cuda()
    x, cos, sin = K.embed_rope(ids, table, pos, rot.inv_freq.float().contiguous(), float(rot.attention_scaling))
    want_x = torch.nn.functional.embedding(ids, table)
    want_cos, want_sin = rot(want_x.view(1, N, H), pos.view(1, 1, N).expand(3, 1, N))
    assert torch.equal(x, want_x)
    assert torch.equal(cos, want_cos.reshape(N, -1)) and torch.equal(sin, want_sin.reshape(N, -1))
    bad = ids.clone()
    bad[5] = V + 7                                   # an id outside the table: a zero row, not a fault
    x2, _, _ = K.embed_rope(bad, table, pos, rot.inv_freq.float().contiguous(), 1.0)
    assert x2[5].abs().max().item() == 0 and torch.equal(x2[6:], want_x[6:])
