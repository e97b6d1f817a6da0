"""CPU restatement (torch, fp32 arithmetic on CPU tensors) of the non-GEMM operators of open-jev-fast's hot path.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline legs, never by
the product package. Every function follows the arithmetic and the bf16 rounding points of the reference kernel it names
(path inside open-jev-fast), so that a CUDA kernel can be compared element-wise; reduction order is the only freedom.

Pinning: the reference ships no golden vectors for these operators (its tests compare against the Hugging Face modules
on the real checkpoint). The functions here are pinned against those same Hugging Face `qwen3_5` modules on seeded
inputs in tests/test_oracle_hf.py.
"""
import torch

bf16 = torch.bfloat16


def rbf(x):
    """fp32 value after a round trip through bf16 (src/kernels.cu:14 rbf)."""
    return x.to(bf16).float()


def silu_f(x):
    """x / (1 + exp(-x)) in fp32 (src/kernels.cu:15)."""
    return x / (1.0 + torch.exp(-x))


def sigmoid_f(x):
    """1 / (1 + exp(-x)) in fp32 (src/kernels.cu:16)."""
    return 1.0 / (1.0 + torch.exp(-x))


def add_rmsnorm(x, delta, w1, rowmask, eps):
    """src/kernels.cu:41-73. x, delta bf16 [N, H]; w1 fp32 [H] (= 1 + weight); rowmask int32 [N] or None.
    Returns (h bf16, hn bf16)."""
    h = x.float() if delta is None else rbf(x.float() + delta.float())
    rstd = torch.rsqrt((h * h).sum(-1, keepdim=True) / h.shape[-1] + eps)
    hn = (h * rstd) * w1.float()
    if rowmask is not None:
        hn = hn * (rowmask != 0).float()[:, None]
    return h.to(bf16), hn.to(bf16)


def add_rmsnorm_sk(x, parts, w1, rowmask, eps):
    """src/kernels.cu:1444-1487. parts fp32 [S, N, H]: delta = bf16(sum over S in order)."""
    d = torch.zeros_like(parts[0])
    for s in range(parts.shape[0]):
        d = d + parts[s]
    return add_rmsnorm(x, d.to(bf16), w1, rowmask, eps)


def silu_mul(gu):
    """src/kernels.cu:76-89. gu bf16 [N, 2I] = [gate | up] -> bf16(bf16(silu(gate)) * up)."""
    I = gu.shape[1] // 2
    g, u = gu[:, :I].float(), gu[:, I:].float()
    return (rbf(silu_f(g)) * u).to(bf16)


def act_tables():
    """src/kernels.cu:1288-1295: (silu bf16[65536], sigmoid fp32[65536]) indexed by bf16 bit pattern."""
    bits = torch.arange(65536, dtype=torch.int32)
    x = (bits << 16).view(torch.float32)
    return silu_f(x).to(bf16), sigmoid_f(x)


def gate_mul(att, gate):
    """src/kernels.cu:362-376 / 1416-1430. att bf16 [HQ, T, D] (head-major), gate bf16 [T, HQ*D] ->
    y[T, HQ*D] = bf16(att * bf16(sigmoid(gate)))."""
    HQ, T, D = att.shape
    a = att.float().permute(1, 0, 2).reshape(T, HQ * D)
    return (a * rbf(sigmoid_f(gate.float()))).to(bf16)


def pack_bits(vis):
    """src/kernels.cu:4759-4766 / src/fastmodel.py:178-183. bool [N, N] -> int32 [N, N/32], bit b of word w = key 32w+b."""
    N = vis.shape[0]
    w = (vis.view(N, N // 32, 32).to(torch.int64) << torch.arange(32)).sum(-1)
    return (w - (w >= 2 ** 31).to(torch.int64) * 2 ** 32).to(torch.int32)


def fullattn_prep(proj, qw1, kw1, cosb, sinb, HQ, HKV, D, eps):
    """src/kernels.cu:302-359. proj bf16 [N, 2*HQ*D + 2*HKV*D]: per q head [q | gate], then k heads, then v heads.
    q, k: RMSNorm over D with fp32 (1+w) weights, rounded to bf16; rotary on the first RD dims with bf16 rounding after
    each product and after the sum (rotate-half pairing d <-> d + RD/2). Returns qt [HQ, N, D], kt, vt [HKV, N, D], gate
    [N, HQ*D], all bf16."""
    N = proj.shape[0]
    RD = cosb.shape[1]
    p = proj.float()
    qg = p[:, : HQ * 2 * D].view(N, HQ, 2, D)
    q, gate = qg[:, :, 0], qg[:, :, 1]
    k = p[:, HQ * 2 * D: HQ * 2 * D + HKV * D].view(N, HKV, D)
    v = p[:, HQ * 2 * D + HKV * D:].view(N, HKV, D)

    def norm_rope(x, w1):
        rstd = torch.rsqrt((x * x).sum(-1, keepdim=True) / D + eps)
        nv = rbf((x * rstd) * w1.float())
        rot, rest = nv[..., :RD], nv[..., RD:]
        half = torch.cat([-rot[..., RD // 2:], rot[..., : RD // 2]], -1)
        c, s = cosb.float()[:, None, :], sinb.float()[:, None, :]
        rot = rbf(rbf(rot * c) + rbf(half * s))
        return torch.cat([rot, rest], -1)

    qt = norm_rope(q, qw1).permute(1, 0, 2).contiguous().to(bf16)
    kt = norm_rope(k, kw1).permute(1, 0, 2).contiguous().to(bf16)
    vt = v.permute(1, 0, 2).contiguous().to(bf16)
    return qt, kt, vt, gate.reshape(N, HQ * D).contiguous().to(bf16)


def tree_attention(qt, kt, vt, gate, vis, scale):
    """src/kernels.cu:4287-4438 (fattn_k) as plain masked softmax attention in fp32: qt [HQ, N, D], kt / vt [HKV, N, D],
    vis bool [N, N] (row n sees key m). att = bf16(softmax(scale * q k^T + mask) v); y = bf16(att * bf16(sigmoid(gate))).
    The kernel rounds P to bf16 before P.V and uses exp2; those are below the comparison tolerance and not restated."""
    HQ, N, D = qt.shape
    HKV = kt.shape[0]
    rep = HQ // HKV
    k = kt.float().repeat_interleave(rep, 0)
    v = vt.float().repeat_interleave(rep, 0)
    s = torch.einsum("hnd,hmd->hnm", qt.float(), k) * scale
    s = s.masked_fill(~vis[None], float("-inf"))
    p = torch.softmax(s, -1)
    att = torch.einsum("hnm,hmd->hnd", p, v).to(bf16)
    return gate_mul(att, gate)


def linattn_prep(proj, hist, convw, A_log, dt_bias, KD, VD, HV, HK, HD):
    """Per packed row, src/kernels.cu:1173-1258 (linattn_prep_dedup2_k) without the scatter: causal depthwise conv of
    width 4 over the rows hist[n] = (t-3, t-2, t-1, t) of the row's own tree path (-1 = no row), fp32 accumulate in tap
    order, SiLU, bf16; q and k divided by sqrt(sum x^2 + 1e-6) per HD-wide head; beta = bf16(sigmoid(b));
    g = -exp(A_log) * softplus(a + dt_bias) in fp32 (softplus linear above 20).
    proj bf16 [N, 2KD + 2VD + 2HV] = [q | k | v | z | b | a]. Returns q, k bf16 [N, KD], v bf16 [N, VD], g fp32 [N, HV],
    beta bf16 [N, HV]."""
    N = proj.shape[0]
    C = 2 * KD + VD
    p = proj.float()
    x = p[:, :C]
    w = convw.float()                                      # [C, 4], tap 3 multiplies the row itself
    acc = torch.zeros(N, C)
    for i in range(4):
        idx = hist[:N, i].long()
        rows = torch.where((idx >= 0)[:, None], x[idx.clamp(min=0)], torch.zeros(1, C))
        acc = acc + w[:, i][None, :] * rows
    o = rbf(silu_f(acc))
    qk = o[:, : 2 * KD].view(N, 2 * HK, HD)
    qk = qk * (1.0 / torch.sqrt((qk * qk).sum(-1, keepdim=True) + 1e-6))
    q = qk[:, :HK].reshape(N, KD).to(bf16)
    k = qk[:, HK:].reshape(N, KD).to(bf16)
    v = o[:, 2 * KD:].to(bf16)
    b = p[:, C + VD: C + VD + HV]
    a = p[:, C + VD + HV: C + VD + 2 * HV]
    beta = sigmoid_f(b).to(bf16)
    xs = a + dt_bias.float()[None, :]
    sp = torch.where(xs > 20.0, xs, torch.log1p(torch.exp(xs)))
    g = -torch.exp(A_log.float())[None, :] * sp
    return q, k, v, g, beta


def scatter_slots(rows, src, fill=0.0):
    """Replicated layout of src/fastmodel.py:319: slot (s, t) holds packed row src[s, t], pad slots (-1) hold `fill`."""
    S, L2 = src.shape
    flat = src.reshape(-1).long()
    out = torch.full((S * L2,) + tuple(rows.shape[1:]), fill, dtype=rows.dtype)
    ok = flat >= 0
    out[ok] = rows[flat[ok]]
    return out


def gated_rmsnorm(o, z, w, eps):
    """src/kernels.cu:1333-1363. o bf16 [N, HV, HD] (GDN output), z bf16 [N, HV, HD] (gate columns of proj), w bf16 [HD]:
    bf16(((o * rstd) * w) * z * sigmoid(z)), rstd = 1/sqrt(mean(o^2) + eps) over HD. Returns bf16 [N, HV*HD]."""
    x = o.float()
    rstd = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    zz = z.float()
    y = ((x * rstd) * w.float()) * zz * sigmoid_f(zz)
    return y.reshape(o.shape[0], -1).to(bf16)
