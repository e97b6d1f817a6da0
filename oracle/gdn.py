"""CPU restatement (torch fp32) of the Gated DeltaNet core of open-jev-fast's hot path.

TEST INFRASTRUCTURE ONLY (see oracle/ops.py). The reference runs this operator through src/kernels.cu:4225 (gdn_fused6)
or FLA's chunk_gated_delta_rule (src/fastmodel.py:226,447); both implement the gated delta rule that the Hugging Face
`qwen3_5` module states in plain torch (torch_chunk_gated_delta_rule / torch_recurrent_gated_delta_rule), which is what
"the reference's PyTorch path" executes. `recurrent` is the per-token definition, `chunked` the chunk-of-64 algebra the
kernels use; tests/test_oracle_hf.py pins both against the Hugging Face functions.
"""
import torch


def recurrent(q, k, v, g, beta, scale, init=None):
    """q, k [T, HK, D]; v [T, HV, D]; g, beta [T, HV] (g = natural-log decay <= 0). HV % HK == 0 (grouped value heads:
    value head h uses key head h // (HV/HK), src/fastmodel.py:421). Per token and head, with state S [D(k), D(v)]:
        S <- S * exp(g_t);  delta = (v_t - S^T k_t) * beta_t;  S <- S + k_t delta^T;  o_t = scale * S^T q_t.
    Returns (o fp32 [T, HV, D], final state fp32 [HV, D, D])."""
    T, HK, D = k.shape
    HV = v.shape[1]
    rep = HV // HK
    qf = q.float().repeat_interleave(rep, 1)
    kf = k.float().repeat_interleave(rep, 1)
    vf, gf, bf = v.float(), g.float(), beta.float()
    S = torch.zeros(HV, D, D) if init is None else init.float().clone()
    o = torch.zeros(T, HV, D)
    for t in range(T):
        S = S * torch.exp(gf[t])[:, None, None]
        mem = torch.einsum("hkv,hk->hv", S, kf[t])
        delta = (vf[t] - mem) * bf[t][:, None]
        S = S + kf[t][:, :, None] * delta[:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, qf[t]) * scale
    return o, S


def chunked(q, k, v, g, beta, scale, init=None, chunk=64):
    """Same function through the chunk algebra (zero-padded to a multiple of `chunk`): per chunk with G = cumsum(g),
    A = strict_lower((k beta) k^T * exp(G_i - G_j)), T = (I + A)^-1, u = T (v beta), w = T (k beta e^G),
    v' = u - w S, o = scale * ((q e^G) S + tril(q k^T * exp(G_i - G_j)) v'), S <- S e^(G_L) + (k e^(G_L - G))^T v'."""
    T0, HK, D = k.shape
    HV = v.shape[1]
    rep = HV // HK
    pad = (-T0) % chunk
    z = lambda x: torch.cat([x.float(), torch.zeros((pad,) + tuple(x.shape[1:]))], 0)
    qf, kf = z(q).repeat_interleave(rep, 1), z(k).repeat_interleave(rep, 1)
    vf, gf, bf = z(v), z(g), z(beta)
    S = torch.zeros(HV, D, D) if init is None else init.float().clone()
    out = torch.zeros(T0 + pad, HV, D)
    eye = torch.eye(chunk)
    for c0 in range(0, T0 + pad, chunk):
        sl = slice(c0, c0 + chunk)
        qc, kc, vc = (x[sl].permute(1, 0, 2) for x in (qf, kf, vf))          # [HV, C, D]
        bc, G = bf[sl].t(), gf[sl].t().cumsum(-1)                            # [HV, C]
        gam = torch.exp(G[:, :, None] - G[:, None, :]).tril()
        A = ((kc * bc[:, :, None]) @ kc.transpose(1, 2) * gam).tril(-1)
        Tm = torch.linalg.solve_triangular(eye + A, eye.expand(HV, -1, -1).clone(), upper=False)
        u = Tm @ (vc * bc[:, :, None])
        w = Tm @ (kc * (bc * torch.exp(G))[:, :, None])
        vn = u - w @ S
        o = (qc * torch.exp(G)[:, :, None]) @ S + ((qc @ kc.transpose(1, 2)) * gam).tril() @ vn
        out[sl] = (o * scale).permute(1, 0, 2)
        S = S * torch.exp(G[:, -1])[:, None, None] + (kc * torch.exp(G[:, -1:] - G)[:, :, None]).transpose(1, 2) @ vn
    return out[:T0], S


def tree(q, k, v, g, beta, scale, src):
    """Per packed row of a prefix tree: every candidate path src[s] (-1 padded, src/fastmodel.py:346-348) is run through
    `recurrent` from a zero state; row n takes the output of the first path that contains it. Returns
    (o fp32 [N, HV, D], final states fp32 [S, HV, D, D])."""
    N = q.shape[0]
    o = torch.zeros(N, v.shape[1], v.shape[2])
    done = torch.zeros(N, dtype=torch.bool)
    finals = []
    for s in range(src.shape[0]):
        rows = src[s][src[s] >= 0].long()
        os_, fs = recurrent(q[rows], k[rows], v[rows], g[rows], beta[rows], scale)
        new = ~done[rows]
        o[rows[new]] = os_[new]
        done[rows] = True
        finals.append(fs)
    return o, torch.stack(finals)
