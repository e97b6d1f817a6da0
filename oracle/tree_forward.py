"""Packed prefix-tree forward composed from the operator restatements of oracle/ops.py and oracle/gdn.py (CPU, torch).

TEST INFRASTRUCTURE ONLY. Follows FastQwen35.forward_gtree of open-jev-fast (src/fastmodel.py:400-482) launch by launch,
with the GEMMs as fp32 matmuls of the bf16 operands rounded to bf16 where the reference's GEMMs write bf16. It ties the
per-operator restatements to the Hugging Face path: tests/test_oracle_hf.py checks that this packed forward gives the same
last-token hidden states as running every candidate as its own sequence through the Hugging Face model.
"""
import torch

from . import gdn as G
from . import ops as O

bf16 = torch.bfloat16


def _mm(x, w):
    return (x.float() @ w.float().t()).to(bf16)


@torch.no_grad()
def forward_gtree(core, ids, lay, exact_gdn=True):
    """core: Hugging Face Qwen3_5TextModel on CPU with bf16 weights; ids int64 [N]; lay: dict from oracle.layout.gtree_layout.
    Returns bf16 [N, H] (final norm applied) for all packed rows."""
    cfg = core.config
    eps = cfg.rms_norm_eps
    N = lay["N"]
    ids = torch.as_tensor(ids)
    pos = torch.as_tensor(lay["pos"])
    rowmask = torch.as_tensor(lay["rowmask"])
    hist = torch.as_tensor(lay["hist"])
    src = torch.as_tensor(lay["src"])
    vis = torch.as_tensor(lay["vis"])
    x = core.embed_tokens(ids).to(bf16)
    cos, sin = core.rotary_emb(x.view(1, N, -1), pos.view(1, 1, N).expand(3, 1, N))
    cos, sin = cos.reshape(N, -1).to(bf16), sin.reshape(N, -1).to(bf16)
    w1 = lambda n: 1.0 + n.weight.float()
    types = list(cfg.layer_types)
    lin = [t == "linear_attention" for t in types]
    h, hn = O.add_rmsnorm(x, None, w1(core.layers[0].input_layernorm), rowmask if lin[0] else None, eps)
    for i, L in enumerate(core.layers):
        if lin[i]:
            la = L.linear_attn
            KD, VD, HV, HK, HD = la.key_dim, la.value_dim, la.num_v_heads, la.num_k_heads, la.head_v_dim
            w_in = torch.cat([la.in_proj_qkv.weight, la.in_proj_z.weight, la.in_proj_b.weight, la.in_proj_a.weight], 0)
            proj = _mm(hn, w_in)
            q, k, v, g, beta = O.linattn_prep(proj, hist, la.conv1d.weight.squeeze(1), la.A_log, la.dt_bias, KD, VD, HV, HK, HD)
            o, _ = G.tree(q.view(N, HK, HD), k.view(N, HK, HD), v.view(N, HV, HD), g, beta, HD ** -0.5, src)
            z = proj[:, 2 * KD + VD: 2 * KD + 2 * VD].view(N, HV, HD)
            neps = getattr(la.norm, "eps", getattr(la.norm, "variance_epsilon", eps))
            y = O.gated_rmsnorm(o.to(bf16), z, la.norm.weight, neps)
            w_out = la.out_proj.weight
        else:
            sa = L.self_attn
            HQ, HKV, D = cfg.num_attention_heads, cfg.num_key_value_heads, sa.head_dim
            proj = _mm(hn, torch.cat([sa.q_proj.weight, sa.k_proj.weight, sa.v_proj.weight], 0))
            qt, kt, vt, gate = O.fullattn_prep(proj, w1(sa.q_norm), w1(sa.k_norm), cos, sin, HQ, HKV, D, eps)
            y = O.tree_attention(qt, kt, vt, gate, vis, sa.scaling)
            w_out = sa.o_proj.weight
        delta = (y.float() @ w_out.float().t())[None]
        h, hn = O.add_rmsnorm_sk(h, delta, w1(L.post_attention_layernorm), None, eps)
        gu = _mm(hn, torch.cat([L.mlp.gate_proj.weight, L.mlp.up_proj.weight], 0))
        m = O.silu_mul(gu)
        last = i == len(core.layers) - 1
        nw = w1(core.norm) if last else w1(core.layers[i + 1].input_layernorm)
        delta = (m.float() @ L.mlp.down_proj.weight.float().t())[None]
        h, hn = O.add_rmsnorm_sk(h, delta, nw, None if last or not lin[i + 1] else rowmask, eps)
    return hn
