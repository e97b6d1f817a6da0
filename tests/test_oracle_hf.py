"""Pins the CPU oracle: the operator restatements (oracle/ops.py, oracle/gdn.py) and their packed-tree composition
(oracle/tree_forward.py) against the Hugging Face qwen3_5 modules, i.e. the reference's PyTorch path. CPU only."""
import pytest
import torch

from ojb200 import trees
from oracle import gdn as OG
from oracle import hf_path as OH
from oracle import layout as OL
from oracle import tree_forward as OT

bf16 = torch.bfloat16


def test_gdn_oracle_matches_hf_functions():
    from ojb200 import modelgen  # noqa: F401  (switches transformers to its pure-torch path)
    from transformers.models.qwen3_5 import modeling_qwen3_5 as M
    g_ = torch.Generator().manual_seed(0)
    T, H, D = 150, 4, 128
    q, k, v = (torch.randn(1, T, H, D, generator=g_) for _ in range(3))
    g = torch.nn.functional.logsigmoid(torch.randn(1, T, H, generator=g_))
    beta = torch.sigmoid(torch.randn(1, T, H, generator=g_))
    o_hf, s_hf = M.torch_chunk_gated_delta_rule(q, k, v, g, beta, output_final_state=True, use_qk_l2norm_in_kernel=True)
    o_hr, s_hr = M.torch_recurrent_gated_delta_rule(q, k, v, g, beta, None, True, use_qk_l2norm_in_kernel=True)
    qn, kn = M.l2norm(q[0]), M.l2norm(k[0])
    o1, s1 = OG.recurrent(qn, kn, v[0], g[0], beta[0], D ** -0.5)
    o2, s2 = OG.chunked(qn, kn, v[0], g[0], beta[0], D ** -0.5)
    for o, s in ((o1, s1), (o2, s2)):
        assert torch.allclose(o, o_hf[0], atol=2e-5, rtol=1e-4)
        assert torch.allclose(o, o_hr[0], atol=2e-5, rtol=1e-4)
        assert torch.allclose(s, s_hf[0], atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("case", ["doc", "nostem", "prefix_of"])
def test_packed_tree_forward_matches_per_candidate_hf(case):
    from ojb200 import modelgen as MG
    cfg = MG.make_config(**MG.SMALL)
    core = MG.build_core(cfg, device="cpu", seed=0, std=0.05, draw_on="cpu")
    seqs, groups, pad_id, NB, PB = trees.layout_cases()[case]
    seqs = [[t % cfg.vocab_size for t in s] for s in seqs]
    lay = OL.gtree_layout(seqs, groups, pad_id % cfg.vocab_size, NB, PB)
    hn = OT.forward_gtree(core, lay["ids"], lay)
    got = hn[torch.as_tensor(lay["lastidx"])].float()
    ref = OH.candidate_hidden(OH.prepare(core, upcast=True), seqs)
    rel = ((got - ref).norm() / ref.norm()).item()
    # bf16 activations between operators (the rounding points of the reference kernels) against an fp32 run: the yardstick
    # is what the Hugging Face model itself loses when it runs in bf16 (about 3e-2 on this narrow 8-layer model)
    noise = OH.candidate_hidden(OH.prepare(core, upcast=False), seqs)
    noise = ((noise - ref).norm() / ref.norm()).item()
    assert rel < 1.25 * noise, (rel, noise)


def test_packed_tree_forward_is_exact_in_fp32():
    """With every bf16 rounding switched off the packed forward equals the per-candidate Hugging Face run to fp32 accuracy:
    the tree semantics (conv history, ancestor mask, positions, state sharing) are those of independent sequences."""
    from ojb200 import modelgen as MG
    from oracle import ops as O
    cfg = MG.make_config(**MG.SMALL)
    core = MG.build_core(cfg, device="cpu", seed=1, std=0.05, draw_on="cpu").float()
    seqs, groups, pad_id, NB, PB = trees.layout_cases()["doc"]
    lay = OL.gtree_layout(seqs, groups, pad_id, NB, PB)
    saved = (O.rbf, O.bf16, OT.bf16)
    O.rbf, O.bf16, OT.bf16 = (lambda x: x), torch.float32, torch.float32
    try:
        hn = OT.forward_gtree(core, lay["ids"], lay)
    finally:
        O.rbf, O.bf16, OT.bf16 = saved
    got = hn[torch.as_tensor(lay["lastidx"])].float()
    ref = OH.candidate_hidden(core, seqs)
    assert ((got - ref).norm() / ref.norm()).item() < 1e-4


@pytest.mark.parametrize("mode,upcast", [("fp32", True), ("bf16", False)])
def test_streamed_oracle_equals_whole_model_forward(mode, upcast):
    """oracle/hf_stream.py applies the Hugging Face decoder layers one at a time (the 64-layer model of the benchmark cannot be
    held a second time in fp32); on a model that fits, it must reproduce the whole-model forward of oracle/hf_path.py."""
    from ojb200 import modelgen as MG
    from oracle import hf_stream as OS
    cfg = MG.make_config(**MG.SMALL)
    core = MG.build_core(cfg, device="cpu", seed=3, std=0.05, draw_on="cpu")
    seqs, groups, pad_id, NB, PB = trees.layout_cases()["doc"]
    ref = OH.candidate_hidden(OH.prepare(core, upcast=upcast), seqs)
    got = OS.candidate_hidden(core, seqs, mode=mode)
    assert ((got - ref).norm() / ref.norm()).item() < (1e-6 if upcast else 1e-9)
    # the operand-rounding floor sits between the fp32 run and the bf16 run
    if upcast:
        low = OS.candidate_hidden(core, seqs, mode="operands")
        b16 = OH.candidate_hidden(OH.prepare(core, upcast=False), seqs)
        e_low = ((low - ref).norm() / ref.norm()).item()
        e_b16 = ((b16 - ref).norm() / ref.norm()).item()
        assert 0 < e_low < e_b16, (e_low, e_b16)
