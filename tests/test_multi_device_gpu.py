"""One process driving two GPUs: launch state that CUDA keeps per device (opt-in shared memory, SM count, status words,
capture streams) must follow the device of the call. Skipped on a box with one GPU. Plain loads only; nothing crosses
between the devices."""
import threading

import pytest
import torch

from ojb200 import trees

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16

needs_two = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")


@needs_two
def test_operators_on_second_device_match_first():
    from ojb200 import ext as K, lt_ext as LT, _lib
    g_ = torch.Generator().manual_seed(5)
    x = (torch.randn(96, 1024, generator=g_) * 0.5).to(bf16)
    w = (torch.randn(512, 1024, generator=g_) * 0.05).to(bf16)
    T, HK, HV = 150, 2, 4
    q = torch.nn.functional.normalize(torch.randn(T, HK, 128, generator=g_), dim=-1).to(bf16)
    k = torch.nn.functional.normalize(torch.randn(T, HK, 128, generator=g_), dim=-1).to(bf16)
    v = torch.randn(T, HV, 128, generator=g_).to(bf16)
    gl = torch.nn.functional.logsigmoid(torch.randn(T, HV, generator=g_))
    beta = torch.sigmoid(torch.randn(T, HV, generator=g_)).to(bf16)
    N, HQ, HKV, D = 64, 12, 2, 256
    qt = torch.randn(1, HQ, N, D, generator=g_).to(bf16)
    kt = torch.randn(1, HKV, N, D, generator=g_).to(bf16)
    vt = torch.randn(1, HKV, N, D, generator=g_).to(bf16)
    gate = torch.randn(N, HQ * D, generator=g_).to(bf16)
    kr = torch.zeros(N, 8, dtype=torch.int32)
    kr[:, 0] = torch.arange(1, N + 1)            # causal: root range [0, row + 1)
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        with torch.cuda.device(dev):
            mm = LT.lt_matmul(x.to(dev), w.to(dev), 0)
            chunks, steps, walks = K._seq_tables(1, T, torch.device(dev))
            o = K.gdn_chunked(q.to(dev), k.to(dev), v.to(dev), gl.to(dev), beta.to(dev), 128 ** -0.5, chunks, steps, walks, 1)
            a1 = K.fattn_tree_ranges(qt.to(dev), kt.to(dev), vt.to(dev), gate.to(dev), kr.to(dev), D ** -0.5, 6)
            a2 = K.fattn_tree_tc(qt.to(dev), kt.to(dev), vt.to(dev).transpose(2, 3).contiguous(), gate.to(dev), kr.to(dev), D ** -0.5)
            torch.cuda.synchronize(dev)
            _lib.check_status(dev)
            outs.append((mm.cpu(), o.cpu(), a1.cpu(), a2.cpu()))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    rel = ((outs[0][2].float() - outs[0][3].float()).norm() / outs[0][2].float().norm()).item()
    assert rel < 6e-3, rel                       # the two attention kernels agree (both are within 4e-3 of the fp32 softmax)
    want = x.float() @ w.float().T
    assert (outs[0][0].float() - want).abs().max() <= 2 ** -8 * want.abs().max() + 1e-3


@needs_two
def test_two_scorers_behind_the_router_capture_and_replay_on_their_own_devices(monkeypatch):
    """Both workers capture their first graphs at the same time (each on its own capture stream) and every request's scores
    equal those of a single-GPU scorer with the same weights (kernel choice by the cost model, not by timing, so that both
    devices run the same kernels)."""
    from ojb200 import fastmodel as FM, modelgen as MG, router as RT, server as SV
    monkeypatch.setattr(FM.FastQwen35, "TUNE_MAX_ROWS", 0)
    cfg = MG.make_config(**MG.SMALL)
    scorers = []
    for i in range(2):
        dev = torch.device("cuda", i)
        with torch.cuda.device(dev):
            core = MG.build_core(cfg, device="cpu", seed=3, std=0.05, draw_on="cpu")
            fast = FM.FastQwen35(core.to(dev))
            W, b = MG.make_head(cfg.hidden_size, A=2, seed=2, device=dev)
            scorers.append(SV.Scorer(fast, W, b, pad_id=0, device=dev, max_graphs=64))
    reqs = [trees.make_tree(30 + i, 40 + 13 * (i % 5), [5, 9], [3, 6, 2, 8], [0, 0, 1, 1], cfg.vocab_size) for i in range(12)]

    def serve(i):
        def fn(req):
            out = scorers[i].score_tokens(req[0], req[1]).cpu()
            from ojb200 import _lib
            _lib.check_status(scorers[i].device)
            return i, out
        return fn
    router = RT.Router([serve(0), serve(1)])
    try:
        got = router.map(reqs) + router.map(reqs)
        st = router.stats()
    finally:
        router.close()
    assert st["alive"] == [True, True] and st["errors"] == [] and min(st["served"]) > 0, st
    for (i, out), req in zip(got, reqs + reqs):
        want = scorers[0].score_tokens(req[0], req[1]).cpu()
        assert out.shape == want.shape
        assert torch.equal(out, want), (i, out, want)
