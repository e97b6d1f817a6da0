"""Graph-per-shape serving shim: replay equals the eager forward, trees of the same key share one graph, the `noul`
convention, LRU eviction, and the scoring head against the oracle."""
import pytest
import torch

from ojb200 import trees
from oracle import hf_path as OH

pytestmark = pytest.mark.gpu


def _scorer(use_graph=True, max_graphs=4, A=2):
    from ojb200 import fastmodel as FM, modelgen as MG, server as SV
    cfg = MG.make_config(**MG.SMALL)
    core = MG.build_core(cfg, device="cpu", seed=3, std=0.05, draw_on="cpu")
    fast = FM.FastQwen35(core.to("cuda"))
    W, b = MG.make_head(cfg.hidden_size, A=A, seed=2, device="cuda")
    return cfg, fast, SV.Scorer(fast, W, b, pad_id=0, use_graph=use_graph, max_graphs=max_graphs), W, b


def _tree(seed, vocab):
    s, g = trees.make_tree(seed, 40, [5, 9], [3, 6, 2, 8], [0, 0, 1, 1], vocab)
    return s, g


def test_graph_replay_equals_eager_and_is_shared_by_key():
    cfg, fast, sc, W, b = _scorer()
    outs = []
    for seed in (1, 2, 3):
        seqs, groups = _tree(seed, cfg.vocab_size)
        got = sc.score_tokens(seqs, groups).clone()
        ids, lay = fast.gtree_build(seqs, groups, 0)
        want = fast.score_gtree(ids, lay, W, b)
        assert torch.equal(got, want)                       # same kernels, same inputs: bit-identical
        outs.append(got)
    assert len(sc.graphs) == 1                              # three different trees, one key, one graph
    assert not torch.equal(outs[0], outs[1])
    assert sc.last["launches"] > 0


def test_concurrent_callers_with_one_key_get_their_own_scores():
    """Two threads push different trees of the same key through one Scorer: the graph's output buffer is shared, so each
    caller must leave with a private copy taken under the lock (src/server.py:97,129 serialises and clones the same way)."""
    import threading
    cfg, fast, sc, W, b = _scorer()
    reqs = [_tree(seed, cfg.vocab_size) for seed in (1, 2, 3, 4)]
    want = [sc.score_tokens(*r).clone() for r in reqs]
    torch.cuda.synchronize()
    assert len(sc.graphs) == 1
    got = [[None] * 40 for _ in reqs]
    start = threading.Barrier(len(reqs))

    def client(i):
        start.wait()
        for j in range(40):
            got[i][j] = sc.forward([{"kind": "choice", "candidates": reqs[i][0][:2]},
                                    {"kind": "choice", "candidates": reqs[i][0][2:]}])
    ths = [threading.Thread(target=client, args=(i,)) for i in range(len(reqs))]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    for i in range(len(reqs)):
        for j in range(40):
            assert torch.equal(torch.cat(got[i][j]), want[i].cpu()), (i, j)


def test_capture_at_second_sight_runs_the_first_request_eagerly():
    """capture_after=2: a key's first request runs without tuning, warm-up or capture; the graph is taken when the key comes
    back, and from then on requests replay it."""
    from ojb200 import fastmodel as FM, modelgen as MG, server as SV
    cfg = MG.make_config(**MG.SMALL)
    fast = FM.FastQwen35(MG.build_core(cfg, device="cpu", seed=3, std=0.05, draw_on="cpu").to("cuda"))
    W, b = MG.make_head(cfg.hidden_size, A=2, seed=2, device="cuda")
    sc = SV.Scorer(fast, W, b, pad_id=0, capture_after=2)
    seqs, groups = _tree(1, cfg.vocab_size)
    outs, infos = [], []
    for _ in range(3):
        o, info = sc.score_tokens(seqs, groups, with_info=True)
        outs.append(o.clone())
        infos.append(info)
    ent = sc.graphs[infos[0]["key"]]
    assert [i["captured"] for i in infos] == [False, True, False] and ent.g is not None and ent.seen == 3
    assert torch.equal(outs[1], outs[2])                                  # capture pass and replay: same graph
    assert (outs[0] - outs[1]).abs().max().item() < 6e-2                  # eager run: cost-model kernels, not the tuned ones
    assert all(i["launches"] > 0 for i in infos)


def test_forward_records_noul_and_lru():
    cfg, fast, sc, W, b = _scorer(max_graphs=2, A=1)
    s1, g1 = _tree(5, cfg.vocab_size)
    recs = [{"kind": "choice", "candidates": s1[:2]}, {"kind": "noul", "candidates": s1[2:3]}]
    out = sc.forward(recs)
    assert out[0].shape == (2, 1) and out[1].shape == (2, 1)
    assert float(out[1][0]) == 0.0                          # noul -> [0, score]
    for n_root in (70, 110, 150):                           # three more keys -> the oldest graphs are evicted
        s, g = trees.make_tree(9, n_root, [4], [3, 5], [0, 0], cfg.vocab_size)
        sc.forward([{"kind": "choice", "candidates": s}])
    assert len(sc.graphs) == 2


def test_score_head_matches_oracle():
    from ojb200 import ext as K
    g = torch.Generator().manual_seed(0)
    hn = torch.randn(64, 256, generator=g).to(torch.bfloat16)
    rows = torch.tensor([3, 17, 63])
    W, b = torch.randn(5, 256, generator=g), torch.randn(5, generator=g)
    got = K.score_head(hn.cuda(), rows.cuda(), W.cuda(), b.cuda()).cpu()
    want = OH.scores(hn[rows].float(), W, b)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-4)


def test_packed_requests_match_separate_forwards():
    """Several requests in one forward: every request's scores and hidden rows equal those of its own forward up to the
    bf16 noise of differently blocked GEMMs (the row count of a GEMM decides its kernel and K split), the packed layout
    shifts the tables correctly (three different tree shapes, the second and third start at non-zero rows), and a second
    call with the same keys replays the captured graph."""
    cfg, fast, sc, W, b = _scorer(A=3)
    V = cfg.vocab_size
    reqs = [trees.make_tree(11, 40, [5, 9], [3, 6, 2, 8], [0, 0, 1, 1], V),
            trees.make_tree(12, 70, [4], [3, 5, 7], [0, 0, 0], V),
            trees.make_tree(13, 9, [0, 6], [2, 4, 3], [0, 1, 1], V)]
    packed = [o.clone() for o in sc.score_packed(reqs)]
    from ojb200 import layout as PL, _lib
    ids, lay, host = PL.pack_requests(reqs, 0, dev="cuda")
    hid = fast.forward_gtree(ids, lay, return_all=True).float()
    base = 0
    for (seqs, groups), got in zip(reqs, packed):
        i1, l1 = fast.gtree_build(seqs, groups, 0)
        want = fast.score_gtree(i1, l1, W, b)
        h1 = fast.forward_gtree(i1, l1, return_all=True).float()
        real = l1.rowmask.bool()
        rel = ((hid[base:base + l1.N][real] - h1[real]).norm() / h1[real].norm()).item()
        assert rel < 2.5e-2, rel
        assert got.shape == want.shape and (got - want).abs().max().item() < 6e-2
        base += l1.N
    _lib.check_status()
    n_graphs = len(sc.graphs)
    again = sc.score_packed(reqs)
    assert len(sc.graphs) == n_graphs and not sc.last["captured"]
    assert all(torch.equal(a, p) for a, p in zip(again, packed))


def test_state_route_matches_tree_route():
    """One question over a long shared context through EntryState (tree_layout / forward_tree, src/server.py:50-70,100-115)
    gives the scores of the general tree route; a second request of the same key (other tokens, other suffix lengths)
    replays the graph."""
    cfg, fast, sc, W, b = _scorer(A=2)
    V = cfg.vocab_size
    for seed, leaf in ((21, [3, 6, 2, 8, 5]), (22, [7, 1, 4, 8, 2])):
        seqs, groups = trees.make_tree(seed, 150, [0], leaf, [0] * 5, V)
        got = sc.score_state(seqs).clone()
        want = sc.score_tokens(seqs, groups).clone()
        assert got.shape == want.shape == (5, 2)
        assert (got - want).abs().max().item() < 6e-2, (got, want)
    from ojb200 import _lib
    _lib.check_status()
    assert sum(1 for k in sc.graphs if k[0] == "state") == 1
