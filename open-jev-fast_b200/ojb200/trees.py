"""Seeded synthetic request trees used by the parity tests, the golden-vector generator and the benchmark.

Token ids are uniform random integers; only the shape of a request (how many questions and candidates, how long the shared
root, the question stems and the candidate tails are) follows the workloads the benchmark is quoted on. No benchmark text.
"""
import numpy as np


def make_tree(seed, root_len, q_lens, leaf_lens, groups, vocab=4096):
    """Candidate token lists for a two-level tree: shared root, one stem per question, one tail per candidate.
    Distinct first tokens are forced at every branching point so that the tree found by the layout builder is the one
    asked for. Returns (seqs, groups)."""
    rng = np.random.default_rng(seed)
    root = rng.integers(8, vocab, root_len).tolist()
    stems = []
    for r, ql in enumerate(q_lens):
        s = rng.integers(8, vocab, ql).tolist()
        if ql:
            s[0] = 8 + r                      # stems differ at their first token
        stems.append(s)
    seqs = []
    per_group = {}
    for c, (ll, r) in enumerate(zip(leaf_lens, groups)):
        t = rng.integers(8 + 64, vocab, ll).tolist()
        t[0] = 8 + 64 + per_group.get(r, 0) + (0 if q_lens[r] else 16 * r)   # tails of one question differ at once
        per_group[r] = per_group.get(r, 0) + 1
        seqs.append(root + stems[r] + t)
    return seqs, list(groups)


def baseline_tree(seed=0, vocab=4096):
    """The benchmark tree: 420-token root, 3 question nodes of about 25 tokens, 7 leaves of 4-12 tokens = 539 rows."""
    rng = np.random.default_rng(1000 + seed)
    q_lens = [24, 25, 26]
    groups = [0, 0, 0, 1, 2, 2, 2]
    # a question with a single candidate keeps all but the last token in its stem (see layout builder), so give that
    # candidate its tokens and let the builder split them
    leaf = rng.integers(4, 13, 7)
    leaf = (leaf * (539 - 420 - sum(q_lens)) / leaf.sum()).round().astype(int)
    leaf[0] += 539 - 420 - sum(q_lens) - leaf.sum()
    return make_tree(seed, 420, q_lens, leaf.tolist(), groups, vocab)


def example_tree(seed=0, vocab=4096):
    """Shape of the reference's example request: 7 candidates, 539 prompt tokens in total, 277 packed rows -> key
    (288, 7, 96)."""
    # prompt tokens = sum of path lengths = 7*30 + (3*20 + 2*20 + 2*22) + 185 = 539; rows = 30 + 62 + 185 = 277
    q_lens = [20, 20, 22]
    groups = [0, 0, 0, 1, 1, 2, 2]
    leaf_lens = [20, 25, 30, 24, 28, 26, 32]
    return make_tree(seed, 30, q_lens, leaf_lens, groups, vocab)


def layout_cases():
    """name -> (seqs, groups, pad_id, NB, PB) for the layout parity tests and goldens."""
    cases = {}
    cases["doc"] = ([[10, 11, 12, 20, 21, 30], [10, 11, 12, 20, 21, 31, 32], [10, 11, 12, 25, 40, 41]], [0, 0, 1], 0, 32, 4)
    s, g = baseline_tree(0)
    cases["baseline"] = (s, g, 0, 32, 16)
    s, g = example_tree(0)
    cases["example"] = (s, g, 0, 32, 16)
    s, g = make_tree(3, 5, [0, 3], [2, 4, 1], [0, 0, 1])
    cases["nostem"] = (s, g, 1, 32, 16)
    s, g = make_tree(4, 70, [9], [1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1], [0] * 12)
    cases["wide"] = (s, g, 0, 32, 16)
    s, g = make_tree(5, 31, [1], [33], [0])
    cases["single"] = (s, g, 7, 32, 16)
    s, g = make_tree(6, 200, [12, 7, 30, 1], [3, 17, 5, 2, 40, 8, 8, 21], [0, 0, 1, 1, 1, 2, 3, 3])
    cases["ragged"] = (s, g, 0, 32, 16)
    # candidates with identical prefixes of different lengths (one candidate is a prefix of another)
    cases["prefix_of"] = ([[5, 6, 7, 8], [5, 6, 7, 8, 9, 10], [5, 6, 7]], [0, 0, 0], 0, 32, 16)
    s, g = make_tree(7, 1000, [20, 22], [6, 9, 4, 12], [0, 0, 1, 1])
    cases["long"] = (s, g, 0, 32, 16)
    return cases


def state_cases():
    """name -> (prefix ids, suffix ids [S, Ls], suffix mask, left pad) for the single-level layout (long-prefix path)."""
    rng = np.random.default_rng(11)
    cases = {}
    for name, (Lp, S, Ls, pad) in {"st_small": (32, 3, 16, 5), "st_nopad": (64, 2, 16, 0), "st_wide": (96, 6, 32, 17)}.items():
        pre = rng.integers(8, 4096, Lp)
        pre[:pad] = 0
        lens = rng.integers(1, Ls + 1, S)
        suf = rng.integers(8, 4096, (S, Ls))
        msk = (np.arange(Ls)[None, :] < lens[:, None]).astype(np.int64)
        suf = suf * msk
        cases[name] = (pre.tolist(), suf.tolist(), msk.tolist(), pad)
    return cases
