"""Generates tests/golden/layout_golden.npz from the reference's own `gtree_build` and `tree_layout`.

Run in a container that mounts open-jev-fast ($OJ_REFERENCE, else the directory `reference` next to this repository):
    python tests/golden/make_layout_golden.py
The two functions are lifted out of src/fastmodel.py by AST (the module itself cannot be imported without a GPU because it
builds its CUDA extension at import) and executed unmodified with dev="cpu". The inputs are the seeded synthetic trees of
open-jev-fast_b200/ojb200/trees.py; only integers are stored.
"""
import ast
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(HERE)), "open-jev-fast_b200"))
from ojb200 import trees  # noqa: E402

REF = os.environ.get("OJ_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))


def reference_functions():
    src = open(os.path.join(REF, "src", "fastmodel.py")).read()
    mod = ast.parse(src)
    cls = next(n for n in mod.body if isinstance(n, ast.ClassDef) and n.name == "FastQwen35")
    out = {}
    for fn in cls.body:
        if isinstance(fn, ast.FunctionDef) and fn.name in ("gtree_build", "tree_layout"):
            fn.decorator_list = []
            m = ast.Module(body=[fn], type_ignores=[])
            ns = {"torch": torch, "SimpleNamespace": types.SimpleNamespace}
            exec(compile(ast.fix_missing_locations(m), "fastmodel.py", "exec"), ns)
            out[fn.name] = ns[fn.name]
    return out


def main():
    fns = reference_functions()
    blob = {}
    for name, (seqs, groups, pad_id, NB, PB) in trees.layout_cases().items():
        ids, lay = fns["gtree_build"](seqs, groups, pad_id, NB=NB, PB=PB, dev="cpu")
        blob[f"{name}/ids"] = ids.numpy()
        for f in ("pos", "rowmask", "vbits", "src", "inv", "lastidx", "rep_ptr", "rep_pos", "hist", "canon"):
            blob[f"{name}/{f}"] = getattr(lay, f).numpy()
        blob[f"{name}/amask"] = np.packbits(lay.amask[0, 0].numpy(), axis=1, bitorder="little")
        blob[f"{name}/meta"] = np.array([lay.N, lay.S, lay.R, lay.L2, lay.Lr, lay.Nreal], np.int64)
    for name, (pre, suf, msk, pad) in trees.state_cases().items():
        lay = fns["tree_layout"](None, torch.tensor(pre), torch.tensor(suf), torch.tensor(msk), pad=pad)
        for f in ("pos", "rowmask", "lastidx", "repidx"):
            blob[f"{name}/{f}"] = getattr(lay, f).numpy()
        blob[f"{name}/amask"] = np.packbits(lay.amask[0, 0].numpy(), axis=1, bitorder="little")
        blob[f"{name}/meta"] = np.array([lay.Lp, lay.S, lay.Ls, lay.N], np.int64)
    np.savez_compressed(os.path.join(HERE, "layout_golden.npz"), **blob)
    print("wrote", len(blob), "arrays")


if __name__ == "__main__":
    main()
