"""Test infrastructure: builds the reference's own CUDA operators for sm_100a so that GPU tests can compare against them.

    python oracle/build_ref_kernels.py [reference root]

(default: $OJ_REFERENCE, else the directory `reference` next to this repository)

Nothing of the reference is copied: its `src/kernels.cu` and the prototype string of its `src/ext.py` are read where they
lie and handed to torch's inline-extension builder, exactly as `src/ext.py:47-56` does, except for the target architecture
(`compute_100a` instead of `compute_103`). Its Python forward (`src/fastmodel.py`, unmodified) is byte-compiled where it lies.
The only outputs are `oracle/_ref/ojref/ojref.so` and `oracle/_ref/ojref/fastmodel_bytecode.bin` (git-ignored, built artefacts). Tests
and the benchmark's reference legs load them when they exist and skip otherwise; the product never touches them.
"""
import importlib.util
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "ojref")


def default_ref_root():
    return os.environ.get("OJ_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def build_forward(ref_root=None):
    """Byte-compiles the reference's src/fastmodel.py (FastQwen35 with gtree_build / forward_gtree) into
    oracle/_ref/ojref/fastmodel_bytecode.bin. Returns the path, or None when the reference tree is not around."""
    import py_compile
    ref_root = ref_root or default_ref_root()
    src = os.path.join(ref_root, "src", "fastmodel.py")
    if not os.path.exists(src):
        return None
    out = os.path.join(OUT, "fastmodel_bytecode.bin")
    if os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    os.makedirs(OUT, exist_ok=True)
    py_compile.compile(src, cfile=out, dfile="open-jev-fast/src/fastmodel.py", doraise=True)
    return out


def build(ref_root=None, verbose=False):
    ref_root = ref_root or default_ref_root()
    src_dir = os.path.join(ref_root, "src")
    cu = os.path.join(src_dir, "kernels.cu")
    if not os.path.exists(cu):
        return None
    build_forward(ref_root)
    so = os.path.join(OUT, "ojref.so")
    if os.path.exists(so) and os.path.getmtime(so) >= max(os.path.getmtime(cu), os.path.getmtime(os.path.join(src_dir, "ext.py"))):
        return so
    spec = importlib.util.spec_from_file_location("_oj_ref_ext", os.path.join(src_dir, "ext.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)                      # defines the prototype string and a loader; builds nothing
    protos = mod._CPP
    names = re.findall(r"^\s*(?:std::vector<torch::Tensor>|torch::Tensor|void)\s+(\w+)\s*\(", protos, flags=re.M)
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    from torch.utils.cpp_extension import load_inline
    load_inline(name="ojref", cpp_sources=[protos], cuda_sources=[open(cu).read()], functions=names,
                extra_cuda_cflags=["-O3", "-gencode=arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr", "-lineinfo"],
                build_directory=OUT, verbose=verbose, is_python_module=True)
    for f in os.listdir(OUT):                         # keep the built files only: the builder's scratch holds a copy of the sources
        if f not in ("ojref.so", "fastmodel_bytecode.bin"):
            os.remove(os.path.join(OUT, f))
    return so if os.path.exists(so) else None


def load():
    """The built module, or None when it has not been built (or no GPU build of torch is around)."""
    so = os.path.join(OUT, "ojref.so")
    if not os.path.exists(so):
        return None
    import torch  # noqa: F401  (the extension links against it)
    spec = importlib.util.spec_from_file_location("ojref", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_fastmodel():
    """The reference's `fastmodel` module (FastQwen35, gdn_split, ...) from the byte-compiled file, bound to the rebuilt
    operators: the module does `from ext import load; K = load()` at import (src/fastmodel.py:42-43), which is answered here
    with the sm_100a build; its cuBLASLt search (`lt_ext`) is not built, so it uses F.linear / torch.bmm, its own fallback
    (src/fastmodel.py:65-69). Returns None when either built file is missing."""
    import importlib.machinery
    import sys
    import types
    pyc = os.path.join(OUT, "fastmodel_bytecode.bin")
    K = load()
    if K is None or not os.path.exists(pyc):
        return None
    if "oj_ref_fastmodel" in sys.modules:
        return sys.modules["oj_ref_fastmodel"]
    try:                                              # the module imports FLA's Triton entry points although its default path
        import fla.ops.gated_delta_rule  # noqa: F401   (GDN_FUSED) never calls them; stand-ins keep the import alive without FLA
        from fla.ops.gated_delta_rule.chunk_fwd import chunk_gated_delta_rule_fwd_kkt_solve_kernel  # noqa: F401
        from fla.ops.gated_delta_rule.wy_fast import recompute_w_u_fwd  # noqa: F401
        from fla.ops.common.chunk_delta_h import chunk_gated_delta_rule_fwd_h  # noqa: F401
        from fla.ops.common.chunk_o import chunk_fwd_o  # noqa: F401
        from fla.ops.utils import chunk_local_cumsum  # noqa: F401
        from fla.ops.utils.constant import RCP_LN2  # noqa: F401
    except Exception:
        def _absent(*a, **k):
            raise RuntimeError("flash-linear-attention is not installed: only the reference's fused GDN path is available")
        names = {"fla": [], "fla.ops": [], "fla.ops.gated_delta_rule": ["chunk_gated_delta_rule"],
                 "fla.ops.utils": ["chunk_local_cumsum"], "fla.ops.utils.constant": [],
                 "fla.ops.gated_delta_rule.chunk_fwd": ["chunk_gated_delta_rule_fwd_intra", "chunk_gated_delta_rule_fwd_kkt_solve_kernel"],
                 "fla.ops.common": [], "fla.ops.common.chunk_delta_h": ["chunk_gated_delta_rule_fwd_h"],
                 "fla.ops.common.chunk_o": ["chunk_fwd_o"], "fla.ops.gated_delta_rule.wy_fast": ["recompute_w_u_fwd"]}
        for mname, attrs in names.items():
            m = types.ModuleType(mname)
            m.__path__ = []
            for a in attrs:
                setattr(m, a, _absent)
            sys.modules[mname] = m
        sys.modules["fla.ops.utils.constant"].RCP_LN2 = 1.4426950408889634
    shim = types.ModuleType("ext")
    shim.load = lambda verbose=False: K
    saved = {n: sys.modules.get(n) for n in ("ext", "lt_ext")}
    sys.modules["ext"] = shim
    sys.modules.pop("lt_ext", None)
    try:
        loader = importlib.machinery.SourcelessFileLoader("oj_ref_fastmodel", pyc)
        spec = importlib.util.spec_from_loader("oj_ref_fastmodel", loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
    finally:
        for n, m in saved.items():
            if m is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = m
    sys.modules["oj_ref_fastmodel"] = mod
    return mod


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), verbose=True))
