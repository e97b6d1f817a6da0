"""Test infrastructure: builds the reference's own CUDA operators for sm_100a so that GPU tests can compare against them.

    python oracle/build_ref_kernels.py [reference root]

(default: $OJ_REFERENCE, else the directory `reference` next to this repository)

Nothing of the reference is copied: its `src/kernels.cu` and the prototype string of its `src/ext.py` are read where they
lie and handed to torch's inline-extension builder, exactly as `src/ext.py:47-56` does, except for the target architecture
(`compute_100a` instead of `compute_103`). The only output is `oracle/_ref/ojref/ojref.so` (git-ignored). Tests load that file
when it exists and skip otherwise; the product never touches it.
"""
import importlib.util
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "ojref")


def default_ref_root():
    return os.environ.get("OJ_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def build(ref_root=None, verbose=False):
    ref_root = ref_root or default_ref_root()
    src_dir = os.path.join(ref_root, "src")
    cu = os.path.join(src_dir, "kernels.cu")
    if not os.path.exists(cu):
        return None
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
    for f in os.listdir(OUT):                         # keep the module only: the builder's scratch holds a copy of the sources
        if f != "ojref.so":
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


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), verbose=True))
