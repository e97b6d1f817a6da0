"""The C-ABI library loads without a GPU and exports every entry point that include/ojb200.h declares; host-only entry
points (layout builder) are exercised in test_layout.py. No compute call is made here."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "ojb200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(ojb_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_the_hot_path():
    names = _declared()
    for must in ("ojb_gemm_bf16", "ojb_gemm_bf16_swiglu", "ojb_gemm_bf16_splitk", "ojb_add_rmsnorm", "ojb_add_rmsnorm_sk",
                 "ojb_gdn_prep", "ojb_gdn_chunked", "ojb_gated_rmsnorm", "ojb_fullattn_prep", "ojb_tree_attn", "ojb_score_head",
                 "ojb_gtree_dims", "ojb_gtree_fill"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from ojb200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in _declared() if not hasattr(lib, n)]
    assert not missing, missing
    lib.ojb_abi_version.restype = ctypes.c_int
    assert lib.ojb_abi_version() == _lib.ABI_VERSION


def test_argument_checks_need_no_gpu():
    """Precondition failures are reported before anything touches CUDA."""
    from ojb200 import _lib
    lib = _lib.lib()
    lib.ojb_gemm_bf16.restype = ctypes.c_int
    rc = lib.ojb_gemm_bf16(None, None, None, ctypes.c_int64(1), ctypes.c_int64(1), ctypes.c_int64(8), 0, None, None)
    assert rc == -1
    lib.ojb_tree_attn.restype = ctypes.c_int
    one = ctypes.c_void_p(16)
    rc = lib.ojb_tree_attn(one, one, one, one, one, None, one, ctypes.c_int64(33), ctypes.c_int64(4), ctypes.c_int64(2),
                           ctypes.c_int64(256), ctypes.c_int64(2), ctypes.c_float(1.0), None)
    assert rc == -1      # N must be a multiple of 32


def test_gemm_plan_is_host_arithmetic():
    """ojb_gemm_plan needs no GPU: it returns a valid variant, a split count within bounds, and a finite time."""
    from ojb200 import lt_ext
    for M, N, K, kind in [(544, 12352, 5120, 0), (544, 34816, 5120, 1), (544, 5120, 17408, 2), (64, 5120, 4096, 2), (16384, 5120, 17408, 2),
                          (1, 16, 8, 0)]:
        v, s, us = lt_ext.gemm_plan(M, N, K, kind)
        assert v in (1, 2, 3, 4) and 1 <= s <= 16 and 0 < us < 1e6
        if kind != 2:
            assert s == 1
        kb = -(-K // 64)
        assert (s - 1) * -(-kb // s) < kb          # no empty K range
    # more rows never make the modelled time shorter
    t = [lt_ext.gemm_plan(M, 34816, 5120, 1)[2] for M in (256, 512, 1024, 2048, 4096)]
    assert all(a <= b for a, b in zip(t, t[1:]))


def test_operator_surface_has_every_name_of_the_reference():
    """The 40 operator names of open-jev-fast's src/ext.py:52 and the 8 of src/lt_ext.py:7 exist in the Python layer (legacy
    variants alias the production kernels under their own layout contract)."""
    from ojb200 import ext, lt_ext
    ops = ["add_rmsnorm", "silu_mul", "linattn_prep", "gated_rmsnorm", "fullattn_prep", "gate_mul", "linattn_prep2", "fullattn_prep2",
           "gate_mul2", "linattn_prep_tree", "add_rmsnorm_sk", "linattn_prep_rep", "gated_rmsnorm_map", "linattn_prep_map",
           "gated_rmsnorm_inv", "linattn_prep_map2", "linattn_prep_dedup", "linattn_prep_dedup2", "act_tables", "silu_mul_lut",
           "gated_rmsnorm_inv2", "l2_prefetch", "linattn_prep_dedup3", "gate_mul3", "add_rmsnorm_sk2", "gdn_fused", "gdn_fused2",
           "gdn_fused3", "gdn_fused4", "gdn_fused5", "gdn_fused6", "gdn_fused7", "gdn_fused6ts", "fattn_tree", "fattn_tree2",
           "fattn_tree2_ts", "fattn_tree3", "pack_bits", "gdn_fused8", "gdn_fused9"]
    assert len(ops) == 40
    assert not [n for n in ops if not callable(getattr(ext, n, None))]
    lt = ["lt_setup", "lt_matmul", "lt2_plan", "lt2_search", "lt2_info", "lt2_run", "lt2_raw", "lt2_add_raw"]
    assert not [n for n in lt if not callable(getattr(lt_ext, n, None))]
