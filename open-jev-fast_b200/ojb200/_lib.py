"""ctypes binding of libojb200.so — the only place that touches the C ABI declared in include/ojb200.h.

There is no fallback: if the library is missing or a call fails, a RuntimeError names the entry point.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libojb200.so")
ABI_VERSION = 6

_ERR = {-1: "invalid argument (shape / alignment / null pointer)", -2: "CUDA launch or API failure",
        -3: "CUDA driver tensor-map encoder unavailable", -4: "size beyond the documented maximum"}

_lib = None
_status = {}


def lib():
    """The loaded library (loads on first use)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m ojb200.build` (nvcc, sm_100a). "
                               "There is no CPU or PyTorch fallback for these ops.")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.ojb_abi_version.restype = ctypes.c_int
        if _lib.ojb_abi_version() != ABI_VERSION:
            raise RuntimeError("libojb200.so was built from a different ABI version; rebuild it")
    return _lib


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    """Device (or host) address of a tensor, or NULL for None."""
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def i64(v):
    return ctypes.c_int64(int(v))


def i32(v):
    return ctypes.c_int(int(v))


def f32(v):
    return ctypes.c_float(float(v))


def status_word(device):
    """Per-device int32 word that kernels with bounded waits write on a timeout."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = _status[key] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    return t


def check_status(device=None):
    """Read the status word back (synchronises). Raises if a device-side wait ran out."""
    key = torch.cuda.current_device() if device is None else torch.device(device).index
    t = _status.get(key)
    if t is not None:
        v = int(t.item())
        if v != 0:
            t.zero_()
            raise RuntimeError(f"ojb200: device-side wait ran out (status {v}); results of the last calls are invalid")


_KERNELS_PER_CALL = {"ojb_gdn_chunked": 2, "ojb_gdn_chunked_proj": 2, "ojb_gdn_chunked_static": 2, "ojb_gdn_chunked_levels": 4, "ojb_gemm_plan": 0,
                     "ojb_gemm_set_trace": 0}
_launches = 0


def launch_count():
    """Number of kernels this process has launched through the C ABI so far."""
    return _launches


def call(name, *args):
    global _launches
    fn = getattr(lib(), name)
    fn.restype = ctypes.c_int
    rc = fn(*args)
    if rc != 0:
        raise RuntimeError(f"{name} failed: {_ERR.get(rc, rc)}")
    _launches += _KERNELS_PER_CALL.get(name, 1)


def need_cuda_bf16(*tensors):
    for t in tensors:
        if t is None:
            continue
        if not (t.is_cuda and t.is_contiguous()):
            raise RuntimeError("ojb200: tensors must be contiguous CUDA tensors")
