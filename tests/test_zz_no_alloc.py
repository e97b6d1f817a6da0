"""The scratch-free Gated DeltaNet entry point (ojb_gdn_chunked_static) gives the same output as ojb_gdn_chunked.

Some users of this library cannot allocate device memory around a call — a serving process that freezes its memory plan
after start-up, or a host program without a device allocator. For them the library carries a fixed scratch array; this test
calls that entry point directly through the C ABI, twice in a row with different inputs (the array is shared and keeps the
previous call's contents), and compares with the allocating entry point. Collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def _inputs(T, HK, HV, seed):
    g_ = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(T, HK, 128, generator=g_), dim=-1).to(bf16).cuda()
    k = torch.nn.functional.normalize(torch.randn(T, HK, 128, generator=g_), dim=-1).to(bf16).cuda()
    v = torch.randn(T, HV, 128, generator=g_).to(bf16).cuda()
    g = torch.nn.functional.logsigmoid(torch.randn(T, HV, generator=g_)).cuda()
    beta = torch.sigmoid(torch.randn(T, HV, generator=g_)).to(bf16).cuda()
    return q, k, v, g, beta


def test_static_scratch_entry_point_matches_allocating_one():
    from ojb200 import _lib, ext as K
    from ojb200._lib import call, f32, i64, ptr, stream_ptr
    lib = _lib.lib()
    lib.ojb_gdn_static_max_items.restype = ctypes.c_int64
    assert lib.ojb_gdn_static_max_items() == 1024
    HK, HV, scale = 2, 4, 128 ** -0.5
    # two calls in a row with different shapes and data, then one that fills the array exactly (256 chunks x 4 heads = 1024)
    for call_no, (B, T) in enumerate([(3, 150), (2, 96), (1, 256 * 64)]):
        chunks, steps, walks = K._seq_tables(B, T, torch.device("cuda"))
        q, k, v, g, beta = _inputs(B * T, HK, HV, 40 + call_no)
        want = K.gdn_chunked(q, k, v, g, beta, scale, chunks, steps, walks, B)
        got = torch.empty_like(want)                                 # outputs are the caller's; the call allocates nothing
        call("ojb_gdn_chunked_static", ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(chunks), i64(chunks.shape[0]),
             ptr(steps), ptr(walks), i64(B), ptr(None), ptr(None), ptr(got), i64(HK), i64(HV), f32(scale),
             ptr(_lib.status_word(got.device)), stream_ptr())
        torch.cuda.synchronize()
        _lib.check_status()
        rel = ((got.float() - want.float()).norm() / want.float().norm()).item()
        assert rel < 4e-3, (call_no, rel)           # the tolerance of the other Gated DeltaNet tests; in practice 0
        assert torch.equal(got, want)               # same kernels, same inputs


def test_static_scratch_rejects_oversize():
    from ojb200 import _lib
    from ojb200._lib import f32, i64, ptr, stream_ptr
    lib = _lib.lib()
    lib.ojb_gdn_chunked_static.restype = ctypes.c_int
    t = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = lib.ojb_gdn_chunked_static(ptr(t), ptr(t), ptr(t), ptr(t), ptr(t), ptr(t), i64(300), ptr(t), ptr(t), i64(1), ptr(None),
                                    ptr(None), ptr(t), i64(2), i64(4), f32(1.0), ptr(None), stream_ptr())
    assert rc == -4                                 # 300 * 4 items > 1024: refused, nothing launched
