"""tcgen05 GEMM against torch.matmul on fp32-upcast operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def _mk(M, N, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).to(bf16)
    w = (torch.randn(N, K, generator=g, device="cuda", dtype=torch.float32) * 0.02).to(bf16)
    return x, w


def _ref(x, w):
    return x.float() @ w.float().t()


# tolerance: bf16 output rounding (2^-9 relative) + fp32 accumulation-order noise
def _close(out, ref):
    err = (out.float() - ref).abs().max().item()
    tol = ref.abs().max().item() * 2 ** -8 + 1e-3
    assert err <= tol, (err, tol)


# lt_matmul indices: 0 planner, 1 / 2 tile128, 3 block256, 4-6 block256 with forced width, 7 block256 all swapped,
# 8 / 9 CTA-pair kernel (automatic width / all swapped), 10 block256 with blocks + two exact swapped chunks
@pytest.mark.parametrize("variant", [0, 1, 3, 4, 5, 7, 8, 9, 10])
@pytest.mark.parametrize("M,N,K", [(64, 512, 256), (16, 48, 64), (257, 300, 136), (400, 1000, 512), (1000, 520, 192), (128, 256, 64), (288, 1280, 5120), (539, 12352, 5120), (100, 200, 72),
                                   (1024, 5120, 6144), (544, 5120, 4096)])
def test_gemm_plain(M, N, K, variant):
    from ojb200 import lt_ext, _lib
    if variant == 7 and M > 2048:
        pytest.skip("the all-swapped form serves M <= 2048")
    x, w = _mk(M, N, K, 1)
    out = lt_ext.lt_matmul(x, w, variant)
    torch.cuda.synchronize()
    _lib.check_status()
    _close(out, _ref(x, w))


@pytest.mark.parametrize("variant", [0, 1, 3, 7, 8, 9, 10])
@pytest.mark.parametrize("M,I,K", [(64, 128, 128), (288, 1024, 5120), (544, 17408, 5120), (256, 256, 320), (700, 384, 512), (539, 2048, 1024)])
def test_gemm_swiglu(M, I, K, variant):
    from ojb200 import lt_ext, _lib
    if variant == 7 and M > 2048:
        pytest.skip("the all-swapped form serves M <= 2048")
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(M, K, generator=g, device="cuda").to(bf16)
    wg = (torch.randn(I, K, generator=g, device="cuda") * 0.02).to(bf16)
    wu = (torch.randn(I, K, generator=g, device="cuda") * 0.02).to(bf16)
    # the CTA-pair kernel with block units reads gate / up interleaved in blocks of 64 rows, all others in blocks of 128
    out = lt_ext.gemm_swiglu(x, lt_ext.interleave_gate_up(wg, wu, 64 if variant == 8 else 128), variant)
    torch.cuda.synchronize()
    _lib.check_status()
    gg = _ref(x, wg).to(bf16).float()
    uu = _ref(x, wu).to(bf16).float()
    ref = torch.nn.functional.silu(gg).to(bf16).float() * uu
    err = (out.float() - ref).abs().max().item()
    # one bf16 ulp of gate or up can flip through the product: 2^-7 relative on the largest value
    tol = ref.abs().max().item() * 2 ** -6 + 1e-3
    assert err <= tol, (err, tol)


@pytest.mark.parametrize("variant", [0, 1, 3, 7, 8, 10])
@pytest.mark.parametrize("M,N,K,S", [(64, 256, 256, 2), (288, 5120, 6144, 2), (544, 5120, 17408, 4), (539, 5120, 4096, 2),
                                     (544, 5120, 17408, 7), (64, 5120, 4096, 16), (300, 520, 1000, 3)])
def test_gemm_splitk(M, N, K, S, variant):
    from ojb200 import lt_ext, _lib
    if variant == 7 and M > 2048:
        pytest.skip("the all-swapped form serves M <= 2048")
    x, w = _mk(M, N, K, 3)
    parts = lt_ext.gemm_splitk(x, w, S, variant)
    torch.cuda.synchronize()
    _lib.check_status()
    assert parts.shape == (S, M, N)
    kb = -(-K // 64)
    ks = -(-kb // S) * 64                  # ranges are whole 64-column k-blocks, the last one may be shorter
    for s in range(S):
        ref = x[:, s * ks:(s + 1) * ks].float() @ w[:, s * ks:(s + 1) * ks].float().t()
        err = (parts[s] - ref).abs().max().item()
        assert err <= ref.abs().max().item() * 1e-4 + 1e-4, (s, err)


def test_trace_hook_records_every_unit():
    """The measurement hook appends one timeline record per work unit and leaves the result untouched."""
    import ctypes
    from ojb200 import lt_ext, _lib
    x, w = _mk(544, 1024, 512, 4)
    ref = lt_ext.lt_matmul(x, w, 4)
    cap = 64
    rec = torch.zeros(1 + 4 * cap, dtype=torch.int64, device="cuda")
    _lib.call("ojb_gemm_set_trace", _lib.ptr(rec), _lib.i32(cap), _lib.i32(1), _lib.i32(0))
    try:
        out = lt_ext.lt_matmul(x, w, 4)
        torch.cuda.synchronize()
    finally:
        _lib.call("ojb_gemm_set_trace", None, _lib.i32(0), _lib.i32(1), _lib.i32(0))
    _lib.check_status()
    assert torch.equal(out, ref)
    r = rec.cpu()
    assert int(r[0]) == 2 * 4 + 4            # two 256-row blocks and one tail unit per 256-wide w tile
    t = r[1:1 + 4 * int(r[0])].view(-1, 4)
    assert bool((t[:, 1] <= t[:, 2]).all()) and bool((t[:, 2] <= t[:, 3]).all())


def _deq(q, s):
    return q.view(torch.float8_e4m3fn).float() * s[:, None]


@pytest.mark.parametrize("M,K", [(1, 64), (37, 520), (544, 5120)])
def test_quantize_rows_e4m3(M, K):
    """ojb_quantize_rows_e4m3 against torch's own e4m3 conversion of x / scale."""
    from ojb200 import lt_ext, _lib
    x = (torch.randn(M, K, device="cuda") * 3).to(bf16)
    if M > 1:
        x[1].zero_()
    q, s = lt_ext.quantize_rows_e4m3(x)
    amax = x.float().abs().amax(dim=1)
    ref_s = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    assert torch.allclose(s, ref_s, rtol=1e-6, atol=0)
    ref_q = (x.float() * (1.0 / s)[:, None]).to(torch.float8_e4m3fn).view(torch.uint8)
    assert (q != ref_q).float().mean().item() < 1e-3      # the reciprocal of the scale may tip a tie
    assert (_deq(q, s) - x.float()).abs().max().item() <= amax.max().item() * 2 ** -4 + 1e-6


@pytest.mark.parametrize("M,N,K", [(64, 512, 256), (256, 256, 128), (544, 1024, 640), (539, 12352, 5120), (288, 1280, 5120), (300, 520, 1008)])
def test_gemm_e4m3_plain(M, N, K):
    """8-bit GEMM against fp32 matmul of the same dequantised operands: only the accumulation order differs."""
    from ojb200 import lt_ext, _lib
    x = torch.randn(M, K, device="cuda").to(bf16)
    w = (torch.randn(N, K, device="cuda") * 0.02).to(bf16)
    xq, sx = lt_ext.quantize_rows_e4m3(x)
    wq, sw = lt_ext.quantize_weight_e4m3(w)
    ref = _deq(xq, sx) @ _deq(wq, sw).t()
    out = lt_ext.gemm_e4m3(xq, sx, wq, sw, 0)
    torch.cuda.synchronize()
    _lib.check_status()
    assert (out.float() - ref).abs().max().item() <= ref.abs().max().item() * 2 ** -8 + 1e-4
    # and the quantisation itself stays within a few per cent of the bf16 product
    full = x.float() @ w.float().t()
    assert ((out.float() - full).norm() / full.norm()).item() < 6e-2


@pytest.mark.parametrize("M,N,K,S", [(544, 5120, 17408, 2), (288, 5120, 4096, 3), (64, 512, 1024, 2), (539, 520, 1008, 1)])
def test_gemm_e4m3_splitk(M, N, K, S):
    from ojb200 import lt_ext, _lib
    x = torch.randn(M, K, device="cuda").to(bf16)
    w = (torch.randn(N, K, device="cuda") * 0.02).to(bf16)
    xq, sx = lt_ext.quantize_rows_e4m3(x)
    wq, sw = lt_ext.quantize_weight_e4m3(w)
    ref = _deq(xq, sx) @ _deq(wq, sw).t()
    parts = lt_ext.gemm_e4m3(xq, sx, wq, sw, 2, S)
    torch.cuda.synchronize()
    _lib.check_status()
    assert parts.shape == (S, M, N)
    assert (parts.sum(0) - ref).abs().max().item() <= ref.abs().max().item() * 1e-5 + 1e-5


@pytest.mark.parametrize("M,I,K", [(64, 128, 128), (288, 1024, 5120), (544, 17408, 5120), (539, 2048, 1024)])
def test_gemm_e4m3_swiglu(M, I, K):
    from ojb200 import lt_ext, _lib
    x = torch.randn(M, K, device="cuda").to(bf16)
    wg = (torch.randn(I, K, device="cuda") * 0.02).to(bf16)
    wu = (torch.randn(I, K, device="cuda") * 0.02).to(bf16)
    xq, sx = lt_ext.quantize_rows_e4m3(x)
    wq, sw = lt_ext.quantize_weight_e4m3(lt_ext.interleave_gate_up(wg, wu, 128))
    out = lt_ext.gemm_e4m3(xq, sx, wq, sw, 1)
    torch.cuda.synchronize()
    _lib.check_status()
    wd = _deq(wq, sw).view(-1, 2, 128, K)
    xd = _deq(xq, sx)
    g = (xd @ wd[:, 0].reshape(-1, K).t()).to(bf16).float()
    u = (xd @ wd[:, 1].reshape(-1, K).t()).to(bf16).float()
    ref = torch.nn.functional.silu(g).to(bf16).float() * u
    assert out.shape == (M, I)
    err = (out.float() - ref).abs().max().item()
    assert err <= ref.abs().max().item() * 2 ** -6 + 1e-3, err


# the four projection shapes of the model at the ends of the row-count sweep (64 and 4096 rows), library's own choice of kernel
@pytest.mark.parametrize("M", [64, 4096])
@pytest.mark.parametrize("K,N", [(5120, 12288), (5120, 34816), (17408, 5120), (6144, 5120)])
def test_gemm_projection_shapes_at_64_and_4096_rows(M, K, N):
    from ojb200 import lt_ext, _lib
    x, w = _mk(M, N, K, 7)
    out = lt_ext.lt_matmul(x, w, 0)
    torch.cuda.synchronize()
    _lib.check_status()
    _close(out, _ref(x, w))
    if N == 34816:                                  # the fused SwiGLU form of the gate/up shape
        I = N // 2
        wb = lt_ext.interleave_gate_up(w[:I].contiguous(), w[I:].contiguous())
        got = lt_ext.gemm_swiglu(x, wb, 0)
        torch.cuda.synchronize()
        _lib.check_status()
        r = _ref(x, w)
        ref = torch.nn.functional.silu(r[:, :I]) * r[:, I:]
        assert (got.float() - ref).abs().max().item() <= ref.abs().max().item() * 2 ** -7 + 1e-3
    if N == 5120:                                   # the split-K form of the two output projections
        S = lt_ext.plan_splitk(M, N, K)
        parts = lt_ext.gemm_splitk(x, w, S, 0)
        torch.cuda.synchronize()
        _lib.check_status()
        r = _ref(x, w)
        assert (parts.sum(0) - r).abs().max().item() <= r.abs().max().item() * 2 ** -12 + 1e-4


def test_bounded_wait_runs_out_and_reports_through_the_status_word():
    """Every device-side wait of the GEMM kernels has a limit. With the limit set to 50 ms and the host-side failure switch
    on, the producer of a one-CTA GEMM leaves out the copies of its second k-block: the consumer's wait runs out, the kernel
    writes OJB_DEV_WAIT_TIMEOUT, frees its tensor memory and returns; the host sees the status, and the next launch on the
    same context is correct. Nothing faults or spins without a limit."""
    import ctypes
    from ojb200 import lt_ext, _lib
    lib = _lib.lib()
    x, w = _mk(128, 256, 128, 11)                   # one 128 x 256 tile, two k-blocks
    good = lt_ext.lt_matmul(x, w, 1)
    torch.cuda.synchronize()
    _lib.check_status()
    try:
        assert lib.ojb_gemm_set_wait_limit_ms(ctypes.c_int32(50)) == 0
        assert lib.ojb_gemm_test_drop_copy(ctypes.c_int32(1)) == 0
        t0 = __import__("time").perf_counter()
        lt_ext.lt_matmul(x, w, 1)
        torch.cuda.synchronize()
        dt = __import__("time").perf_counter() - t0
    finally:
        lib.ojb_gemm_test_drop_copy(ctypes.c_int32(0))
        lib.ojb_gemm_set_wait_limit_ms(ctypes.c_int32(0))
    assert dt < 1.5, dt                             # gave up after the 50 ms limit, not after the default 2 s
    with pytest.raises(RuntimeError, match="wait ran out"):
        _lib.check_status()
    again = lt_ext.lt_matmul(x, w, 1)               # the context is intact
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(again, good)


@pytest.mark.parametrize("M", [16384 + 32, 13 * 256 * 2])
def test_x_larger_than_l2_runs_in_bands(M):
    """With more rows of x than the L2 keeps (tens of thousands), the block kernel deals its units band by band (x blocks of
    one band stay in L2, the weight is streamed once per band). Every output row must still be produced exactly once: plain,
    SwiGLU and split-K forms, with and without a 32-row remainder after the last block, against fp32 matmul."""
    from ojb200 import lt_ext, _lib
    K, N = 5120, 1280
    x, w = _mk(M, N, K, 21)
    ref = _ref(x, w)
    _close(lt_ext.lt_matmul(x, w, 3), ref)
    parts = lt_ext.gemm_splitk(x, w, 2, 3)
    assert (parts.sum(0) - ref).abs().max().item() <= ref.abs().max().item() * 2 ** -8 + 1e-3
    I = N // 2
    out = lt_ext.gemm_swiglu(x, lt_ext.interleave_gate_up(w[:I].contiguous(), w[I:].contiguous(), 128), 3)
    torch.cuda.synchronize()
    _lib.check_status()
    gg, uu = ref[:, :I], ref[:, I:]
    want = torch.nn.functional.silu(gg) * uu
    assert (out.float() - want).abs().max().item() <= want.abs().max().item() * 2 ** -7 + 2e-3
