"""bi8_gemm_dequant_static: the GEMM entry point for callers that cannot allocate device memory at call time
(a serving loop that must stay away from cudaMalloc after start-up, a plugin without access to its host's
allocator, a fixed-footprint deployment).  Its split-K scratch is a fixed array inside the library.

Called here through the C ABI, twice in a row, on a small-M shape whose plan does use the scratch, and compared with
bi8_gemm_dequant given a caller workspace: the two run the same kernels with the same plan, so the results must be
bit-identical (the tolerance of the other GEMM tests is met trivially).  Collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from blockwise_int8_linear_b200 import _lib
    L = _lib.lib()
    c = ctypes
    vp, i64, i32 = c.c_void_p, c.c_int64, c.c_int
    L.bi8_gemm_dequant_static.argtypes = [vp, i64, vp, i64, vp, vp, vp, i32, vp, i64, i32, i64, i64, i64, i32, i32, vp]
    L.bi8_gemm_dequant_static.restype = i32
    L.bi8_gemm_static_scratch_bytes.restype = c.c_size_t
    return _lib, L


def _operands(m, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).cuda()
    bt = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).cuda()
    sa = (torch.rand((k // 64, m), generator=g) + 0.5).cuda()
    sb = (torch.rand((k // 64, n), generator=g) + 0.5).cuda()
    bias = torch.randn(n, generator=g).to(torch.bfloat16).cuda()
    return a, bt, sa, sb, bias


def _run(L, lib, fn, a, bt, sa, sb, bias, ws):
    m, k = a.shape
    n = bt.shape[0]
    c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    p, st = lib.ptr, lib.stream_ptr()
    if fn == "static":
        rc = L.bi8_gemm_dequant_static(p(a), k, p(bt), k, p(sa), p(sb), p(bias), 0, p(c), n, 0, m, n, k, 64, 0, st)
    else:
        rc = L.bi8_gemm_dequant(p(a), k, p(bt), k, p(sa), p(sb), p(bias), 0, p(c), n, 0, m, n, k, 64, p(ws),
                                0 if ws is None else ws.numel(), 0, st)
    lib.check(rc, fn)
    torch.cuda.synchronize()
    return c


def test_static_scratch_entry_point_matches_workspace_entry_point():
    lib, L = _lib()
    assert L.bi8_gemm_static_scratch_bytes() == 8 << 20
    for call, (m, k, n) in enumerate(((16, 2048, 1024), (96, 1024, 640))):      # two calls in a row, both split over K
        need = L.bi8_gemm_workspace_bytes(m, n, k, 64)
        assert 0 < need <= 8 << 20, "the shape must exercise the scratch"
        a, bt, sa, sb, bias = _operands(m, k, n, seed=100 + call)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        expect = _run(L, lib, "workspace", a, bt, sa, sb, bias, ws)
        got = _run(L, lib, "static", a, bt, sa, sb, bias, None)
        assert torch.equal(got, expect)
        # and against the CPU oracle, with the tolerance of the GEMM tests
        from oracle import blockwise_int8_oracle as O
        acc = O.gemm_acc(a.cpu(), bt.cpu().t(), sa.cpu(), sb.cpu(), 64)
        mag = O.gemm_term_abs_sum(a.cpu(), bt.cpu().t(), sa.cpu(), sb.cpu(), 64) + bias.float().cpu().abs()
        err = (got.float().cpu() - (acc + bias.float().cpu())).abs()
        assert (err <= 12 * 2.0 ** -24 * mag + (got.float().cpu().abs() + acc.abs()) * 2.0 ** -8).all()
    assert lib.device_status() == 0


def test_static_scratch_too_small_for_the_decode_kernel_takes_the_general_kernel():
    """33 <= M <= 64: the decode kernel's plan does not fit the built-in array, so the dispatcher declines it and the
    general kernel runs with the array as its split-K scratch: same result as bi8_gemm_dequant forced onto that kernel."""
    lib, L = _lib()
    m, k, n = 48, 4096, 4096
    a, bt, sa, sb, bias = _operands(m, k, n, seed=11)
    need = L.bi8_gemm_workspace_bytes(m, n, k, 64)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    p = lib.ptr
    rc = L.bi8_gemm_dequant(p(a), k, p(bt), k, p(sa), p(sb), p(bias), 0, p(c), n, 0, m, n, k, 64, p(ws), ws.numel(),
                            lib.GEMM_FORCE_TC, lib.stream_ptr())
    lib.check(rc, "bi8_gemm_dequant")
    got = _run(L, lib, "static", a, bt, sa, sb, bias, None)
    torch.cuda.synchronize()
    assert torch.equal(got, c)
    assert lib.device_status() == 0


def test_static_scratch_rejects_oversized_plans():
    lib, L = _lib()
    m, k, n = 128, 4096, 11008         # on a 148-SM device the plan wants 2 x 128 x 11008 floats: more than 8 MiB
    need = L.bi8_gemm_workspace_bytes(m, n, k, 64)
    if need <= 8 << 20:
        pytest.skip("this device's plan for the shape fits the built-in scratch")
    a, bt, sa, sb, bias = _operands(m, k, n, seed=7)
    c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    p = lib.ptr
    rc = L.bi8_gemm_dequant_static(p(a), k, p(bt), k, p(sa), p(sb), p(bias), 0, p(c), n, 0, m, n, k, 64, 0, lib.stream_ptr())
    assert rc == -9 and b"built-in array" in L.bi8_last_error_string()
