"""Int8 block GEMM with fused dequantize on the GPU against the CPU oracle.

Stated tolerances:
* int32 block partial sums: exact.
* CUDA-core (generic) kernel, fp32 output: bit-exact against the oracle (same operation order as the reference).
* tensor-core kernel, fp32 output: |c - oracle| <= 12 * 2^-24 * sum_j |term_j| per element.  The kernel multiplies the three
  factors of a term in another order than the reference and, in seeded mode, rounds sA/127^2 to 22 bits: up to 4 roundings of
  2^-24 per term against the reference's 3, so the two sides differ by at most 7 * 2^-24 |term_j| per term, plus the
  difference of the two fp32 running sums (each rounding of a partial sum is bounded by 2^-24 * sum_j |term_j|; they mostly
  cancel between the two sides).  Observed worst case over the test shapes: 6.7 * 2^-24 * sum_j |term_j|.
* tensor-core kernel, bf16 output: the bf16 value is the RNE cast of that fp32 accumulator, so
  |c - oracle_fp32| <= 12 * 2^-24 * sum_j |term_j| + half a bf16 step of |c|; and >= 99 % of the elements are bit-identical
  to the oracle's bf16 result.  (Where the terms cancel, "within one bf16 step of the oracle's bf16 value" is not a meaningful
  bound: a tiny result has tiny steps, while its error is set by the magnitude of the terms.)
"""
import pytest
import torch

from oracle import blockwise_int8_oracle as O
from tests.gpu_util import DEV, assert_clean_device, bf16_ulp_distance, quantized_pair, randn_bf16, set_config
from tests.helpers import golden_names, load_golden

pytestmark = pytest.mark.gpu

GENERIC, TC, NO_SEED = 1, 2, 4
FP32_TOL = 12 * 2.0 ** -24


def _gemm(xq, wq, xs, ws, bias=None, flags=0):
    from triton_functions import int8_matmul_block64_rowwise_dequantize as mm
    return mm(xq.to(DEV), wq.to(DEV).t(), xs.to(DEV), ws.to(DEV), None if bias is None else bias.to(DEV), flags=flags)


def _check_fp32(c, xq, wq, xs, ws, block, bias=None):
    acc = O.gemm_acc(xq, wq.t(), xs, ws, block)
    mag = O.gemm_term_abs_sum(xq, wq.t(), xs, ws, block)
    if bias is not None:
        acc = acc + bias.float()
        mag = mag + bias.float().abs()
    err = (c.cpu() - acc).abs()
    bad = err > (FP32_TOL * mag + 1e-30)
    assert not bad.any(), f"{bad.sum().item()} elements beyond tolerance, worst ratio {(err / (mag + 1e-30)).max().item() / 2.0 ** -24:.2f} x 2^-24"


def _check_bf16(c, xq, wq, xs, ws, block, bias=None, identical=0.99):
    acc = O.gemm_acc(xq, wq.t(), xs, ws, block)
    mag = O.gemm_term_abs_sum(xq, wq.t(), xs, ws, block)
    ref = acc.to(torch.bfloat16)
    if bias is not None:
        ref = ref + bias.to(torch.bfloat16)
        mag = mag + bias.float().abs()
    cf = c.float().cpu()
    # half a bf16 step of the stored value, plus half a step of the intermediate cast when a bias is added after it
    half_step = cf.abs() * 2.0 ** -8
    if bias is not None:
        half_step = half_step + acc.abs() * 2.0 ** -8
    err = (cf - (acc if bias is None else acc + bias.float())).abs()
    bad = err > (FP32_TOL * mag + half_step + 1e-30)
    assert not bad.any(), f"{bad.sum().item()} elements beyond tolerance"
    same = (bf16_ulp_distance(c.cpu(), ref) == 0).float().mean().item()
    assert same >= identical, f"only {same:.4f} identical"


SHAPES = [
    # (M, K, N, block)
    (128, 128, 256, 64),      # one tile, one stage
    (128, 512, 256, 64),      # one tile, ring wraps
    (256, 1024, 512, 64),     # several tiles
    (300, 640, 600, 64),      # M, N tails, persistent loop
    (1, 4096, 512, 64),       # single row
    (16, 1024, 1024, 64),
    (130, 192, 264, 64),      # K = 1.5 stages: second stage half out of range
    (64, 4096, 300, 64),
    (200, 256, 136, 32),
    (200, 416, 136, 32),      # K tail inside a stage, block 32
    (72, 1024, 520, 128),
    (72, 400, 520, 128),      # last block partial (K % 128 = 16)
    (129, 272, 75, 64),       # odd N: scalar scale loads and stores
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("flags", [TC, GENERIC])
def test_block_partials_exact(shape, flags):
    from triton_functions import int8_matmul_block_partials
    m, k, n, block = shape
    xq, xs, wq, ws = quantized_pair(m, k, n, block, seed=m + k + n)
    p = int8_matmul_block_partials(xq.to(DEV), wq.to(DEV).t(), block, flags=flags)
    ref = O.gemm_block_partials(xq, wq.t(), block)
    assert torch.equal(p.cpu(), ref)
    if flags == TC:
        p2 = int8_matmul_block_partials(xq.to(DEV), wq.to(DEV).t(), block, flags=TC | NO_SEED)
        assert torch.equal(p2.cpu(), ref)
    assert_clean_device()


def test_partials_extreme_values():
    """All operands at +-127: |P| reaches 127*127*block, the largest value a block can produce."""
    from triton_functions import int8_matmul_block_partials
    for block in (32, 64, 128):
        m, k, n = 128, 2 * block, 256
        a = torch.full((m, k), 127, dtype=torch.int8)
        b = torch.full((n, k), -127, dtype=torch.int8)
        b[::2] = 127
        p = int8_matmul_block_partials(a.to(DEV), b.to(DEV).t(), block, flags=TC)
        assert torch.equal(p.cpu(), O.gemm_block_partials(a, b.t(), block))


@pytest.mark.parametrize("shape", SHAPES)
def test_generic_kernel_bit_exact_fp32(shape):
    m, k, n, block = shape
    set_config(block, torch.float32)
    xq, xs, wq, ws = quantized_pair(m, k, n, block, seed=3 * m + k + n)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(n))
    c = _gemm(xq, wq, xs, ws, bias, flags=GENERIC)
    ref = O.gemm(xq, wq.t(), xs, ws, bias, block, torch.float32)
    assert torch.equal(c.cpu(), ref)
    set_config(64)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("mode", [TC, TC | NO_SEED])
def test_tensor_core_kernel_fp32(shape, mode):
    m, k, n, block = shape
    set_config(block, torch.float32)
    xq, xs, wq, ws = quantized_pair(m, k, n, block, seed=5 * m + k + n)
    c = _gemm(xq, wq, xs, ws, flags=mode)
    assert c.dtype == torch.float32 and tuple(c.shape) == (m, n)
    _check_fp32(c, xq, wq, xs, ws, block)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(n)).to(torch.bfloat16)
    _check_fp32(_gemm(xq, wq, xs, ws, bias, flags=mode), xq, wq, xs, ws, block, bias)
    assert_clean_device()
    set_config(64)


@pytest.mark.parametrize("shape", SHAPES)
def test_tensor_core_kernel_bf16(shape):
    m, k, n, block = shape
    set_config(block, torch.bfloat16)
    xq, xs, wq, ws = quantized_pair(m, k, n, block, seed=7 * m + k + n)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(n)).to(torch.bfloat16)
    for b in (None, bias):
        c = _gemm(xq, wq, xs, ws, b, flags=TC)
        assert c.dtype == torch.bfloat16
        _check_bf16(c, xq, wq, xs, ws, block, b)
    set_config(64)


def test_default_dispatch_matches_forced_paths():
    set_config(64, torch.float32)
    xq, xs, wq, ws = quantized_pair(160, 512, 384, 64, seed=99)
    assert torch.equal(_gemm(xq, wq, xs, ws), _gemm(xq, wq, xs, ws, flags=TC))
    # K = 150: rows are not 16-byte aligned, the default path is the CUDA-core kernel
    xq, xs, wq, ws = quantized_pair(20, 150, 24, 64, seed=98)
    assert torch.equal(_gemm(xq, wq, xs, ws), _gemm(xq, wq, xs, ws, flags=GENERIC))
    from blockwise_int8_linear_b200._lib import Bi8Error
    with pytest.raises(Bi8Error):
        _gemm(xq, wq, xs, ws, flags=TC)
    set_config(64)


@pytest.mark.parametrize("name", golden_names("ops_"))
def test_golden_gemm(name):
    g = load_golden(name)
    set_config(g["block"], torch.float32)
    bias = g.get("bias")
    c = _gemm(g["xq"], g["wq"], g["xs"], g["ws"], bias, flags=GENERIC)
    assert torch.equal(c.cpu(), g["c_f32"])
    c = _gemm(g["xq"], g["wq"], g["xs"], g["ws"], bias)
    _check_fp32(c, g["xq"], g["wq"], g["xs"], g["ws"], g["block"], bias)
    set_config(64)


def test_operand_layouts():
    """b given as a contiguous [K, N] tensor and a given as a transposed view: handled like the reference (149-152)."""
    from triton_functions import int8_matmul_block64_rowwise_dequantize as mm
    set_config(64, torch.float32)
    xq, xs, wq, ws = quantized_pair(96, 256, 160, 64, seed=21)
    ref = _gemm(xq, wq, xs, ws)
    b_kn = wq.t().contiguous().to(DEV)                    # [K, N] row-major
    assert torch.equal(mm(xq.to(DEV), b_kn, xs.to(DEV), ws.to(DEV)), ref)
    a_t = xq.t().contiguous().to(DEV).t()                 # [M, K] view with strides (1, M)
    assert torch.equal(mm(a_t, wq.to(DEV).t(), xs.to(DEV), ws.to(DEV)), ref)
    with pytest.raises(AssertionError, match="incompatible dimensions"):
        mm(xq.to(DEV), wq.to(DEV)[:, :128].t(), xs.to(DEV), ws.to(DEV))
    with pytest.raises(ValueError):
        mm(xq.to(DEV), wq.to(DEV).t(), xs.to(DEV)[:2], ws.to(DEV))
    set_config(64)


@pytest.mark.parametrize("kn", [(4096, 4096), (4096, 11008), (11008, 4096)])
@pytest.mark.parametrize("m", [1, 16, 128, 2048])
def test_llama_projection_shapes(kn, m):
    """BASELINE config: activations N(0,1) quantized on the fly, weights N(0, 0.02) pre-quantized, block 64, bf16 out."""
    from triton_functions import quantize_block_rowwise
    k, n = kn
    set_config(64, torch.bfloat16)
    x = O.synthetic((m, k), 3000 + m, outlier_frac=0.0)
    w = O.synthetic((n, k), 3100 + n % 97, std=0.02, outlier_frac=0.0)
    wq, ws = O.quantize(w, 64)
    xq_g, xs_g = quantize_block_rowwise(x.to(DEV))
    xq, xs = O.quantize(x, 64)
    assert torch.equal(xq_g.cpu(), xq) and torch.equal(xs_g.cpu(), xs)
    c = _gemm(xq, wq, xs, ws)
    rows = slice(0, min(m, 256))
    _check_bf16(c[rows], xq[rows], wq, xs[:, rows], ws, 64)
    assert_clean_device()


@pytest.mark.parametrize("kn", [(4096, 11008), (4096, 4096), (11008, 4096)])
def test_largest_projection_shape_properties(kn):
    """M = 8192 on each of the three projection shapes: the oracle is evaluated on a sample of rows; the rest is covered
    by a size-independent property (row blocks of the same input give the same output rows).  (11008, 4096) has 172
    blocks per row, the longest fp32 accumulation chain of the configurations: the stated bound is checked there at
    full M."""
    from triton_functions import quantize_block_rowwise
    set_config(64, torch.bfloat16)
    m = 8192
    k, n = kn
    x = O.synthetic((256, k), 3333 + k % 13, outlier_frac=0.0)
    w = O.synthetic((n, k), 3334 + n % 13, std=0.02, outlier_frac=0.0)
    wq, ws = O.quantize(w, 64)
    xg = x.to(DEV).repeat(m // 256, 1)                     # 32 copies of the same 256 rows
    xq_g, xs_g = quantize_block_rowwise(xg)
    from triton_functions import int8_matmul_block64_rowwise_dequantize as mm
    c = mm(xq_g, wq.to(DEV).t(), xs_g, ws.to(DEV))
    xq, xs = O.quantize(x, 64)
    _check_bf16(c[:256], xq, wq, xs, ws, 64)
    assert torch.equal(c.view(m // 256, 256, n), c[:256].unsqueeze(0).expand(m // 256, 256, n))
    assert_clean_device()


@pytest.mark.parametrize("block", [32, 128])
@pytest.mark.parametrize("kn", [(4096, 4096), (11008, 4096)])
def test_llama_projection_shapes_other_blocks(kn, block):
    """Blocks of 32 and 128 elements on projection shapes (M = 2048; the oracle on the first 128 rows)."""
    from triton_functions import quantize_block_rowwise
    k, n = kn
    m = 2048
    set_config(block, torch.bfloat16)
    x = O.synthetic((m, k), 3500 + block, outlier_frac=0.0)
    w = O.synthetic((n, k), 3600 + block, std=0.02, outlier_frac=0.0)
    wq, ws = O.quantize(w, block)
    xq_g, xs_g = quantize_block_rowwise(x.to(DEV))
    xq, xs = O.quantize(x, block)
    assert torch.equal(xq_g.cpu(), xq) and torch.equal(xs_g.cpu(), xs)
    c = _gemm(xq, wq, xs, ws)
    rows = slice(0, 128)
    _check_bf16(c[rows], xq[rows], wq, xs[:, rows], ws, block)
    assert_clean_device()
    set_config(64)


def test_bounded_wait_gives_up_cleanly():
    """The general kernel's mbarrier waits are bounded.  bi8_gemm_wait_selftest makes one of them run out (the producer
    leaves out the copies of one K stage, the limit is set to 200 us): the kernel must return by itself, the device
    status must say BI8_ERR_TIMEOUT with the code of the wait for operand tiles, and the next ordinary GEMM must be
    correct (the tensor memory was freed, nothing is left hanging)."""
    import ctypes
    from blockwise_int8_linear_b200 import _lib
    L = _lib.lib()
    set_config(64, torch.float32)
    m, k, n = 256, 1024, 320
    xq, xs, wq, ws = quantized_pair(m, k, n, 64, seed=4242)
    a, bt, sa, sb = xq.to(DEV), wq.to(DEV), xs.to(DEV), ws.to(DEV)
    c = torch.empty((m, n), dtype=torch.float32, device=DEV)
    assert _lib.device_status() == 0
    for skip in (0, 3):
        rc = L.bi8_gemm_wait_selftest(_lib.ptr(a), k, _lib.ptr(bt), k, _lib.ptr(sa), _lib.ptr(sb), _lib.ptr(c), n, _lib.BI8_F32,
                                      m, n, k, 64, 200, skip, _lib.stream_ptr())
        _lib.check(rc, "bi8_gemm_wait_selftest")
        torch.cuda.synchronize()                       # returns: the kernel left its loops by itself
        detail = ctypes.c_int(0)
        assert L.bi8_device_status(ctypes.byref(detail)) == -6      # BI8_ERR_TIMEOUT
        assert detail.value == 2                                      # wait for the operand tiles of a stage
        assert _lib.device_status() == 0                              # reading cleared the word
        good = _gemm(xq, wq, xs, ws, flags=TC)
        _check_fp32(good, xq, wq, xs, ws, 64)
    assert_clean_device()
    set_config(64)


def test_unaligned_long_contraction_is_repitched_onto_the_tensor_cores():
    """K = 1000 + 17: not a multiple of 16.  The shim re-pitches the operands; results equal the CUDA-core kernel's
    within the tensor-core tolerance and the int32 partial sums stay exact."""
    from triton_functions import int8_matmul_block_partials
    set_config(64, torch.float32)
    m, k, n = 160, 1017, 200
    xq, xs, wq, ws = quantized_pair(m, k, n, 64, seed=77)
    c = _gemm(xq, wq, xs, ws)
    _check_fp32(c, xq, wq, xs, ws, 64)
    p = int8_matmul_block_partials(xq.to(DEV), wq.to(DEV).t(), 64)
    assert torch.equal(p.cpu(), O.gemm_block_partials(xq, wq.t(), 64))
    set_config(64)


SMALLM = 8
SMALL_SHAPES = [
    # (M, K, N, block)
    (1, 64, 4, 64), (1, 4096, 512, 64), (5, 1056, 75, 64), (8, 2048, 1000, 64), (9, 256, 260, 64), (16, 4096, 1024, 64),
    (3, 192, 33, 32), (8, 1056, 130, 32), (16, 2048, 256, 128), (7, 416, 50, 128), (2, 11008, 64, 64),
]


@pytest.mark.parametrize("shape", SMALL_SHAPES)
def test_small_m_weight_streaming_kernel(shape):
    """M <= 16 (decode): the CUDA-core weight-streaming kernel.  Every term is evaluated in the reference's order; only the
    order of the fp32 additions differs, so the tensor-core tolerance applies; bf16 results as for the tensor-core kernel."""
    m, k, n, block = shape
    xq, xs, wq, ws = quantized_pair(m, k, n, block, seed=11 * m + k + n)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(n)).to(torch.bfloat16)
    set_config(block, torch.float32)
    _check_fp32(_gemm(xq, wq, xs, ws, flags=SMALLM), xq, wq, xs, ws, block)
    _check_fp32(_gemm(xq, wq, xs, ws, bias, flags=SMALLM), xq, wq, xs, ws, block, bias)
    if m <= 8:
        # default dispatch: the skinny tensor-core kernel where it applies (N % 4 == 0), else this kernel
        chosen = 16 if n % 4 == 0 else SMALLM
        assert torch.equal(_gemm(xq, wq, xs, ws), _gemm(xq, wq, xs, ws, flags=chosen)), "default dispatch for M <= 8"
    set_config(block, torch.bfloat16)
    _check_bf16(_gemm(xq, wq, xs, ws, bias, flags=SMALLM), xq, wq, xs, ws, block, bias)
    from blockwise_int8_linear_b200._lib import Bi8Error
    with pytest.raises(Bi8Error):
        big = quantized_pair(17, 128, 32, block, seed=1)
        _gemm(big[0], big[2], big[1], big[3], flags=SMALLM)
    assert_clean_device()
    set_config(64)


SKINNY = 16
SKINNY_SHAPES = [
    # (M, K, N, block): N % 4 == 0, K % 16 == 0; tiles both divided over CTAs and undivided, K and N tails
    (1, 64, 4, 64), (1, 4096, 512, 64), (5, 1056, 76, 64), (8, 2048, 1000, 64), (9, 256, 260, 64), (16, 4096, 1024, 64),
    (3, 192, 36, 32), (8, 1056, 132, 32), (16, 2048, 256, 128), (7, 416, 52, 128), (2, 11008, 64, 64),
    (17, 512, 384, 64), (32, 4096, 640, 64), (25, 1056, 260, 32), (32, 2048, 128, 128), (8, 4096, 11008, 64),
    (4, 128, 40000, 64), (12, 80, 24, 32), (8, 256, 14336, 64),      # the last: 112 tiles, one whole tile per CTA
    # 33..64 activation rows: promotion warps of 32 columns
    (33, 512, 384, 64), (64, 4096, 640, 64), (50, 1056, 260, 64), (64, 2048, 256, 128), (48, 4096, 1024, 64),
    (64, 1056, 132, 32), (41, 11008, 128, 64),
]


@pytest.mark.parametrize("shape", SKINNY_SHAPES)
def test_skinny_tensor_core_kernel(shape):
    """M <= 64 (decode, small batches): tensor-core kernel with exchanged operand roles.  Terms are evaluated in the reference's order;
    a tile whose K range is divided over CTAs adds its parts in a fixed order, so the tensor-core tolerance applies and
    repeated calls are bit-identical."""
    m, k, n, block = shape
    xq, xs, wq, ws = quantized_pair(m, k, n, block, seed=13 * m + k + n)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(n)).to(torch.bfloat16)
    set_config(block, torch.float32)
    first = _gemm(xq, wq, xs, ws, flags=SKINNY)
    _check_fp32(first, xq, wq, xs, ws, block)
    assert torch.equal(first, _gemm(xq, wq, xs, ws, flags=SKINNY)), "deterministic"
    _check_fp32(_gemm(xq, wq, xs, ws, bias, flags=SKINNY), xq, wq, xs, ws, block, bias)
    set_config(block, torch.bfloat16)
    _check_bf16(_gemm(xq, wq, xs, ws, bias, flags=SKINNY), xq, wq, xs, ws, block, bias)
    from blockwise_int8_linear_b200._lib import Bi8Error
    with pytest.raises(Bi8Error):
        big = quantized_pair(65, 128, 32, block, seed=1)
        _gemm(big[0], big[2], big[1], big[3], flags=SKINNY)
    assert_clean_device()
    set_config(64)


FUSED_SHAPES = [
    # (M, K, N, block, dtype)
    (1, 4096, 512, 64, torch.bfloat16), (8, 2048, 1000, 64, torch.bfloat16), (5, 1056, 76, 64, torch.bfloat16),
    (16, 4096, 1024, 64, torch.float16), (7, 416, 52, 128, torch.float32), (3, 208, 36, 32, torch.bfloat16),
    (17, 512, 384, 64, torch.bfloat16), (32, 1056, 260, 32, torch.float32), (32, 2048, 128, 128, torch.float16),
    (8, 4096, 11008, 64, torch.bfloat16), (2, 11008, 4096, 64, torch.bfloat16),
    (40, 512, 256, 64, torch.bfloat16), (64, 4096, 512, 64, torch.bfloat16), (50, 1056, 260, 128, torch.float16),
    (4, 512, 50, 64, torch.bfloat16), (200, 512, 256, 64, torch.bfloat16),     # not eligible: run as two kernels
]


@pytest.mark.parametrize("shape", FUSED_SHAPES)
def test_quantize_on_load_gemm(shape):
    """bi8_gemm_dequant_fused_quant: quantize + GEMM in one call.  For M <= 32 either a decode quantizer kernel overlapped
    with the GEMM's start (default) or quantization inside the GEMM kernel (flag 32).  The quantized activations are
    bit-identical to the standalone quantizer's, so the result must equal the two-call sequence exactly, which in turn
    is checked against the oracle."""
    from triton_functions import (int8_matmul_block64_rowwise_dequantize as mm, quantize_block_rowwise,
                                  quantize_matmul_block_rowwise_dequantize as qmm)
    m, k, n, block, dtype = shape
    x = randn_bf16((m, k), seed=3 * m + k).to(dtype)
    if dtype == torch.float32:
        x = x + torch.randn((m, k), generator=torch.Generator().manual_seed(k)) * 1e-3      # full fp32 mantissas
    x[0, : min(k, block)] = 0                                                                # an all-zero block
    w = randn_bf16((n, k), seed=k + n, std=0.02)
    wq, ws = O.quantize(w, block)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(n)).to(torch.bfloat16)
    for out_dtype in (torch.float32, torch.bfloat16):
        set_config(block, out_dtype)
        xd, wqd, wsd = x.to(DEV), wq.to(DEV), ws.to(DEV)
        xq, xs = quantize_block_rowwise(xd)
        two = mm(xq, wqd.t(), xs, wsd, bias.to(DEV))
        one = qmm(xd, wqd.t(), wsd, bias.to(DEV))
        assert torch.equal(one, two)
        assert torch.equal(qmm(xd, wqd.t(), wsd, bias.to(DEV), flags=32), two), "quantized inside the GEMM kernel"
        assert torch.equal(one, qmm(xd, wqd.t(), wsd, bias.to(DEV))), "deterministic"
    set_config(block, torch.float32)
    oq, os_ = O.quantize(x, block)
    _check_fp32(qmm(x.to(DEV), wq.to(DEV).t(), ws.to(DEV)), oq, wq, os_, ws, block)
    assert_clean_device()
    set_config(64)


def test_zero_sized():
    from triton_functions import int8_matmul_block64_rowwise_dequantize as mm
    set_config(64)
    a = torch.empty((0, 128), dtype=torch.int8, device=DEV)
    b = torch.zeros((256, 128), dtype=torch.int8, device=DEV)
    c = mm(a, b.t(), torch.empty((2, 0), device=DEV), torch.ones((2, 256), device=DEV))
    assert tuple(c.shape) == (0, 256)
