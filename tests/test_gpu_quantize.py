"""Block quantize / dequantize on the GPU against the CPU oracle and the golden vectors: bit-exact."""
import pytest
import torch

from oracle import blockwise_int8_oracle as O
from tests.gpu_util import DEV, assert_clean_device, randn_bf16, set_config
from tests.helpers import golden_names, load_golden

pytestmark = pytest.mark.gpu


def _q(x, block=None):
    from triton_functions import quantize_block_rowwise
    return quantize_block_rowwise(x, block)


def _check_quant(x_cpu, block, **kw):
    q_ref, s_ref = O.quantize(x_cpu, block)
    q, s = _q(x_cpu.to(DEV), block)
    assert q.dtype == torch.int8 and s.dtype == torch.float32
    assert tuple(q.shape) == tuple(x_cpu.shape) and tuple(s.shape) == tuple(s_ref.shape)
    assert torch.equal(s.cpu(), s_ref), "scales differ"
    neq = (q.cpu() != q_ref).sum().item()
    assert neq == 0, f"{neq} int8 values differ"


@pytest.mark.parametrize("name", golden_names("ops_"))
def test_golden_quantize(name):
    g = load_golden(name)
    for src, qk, sk in (("x", "xq", "xs"), ("w", "wq", "ws")):
        q, s = _q(g[src].to(DEV), g["block"])
        assert torch.equal(q.cpu(), g[qk]) and torch.equal(s.cpu(), g[sk])


@pytest.mark.parametrize("name", golden_names("ops_"))
def test_golden_dequantize(name):
    from triton_functions import dequantize_block_rowwise
    g = load_golden(name)
    for dt in (torch.float32, torch.bfloat16):
        set_config(g["block"], dt)
        d = dequantize_block_rowwise(g["xq"].to(DEV), g["xs"].to(DEV))
        assert d.dtype == dt
        assert torch.equal(d.cpu(), g["x_deq_f32"].to(dt))
    set_config(64)


@pytest.mark.parametrize("shape", [(4096, 4096), (8192, 8192)])
def test_config_sweep_shapes(shape):
    """BASELINE config: N(0,1) + 0.1 % x20 outliers, block 64; int8 and scales bit-exact."""
    _check_quant(randn_bf16(shape, 2001 + shape[0]), 64)


def test_largest_config_shape_sampled():
    """16384 x 16384: rows sampled against the oracle, plus determinism of two runs."""
    m = k = 16384
    g = torch.Generator(device=DEV).manual_seed(2003)
    x = torch.randn((m, k), device=DEV, dtype=torch.float32, generator=g)
    x = torch.where(torch.rand((m, k), device=DEV, generator=g) < 0.001, x * 20, x).to(torch.bfloat16)
    q, s = _q(x, 64)
    q2, s2 = _q(x, 64)
    assert torch.equal(q, q2) and torch.equal(s, s2)
    rows = torch.cat([torch.arange(0, 64), torch.arange(8000, 8064), torch.arange(m - 64, m)])
    q_ref, s_ref = O.quantize(x[rows.to(DEV)].cpu(), 64)
    assert torch.equal(q[rows.to(DEV)].cpu(), q_ref)
    assert torch.equal(s[:, rows.to(DEV)].cpu(), s_ref)
    # size-independent property: every block holds +-127 exactly where |x| equals the block scale
    assert int(q.abs().max()) == 127
    del x, q, s, q2, s2


@pytest.mark.parametrize("block", [32, 64, 128, 256])
@pytest.mark.parametrize("shape", [(1, 256), (33, 512), (40, 1040), (257, 72), (31, 1000), (5, 150), (64, 17), (40, 50257)])
def test_ragged_shapes_and_blocks(shape, block):
    # K % 16 == 0: 32-byte lanes; K % 8 == 0: 16-byte lanes; otherwise the generic kernel; K tails in every case
    _check_quant(randn_bf16(shape, shape[0] * 131 + shape[1], outliers=0.01), block)


@pytest.mark.parametrize("block", [48, 96, 512])
def test_unusual_block_sizes(block):
    _check_quant(randn_bf16((19, 1000), block), block)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_other_input_types(dtype):
    x = torch.randn((37, 200), generator=torch.Generator().manual_seed(7)).to(dtype)
    _check_quant(x, 64)
    _check_quant(x[:, :192].contiguous(), 32)


def test_zero_blocks_and_extremes():
    x = randn_bf16((16, 256), 11)
    x[0, :64] = 0
    x[3] = 0
    x[5, 64:128] = 3.0e38          # huge scale: outside the fast-division range
    x[5, 70] = -1.5e38
    x[6, :64] = 1.0e-38            # tiny scale
    x[6, 3] = -2.0e-39
    x[7, 128:192] = 9.2e-41        # denormal bf16 values
    _check_quant(x, 64)


def test_near_ties():
    """127*x/s close to n + 0.5 for many (x, s): needs the IEEE quotient, not a reciprocal product."""
    g = torch.Generator().manual_seed(5)
    s = (torch.rand(512, generator=g) * 3 + 0.5).to(torch.bfloat16).float()
    n = torch.randint(-126, 126, (512, 64), generator=g).float() + 0.5
    x = (n / 127.0 * s[:, None]).to(torch.bfloat16)
    x[:, 0] = s.to(torch.bfloat16)
    _check_quant(x.reshape(64, 512).contiguous(), 64)
    _check_quant(x, 64)


def test_row_strided_input():
    base = randn_bf16((48, 1024), 13).to(DEV)
    view = base[:, 256:768]                       # row pitch 1024, 512 columns
    q, s = _q(view, 64)
    q_ref, s_ref = O.quantize(view.cpu().contiguous(), 64)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    tq, ts = _q(base.t(), 64)                     # column-major view: made contiguous first
    tq_ref, ts_ref = O.quantize(base.cpu().t().contiguous(), 64)
    assert torch.equal(tq.cpu(), tq_ref) and torch.equal(ts.cpu(), ts_ref)


@pytest.mark.parametrize("block", [32, 64, 128, 256, 48])
@pytest.mark.parametrize("shape", [(128, 128), (200, 136), (64, 1000), (1000, 64), (70, 33), (8192, 768), (130, 50257), (50257, 40)])
def test_colwise_equals_transpose_then_rowwise(shape, block):
    from triton_functions import quantize_block_colwise
    x = randn_bf16(shape, shape[0] + 7 * shape[1], outliers=0.01)
    q, s = quantize_block_colwise(x.to(DEV), block)
    q_ref, s_ref = O.quantize(x.t().contiguous(), block)
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu(), q_ref)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("block", [32, 64, 128, 48])
@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (208, 144), (48, 1008), (1008, 48), (8192, 768), (4096, 4096),
                                   (70, 33), (200, 136), (130, 50257)])
def test_dual_equals_both_single_quantizers(shape, block, dt):
    """One read, both quantizations: each output must be bit-identical to its single-purpose function and to the
    oracle (zero columns, NaN-free outliers and ragged tile edges included; shapes the one-pass kernel does not take go
    through the two single kernels)."""
    from triton_functions import quantize_block_colwise, quantize_block_dual, quantize_block_rowwise
    x = randn_bf16(shape, 3 * shape[0] + shape[1], outliers=0.01).to(dt)
    x[:, 1] = 0                                     # a column of zeros: scale 0, result 0
    x[0, :] = 0
    xd = x.to(DEV)
    q_row, s_row, q_col, s_col = quantize_block_dual(xd, block)
    q1, s1 = quantize_block_rowwise(xd, block)
    q2, s2 = quantize_block_colwise(xd, block)
    assert torch.equal(q_row, q1) and torch.equal(s_row, s1)
    assert torch.equal(q_col, q2) and torch.equal(s_col, s2)
    if shape[0] * shape[1] <= 1 << 22:
        qr, sr = O.quantize(x.float() if dt == torch.float16 else x, block)
        qc, sc = O.quantize((x.float() if dt == torch.float16 else x).t().contiguous(), block)
        assert torch.equal(q_row.cpu(), qr) and torch.equal(s_row.cpu(), sr)
        assert torch.equal(q_col.cpu(), qc) and torch.equal(s_col.cpu(), sc)
    assert_clean_device()


def test_dual_strided_rows_and_extremes():
    """Row pitch larger than the row, values at the ends of the bf16 range, and a block whose only nonzero is subnormal in
    fp32 terms (the exact-division shortcut must hand over to the IEEE division there)."""
    from triton_functions import quantize_block_colwise, quantize_block_dual, quantize_block_rowwise
    base = randn_bf16((256, 512), 5).to(DEV)
    base[3, 130] = 3.0e38
    base[64:128, 200] = 1e-38
    base[64:128, 201] = 0
    base[70, 201] = 1e-39
    view = base[:, 128:384]
    q_row, s_row, q_col, s_col = quantize_block_dual(view, 64)
    q1, s1 = quantize_block_rowwise(view, 64)
    q2, s2 = quantize_block_colwise(view, 64)
    assert torch.equal(q_row, q1) and torch.equal(s_row, s1) and torch.equal(q_col, q2) and torch.equal(s_col, s2)
    qc, sc = O.quantize(view.cpu().t().contiguous(), 64)
    assert torch.equal(q_col.cpu(), qc) and torch.equal(s_col.cpu(), sc)


def test_colwise_fp32():
    from triton_functions import quantize_block_colwise
    x = torch.randn((130, 72), generator=torch.Generator().manual_seed(3))
    q, s = quantize_block_colwise(x.to(DEV), 64)
    q_ref, s_ref = O.quantize(x.t().contiguous(), 64)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape,block", [((4096, 4096), 64), ((33, 1040), 64), ((7, 150), 64), ((65, 512), 32),
                                         ((16, 1024), 128), ((9, 768), 256), ((12, 100), 48)])
def test_dequantize(shape, block, dt):
    from triton_functions import dequantize_block_rowwise
    set_config(block, dt)
    x = randn_bf16(shape, 17 + shape[1])
    q_ref, s_ref = O.quantize(x, block)
    if dt == torch.float16:
        ref = O.dequantize(q_ref, s_ref, block, torch.float32).to(torch.float16)
    else:
        ref = O.dequantize(q_ref, s_ref, block, dt)
    d = dequantize_block_rowwise(q_ref.to(DEV), s_ref.to(DEV))
    assert d.dtype == dt and torch.equal(d.cpu(), ref)
    set_config(64)


def test_empty_inputs():
    from triton_functions import dequantize_block_rowwise
    set_config(64)
    q, s = _q(torch.empty((0, 128), dtype=torch.bfloat16, device=DEV), 64)
    assert tuple(q.shape) == (0, 128) and tuple(s.shape) == (2, 0)
    q, s = _q(torch.empty((4, 0), dtype=torch.bfloat16, device=DEV), 64)
    assert tuple(q.shape) == (4, 0) and tuple(s.shape) == (0, 4)
    d = dequantize_block_rowwise(torch.empty((0, 64), dtype=torch.int8, device=DEV),
                                 torch.empty((1, 0), dtype=torch.float32, device=DEV))
    assert tuple(d.shape) == (0, 64)


def test_errors():
    from triton_functions import dequantize_block_rowwise
    with pytest.raises(AssertionError):
        _q(torch.zeros((4, 64), dtype=torch.bfloat16), 64)          # CPU tensor: the reference asserts is_cuda
    with pytest.raises(ValueError):
        _q(torch.zeros((4, 64), dtype=torch.int32, device=DEV), 64)
    with pytest.raises(ValueError):
        dequantize_block_rowwise(torch.zeros((4, 64), dtype=torch.int8, device=DEV),
                                 torch.zeros((4, 1), dtype=torch.float32, device=DEV), 64)
    assert_clean_device()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs a second GPU")
@pytest.mark.parametrize("shape", [(256, 384), (200, 136)])
def test_colwise_block128_on_second_device(shape):
    """Per-device kernel attributes: block 128 needs more than the default 48 KiB of dynamic shared memory in both
    column-wise kernels (the TMA tile kernel takes the first shape, the shared-memory tile kernel the second), and the
    opt-in must have been made on the device the call runs on, not only on the first device the process used."""
    from triton_functions import quantize_block_colwise, quantize_block_dual
    x = randn_bf16(shape, 77, outliers=0.01)
    q0, s0 = quantize_block_colwise(x.to("cuda:0"), 128)
    q1, s1 = quantize_block_colwise(x.to("cuda:1"), 128)
    q_ref, s_ref = O.quantize(x.t().contiguous(), 128)
    assert torch.equal(q0.cpu(), q_ref) and torch.equal(s0.cpu(), s_ref)
    assert torch.equal(q1.cpu(), q_ref) and torch.equal(s1.cpu(), s_ref)
    d = quantize_block_dual(x.to("cuda:1"), 128)
    assert d[2].device.index == 1 and torch.equal(d[2].cpu(), q_ref) and torch.equal(d[3].cpu(), s_ref)


@pytest.mark.parametrize("shape", [(4099, 1031), (1031, 4099), (4112, 1031)])
def test_large_unaligned_tensors_are_padded_not_slowed(shape):
    """Large 16-bit tensors whose row or column count is not a multiple of 16 (GPT-2's 50257-wide logits) are copied once
    into a zero-padded buffer and go through the fast kernels; the results (returned as views of the padded outputs)
    must equal the oracle's on the unpadded tensor, bit for bit."""
    from triton_functions import quantize_block_colwise, quantize_block_dual, quantize_block_rowwise
    x = randn_bf16(shape, 11 * shape[0] + shape[1], outliers=0.01)
    xd = x.to(DEV)
    qr_ref, sr_ref = O.quantize(x, 64)
    qc_ref, sc_ref = O.quantize(x.t().contiguous(), 64)
    q, s = quantize_block_rowwise(xd, 64)
    assert tuple(q.shape) == shape and torch.equal(q.cpu(), qr_ref) and torch.equal(s.cpu(), sr_ref)
    q, s = quantize_block_colwise(xd, 64)
    assert tuple(q.shape) == shape[::-1] and torch.equal(q.cpu(), qc_ref) and torch.equal(s.cpu(), sc_ref)
    a, b, c, d = quantize_block_dual(xd, 64)
    assert torch.equal(a.cpu(), qr_ref) and torch.equal(b.cpu(), sr_ref) and torch.equal(c.cpu(), qc_ref) and torch.equal(d.cpu(), sc_ref)
    assert_clean_device()


def test_tensor_map_kernels_from_a_fresh_thread():
    """A host thread that has made no CUDA call yet has no context current, and the tensor-map encode is a driver call: the
    library binds the primary context itself (an autograd worker thread whose first CUDA work is this layer's backward
    is such a thread)."""
    import threading
    from triton_functions import (int8_matmul_block64_rowwise_dequantize, quantize_block_colwise, quantize_block_dual,
                                  quantize_block_rowwise)
    set_config(64, torch.bfloat16)
    x = randn_bf16((256, 512), 21).to(DEV)
    w = randn_bf16((384, 512), 22).to(DEV)
    xq, xs = quantize_block_rowwise(x)
    wq, ws = quantize_block_rowwise(w)
    want = (quantize_block_dual(x), quantize_block_colwise(x), int8_matmul_block64_rowwise_dequantize(xq, wq.t(), xs, ws))
    torch.cuda.synchronize()
    got, errors = [], []

    def work():
        try:
            got.append((quantize_block_dual(x), quantize_block_colwise(x), int8_matmul_block64_rowwise_dequantize(xq, wq.t(), xs, ws)))
            torch.cuda.synchronize()
        except Exception as e:            # reported in the main thread
            errors.append(e)

    t = threading.Thread(target=work)
    t.start()
    t.join()
    assert not errors, errors
    for a, b in zip(want[0], got[0][0]):
        assert torch.equal(a, b)
    assert torch.equal(want[1][0], got[0][1][0]) and torch.equal(want[2], got[0][2])
