"""The quantizers with a fused producer step (normalisation, gated activation) and the layer call built on them:
CUDA library against the CPU oracle and against the unfused library calls."""
import pytest
import torch
import torch.nn.functional as F

from oracle import blockwise_int8_oracle as O
from tests.gpu_util import DEV, assert_clean_device, randn_bf16, set_config

pytestmark = pytest.mark.gpu

EPS = 1e-5


def _tf():
    import triton_functions as tf
    return tf


def _dequant(q, s, block):
    """fp32 q * s / 127 (exact products of small integers and scales, no rounding to a 16-bit type)."""
    m, k = q.shape
    s_full = s.t().repeat_interleave(block, dim=1)[:, :k]
    return q.float() * s_full / 127.0


@pytest.mark.parametrize("shape", [(8, 4096), (1, 4096), (33, 11008), (5, 768), (3, 8200), (2, 16384), (300, 512), (1500, 1024)])
@pytest.mark.parametrize("block", [64, 128, 32])
def test_rmsnorm_quantize_integer_rows_bit_exact(shape, block):
    """Rows of small integers: the sum of squares is exact in any order, so the fused kernel must return exactly what
    the stand-alone quantizer returns for the normalised tensor built from elementwise torch operations."""
    set_config(block)
    tf = _tf()
    g = torch.Generator().manual_seed(shape[0] * 131 + shape[1])
    x = torch.randint(-6, 7, shape, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randint(1, 5, (shape[1],), generator=g).float() / 2).to(torch.bfloat16).to(DEV)
    for weight in (None, w):
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) / shape[1] + EPS)
        y = xf * rstd
        if weight is not None:
            y = y * weight.float()
        want_q, want_s = tf.quantize_block_rowwise(y.to(torch.bfloat16))
        q, s = tf.rmsnorm_quantize_block_rowwise(x, EPS, weight)
        assert torch.equal(s, want_s)
        assert torch.equal(q, want_q)
    assert_clean_device()


@pytest.mark.parametrize("shape", [(8, 4096), (40, 11008), (7, 1000), (3, 150), (2, 9000)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_rmsnorm_quantize_against_oracle(shape, dt):
    """Random rows against the CPU restatement: the two sums of squares differ in their last bits, which may move a
    normalised value by one step of the activation type, i.e. an int8 value by one, a scale by one step."""
    block = 64
    set_config(block)
    tf = _tf()
    x = randn_bf16(shape, 77 + shape[1]).to(dt)
    want_q, want_s = O.rmsnorm_quantize(x, block, EPS)
    q, s = tf.rmsnorm_quantize_block_rowwise(x.to(DEV), EPS)
    q, s = q.cpu(), s.cpu()
    assert q.shape == want_q.shape and s.shape == want_s.shape
    step = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10, torch.float32: 2.0 ** -20}[dt]
    assert ((s - want_s).abs() <= step * want_s).all()
    assert (q.int() - want_q.int()).abs().max().item() <= 1
    assert (q != want_q).float().mean().item() <= 0.02
    # repeated calls return the same bits (fixed summation order)
    q2, s2 = tf.rmsnorm_quantize_block_rowwise(x.to(DEV), EPS)
    assert torch.equal(q2.cpu(), q) and torch.equal(s2.cpu(), s)
    assert_clean_device()


@pytest.mark.parametrize("shape", [(8, 11008), (1, 1408), (64, 2752), (5, 1000), (3, 150), (200, 704)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("block", [64, 128])
def test_silu_mul_quantize_bit_exact(shape, dt, block):
    """Against the three separate steps on the GPU (torch silu, torch multiply, the library's quantizer) and against the
    oracle; gate and up are the two halves of one tensor, as a fused gate_up projection leaves them."""
    set_config(block)
    tf = _tf()
    m, k = shape
    both = randn_bf16((m, 2 * k), 5 + k, std=2.0).to(dt)
    gu = both.to(DEV)
    gate, up = gu[:, :k], gu[:, k:]
    q, s = tf.silu_mul_quantize_block_rowwise(gate, up)
    want_q, want_s = tf.quantize_block_rowwise(F.silu(gate) * up)
    assert torch.equal(s, want_s)
    assert torch.equal(q, want_q)
    if dt != torch.float32:        # torch's CPU exp may differ from the GPU's in the last bit of an fp32 result
        oq, os_ = O.silu_mul_quantize(both[:, :k], both[:, k:], block)
        assert (q.cpu().int() - oq.int()).abs().max().item() <= 1
        assert (q.cpu() != oq).float().mean().item() <= 0.001
        assert ((s.cpu() - os_).abs() <= 2.0 ** -7 * os_).all()
    assert_clean_device()


def test_pre_quantizers_empty_and_errors():
    set_config(64)
    tf = _tf()
    from blockwise_int8_linear_b200 import _lib
    q, s = tf.rmsnorm_quantize_block_rowwise(torch.empty((0, 128), device=DEV, dtype=torch.bfloat16))
    assert q.shape == (0, 128) and s.shape == (2, 0)
    x = torch.randn((4, 128), device=DEV).to(torch.bfloat16)
    with pytest.raises(ValueError):
        tf.silu_mul_quantize_block_rowwise(x, x[:, :64])
    with pytest.raises(ValueError):
        tf.rmsnorm_quantize_block_rowwise(x, EPS, torch.ones(64, device=DEV))
    with pytest.raises(ValueError):
        tf.pre_quantize_matmul_block_rowwise_dequantize("gelu", x, torch.zeros((128, 8), device=DEV, dtype=torch.int8),
                                                        torch.ones((2, 8), device=DEV))
    rc = _lib.lib().bi8_quantize_rowwise_pre(7, _lib.ptr(x), None, 0, 128, None, 0.0, _lib.ptr(x), _lib.ptr(x), 4, 128, 64, None)
    assert rc == -4
    # an all-zero row: rsqrt(eps) * 0 = 0, scale 0, q 0
    z = torch.zeros((2, 128), device=DEV, dtype=torch.bfloat16)
    q, s = tf.rmsnorm_quantize_block_rowwise(z)
    assert not q.any() and not s.any()
    assert_clean_device()


@pytest.mark.parametrize("m", [1, 8, 33, 64, 70, 300])
@pytest.mark.parametrize("op", ["none", "rmsnorm", "silu_mul"])
def test_fused_layer_call_equals_separate_steps(m, op):
    """pre_quantize_matmul_block_rowwise_dequantize against producer quantizer + GEMM + torch addition: bit-identical
    (the decode path divides tiles over CTAs exactly as the unfused call does), with and without residual, in place,
    with bias, bf16 and fp32 output."""
    block = 64
    tf = _tf()
    import block_linear_config as cfg
    k, n = 1408, 4096
    set_config(block)
    w = randn_bf16((n, k), 11, std=0.02).to(DEV)
    wq, sw = tf.quantize_block_rowwise(w)
    x = randn_bf16((m, 2 * k), 12 + m, std=1.5).to(DEV)
    a, b = x[:, :k], x[:, k:]
    bias = randn_bf16((n,), 13).to(DEV)
    if op == "none":
        xq, sx = tf.quantize_block_rowwise(a)
    elif op == "rmsnorm":
        xq, sx = tf.rmsnorm_quantize_block_rowwise(a, EPS)
    else:
        xq, sx = tf.silu_mul_quantize_block_rowwise(a, b)
    for out_dtype in (torch.bfloat16, torch.float32):
        cfg.INPUT_OUTPUT_TORCH_TYPE = out_dtype
        res = randn_bf16((m, n), 14).to(out_dtype).to(DEV)
        for use_bias in (False, True):
            base = tf.int8_matmul_block64_rowwise_dequantize(xq, wq.t(), sx, sw, bias if use_bias else None)
            kw = dict(x2=b if op == "silu_mul" else None, eps=EPS)
            got = tf.pre_quantize_matmul_block_rowwise_dequantize(op, a, wq.t(), sw, bias if use_bias else None, **kw)
            assert torch.equal(got, base), (m, op, out_dtype, use_bias)
            got = tf.pre_quantize_matmul_block_rowwise_dequantize(op, a, wq.t(), sw, bias if use_bias else None, residual=res, **kw)
            assert torch.equal(got, base + res), (m, op, out_dtype, use_bias, "residual")
            inplace = res.clone()
            got = tf.pre_quantize_matmul_block_rowwise_dequantize(op, a, wq.t(), sw, bias if use_bias else None, residual=inplace,
                                                                  out=inplace, **kw)
            assert got is inplace and torch.equal(inplace, base + res), (m, op, out_dtype, use_bias, "in place")
    cfg.INPUT_OUTPUT_TORCH_TYPE = torch.bfloat16
    assert_clean_device()


def test_module_infer_pre_and_graph_replay():
    """BlockInt8Linear.infer_pre against infer on the separately computed input, eager and replayed from a CUDA graph
    (the decode path: quantizer, GEMM and reduction are one chain of programmatic dependents)."""
    set_config(64)
    from block_linear import BlockInt8Linear
    lin = BlockInt8Linear(4096, 1024, bias=False, device=DEV, dtype=torch.bfloat16).eval()
    lin.weight.data = randn_bf16((1024, 4096), 3, std=0.02).to(DEV)
    x = randn_bf16((2, 4, 4096), 4).to(DEV)
    res = randn_bf16((2, 4, 1024), 5).to(DEV)
    with torch.no_grad():
        q, s = _tf().rmsnorm_quantize_block_rowwise(x.view(-1, 4096), EPS)
        lin.infer(x)                                            # registers W_int8 / state_W
        want = _tf().int8_matmul_block64_rowwise_dequantize(q, lin.W_int8.t(), s, lin.state_W).view(2, 4, 1024) + res
        got = lin.infer_pre(x, "rmsnorm", eps=EPS, residual=res)
        assert torch.equal(got, want)
        gate_up = randn_bf16((8, 8192), 6, std=2.0).to(DEV)
        gate, up = gate_up[:, :4096], gate_up[:, 4096:]
        assert torch.equal(lin.infer_pre(gate, "silu_mul", x2=up), lin.infer(F.silu(gate) * up))
        # graph: the residual stream updated in place, three replays = three layers' worth of updates
        stream = res.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            lin.infer_pre(x, "rmsnorm", eps=EPS, residual=stream.clone())
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = _tf().pre_quantize_matmul_block_rowwise_dequantize("rmsnorm", x.view(-1, 4096), lin.W_int8.t(), lin.state_W, eps=EPS,
                                                                     residual=stream.view(-1, 1024), out=stream.view(-1, 1024))
        expect = res.clone()
        proj = _tf().int8_matmul_block64_rowwise_dequantize(q, lin.W_int8.t(), s, lin.state_W).view(2, 4, 1024)
        for _ in range(3):
            graph.replay()
            expect = expect + proj
        torch.cuda.synchronize()
        assert torch.equal(stream, expect)
    assert_clean_device()


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(8, 32, 128, 545), (2, 4, 64, 30), (1, 1, 2, 3)])
def test_rope_cache_append(dt, shape):
    """One decode step's rotary embedding and cache append in one launch: bit-identical to the same arithmetic written with
    tensor operations (fp32 products and sums rounded one by one), within one step of the activation type of torch's
    complex multiply, and the caches change in row `pos` only; replayed from a CUDA graph the row follows the position."""
    from blockwise_int8_linear_b200.decode_ops import rope_cache_append
    b, h, d, max_len = shape
    g = torch.Generator(device=DEV).manual_seed(b * 1000 + d)
    qkv = torch.randn((b, 3, h, d), device=DEV, generator=g).to(dt)
    ang = torch.rand((d // 2,), device=DEV, generator=g) * 6.28
    cis = torch.polar(torch.ones_like(ang), ang)
    kc = torch.randn((b, h, max_len, d), device=DEV, generator=g).to(dt)
    vc = torch.randn((b, h, max_len, d), device=DEV, generator=g).to(dt)
    k0, v0 = kc.clone(), vc.clone()
    pos = torch.tensor([max_len - 2], device=DEV, dtype=torch.long)
    q = rope_cache_append(qkv, cis, pos, kc, vc)

    def rotate(x):                       # [b, h, d] -> rotated, explicit real arithmetic
        x0, x1 = x[..., 0::2].float(), x[..., 1::2].float()
        c, s = cis.real, cis.imag
        return torch.stack(((x0 * c) - (x1 * s), (x0 * s) + (x1 * c)), dim=-1).flatten(-2).to(dt)

    assert torch.equal(q[:, :, 0], rotate(qkv[:, 0]))
    p = pos.item()
    assert torch.equal(kc[:, :, p], rotate(qkv[:, 1])) and torch.equal(vc[:, :, p], qkv[:, 2])
    keep = torch.ones(max_len, dtype=torch.bool, device=DEV)
    keep[p] = False
    assert torch.equal(kc[:, :, keep], k0[:, :, keep]) and torch.equal(vc[:, :, keep], v0[:, :, keep])
    # torch's complex multiply (the driver's prefill path)
    xc = torch.view_as_complex(qkv[:, 0].float().reshape(b, h, d // 2, 2))
    ref = torch.view_as_real(xc * cis).flatten(-2).to(dt)
    step = 2.0 ** -7 if dt == torch.bfloat16 else 2.0 ** -10
    assert (q[:, :, 0].float() - ref.float()).abs().max().item() <= step * ref.float().abs().max().item()
    # a position outside the cache writes nothing; a replayed graph follows the position
    k1 = kc.clone()
    rope_cache_append(qkv, cis, torch.tensor([max_len], device=DEV), kc, vc)
    assert torch.equal(kc, k1)
    pos.fill_(0)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        rope_cache_append(qkv, cis, pos, kc, vc)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        rope_cache_append(qkv, cis, pos, kc, vc)
        pos.add_(1)
    kc.copy_(k0)
    pos.fill_(0)
    for _ in range(min(3, max_len)):
        graph.replay()
    torch.cuda.synchronize()
    want = rotate(qkv[:, 1])
    for r in range(min(3, max_len)):
        assert torch.equal(kc[:, :, r], want)
    assert_clean_device()
