"""The CPU restatements against the golden vectors produced by the reference's own kernels
(tests/golden/make_golden.py), and against each other.  No GPU needed."""
import pytest
import torch

from oracle import blockwise_int8_oracle as O
from oracle import c_oracle as C
from tests.helpers import golden_names, load_golden

OPS = golden_names("ops_")
AUTOGRAD = golden_names("autograd_")


def test_fixture_inventory():
    assert len(OPS) >= 8 and len(AUTOGRAD) >= 3


@pytest.mark.parametrize("name", OPS)
def test_quantize_matches_reference_kernels(name):
    g = load_golden(name)
    for src, q_ref, s_ref in ((g["x"], g["xq"], g["xs"]), (g["w"], g["wq"], g["ws"])):
        q, s = O.quantize(src, g["block"])
        assert torch.equal(q, q_ref)
        assert torch.equal(s, s_ref)
        qc, sc = C.quantize(src, g["block"])
        assert torch.equal(qc, q_ref)
        assert torch.equal(sc, s_ref)


@pytest.mark.parametrize("name", OPS)
def test_dequantize_matches_reference_kernels(name):
    g = load_golden(name)
    d = O.dequantize(g["xq"], g["xs"], g["block"], torch.float32)
    assert torch.equal(d, g["x_deq_f32"])
    assert torch.equal(C.dequantize(g["xq"], g["xs"], g["block"], torch.float32), g["x_deq_f32"])
    # bf16 output = RNE cast of the fp32 result
    assert torch.equal(O.dequantize(g["xq"], g["xs"], g["block"], torch.bfloat16), g["x_deq_f32"].to(torch.bfloat16))
    assert torch.equal(C.dequantize(g["xq"], g["xs"], g["block"], torch.bfloat16), g["x_deq_f32"].to(torch.bfloat16))


@pytest.mark.parametrize("name", OPS)
def test_gemm_matches_reference_kernels(name):
    g = load_golden(name)
    bias = g.get("bias")
    c = O.gemm(g["xq"], g["wq"].t(), g["xs"], g["ws"], bias, g["block"], torch.float32)
    assert torch.equal(c, g["c_f32"])
    acc = C.gemm_acc(g["xq"], g["wq"], g["xs"], g["ws"], g["block"])
    if bias is not None:
        acc = acc + bias.float()
    assert torch.equal(acc, g["c_f32"])


@pytest.mark.parametrize("name", OPS)
def test_partials_agree(name):
    g = load_golden(name)
    p = O.gemm_block_partials(g["xq"], g["wq"].t(), g["block"])
    assert torch.equal(p, C.gemm_partials(g["xq"], g["wq"], g["block"]))


@pytest.mark.parametrize("name", AUTOGRAD)
def test_autograd_matches_reference(name):
    g = load_golden(name)
    b = g.get("b")
    y = O.linear_forward(g["x"], g["w"], b, g["block"], torch.float32)
    assert torch.equal(y, g["y"])
    gx, gw, gb = O.linear_backward(g["x"], g["w"], g["gy"], g["block"], torch.float32, need_bias=b is not None)
    assert torch.equal(gx, g["gx"])
    assert torch.equal(gw, g["gw"])
    if b is not None:
        assert torch.equal(gb, g["gb"])


def test_config0_error_vs_fp32_product():
    """BASELINE config 0: 256x1024x1024, block 64, N(0,1) + 0.1% x20 outliers; the quantised
    product stays within 3 % (Frobenius) of the fp32 product."""
    x = O.synthetic((256, 1024), 1234)
    w = O.synthetic((1024, 1024), 1235)
    y = O.linear_forward(x, w, None, 64)
    ref = x.float() @ w.float().t()
    rel = ((y.float() - ref).norm() / ref.norm()).item()
    assert rel < 0.03, rel


def test_near_tie_inputs_use_ieee_division():
    """x/s chosen so that 127*x/s lies next to .5: a reciprocal-multiply would round differently."""
    block = 64
    s = torch.tensor(1.7265625)            # bf16-exact
    vals = torch.arange(-127, 128, dtype=torch.float32) + 0.5
    x = (vals / 127.0 * s).to(torch.bfloat16)[:block * 3].reshape(1, -1).clone()
    x[0, 0] = s
    x[0, block] = -s
    x[0, 2 * block] = s
    q, sc = O.quantize(x, block)
    qc, scc = C.quantize(x, block)
    assert torch.equal(q, qc) and torch.equal(sc, scc)
    assert q[0, 0].item() == 127 and q[0, block].item() == -127


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16, torch.float32])
def test_producer_step_restatements_equal_torch_cpu(dt):
    """The oracle's normalisation and gated activation (the steps the fused quantizers absorb) against torch's own CPU
    implementations of the same model code, bit for bit."""
    g = torch.Generator().manual_seed(31)
    x = (torch.randn((16, 704), generator=g) * 1.5).to(dt)
    u = torch.randn((16, 704), generator=g).to(dt)
    w = (1.0 + 0.1 * torch.randn(704, generator=g)).to(dt)
    if dt == torch.float32:
        # torch's fused CPU kernels use a vectorised exp and sum the squares in another order: the last bits of an fp32
        # result may differ; the 16-bit results absorb that in their rounding
        assert torch.allclose(O.silu_mul(x, u), torch.nn.functional.silu(x) * u, rtol=1e-6, atol=1e-7)
        assert torch.allclose(O.rmsnorm(x, 1e-5), torch.nn.functional.rms_norm(x, (704,), eps=1e-5), rtol=1e-6, atol=0)
    else:
        assert torch.equal(O.silu_mul(x, u), torch.nn.functional.silu(x) * u)
        assert torch.equal(O.rmsnorm(x, 1e-5), torch.nn.functional.rms_norm(x, (704,), eps=1e-5))
    q, s = O.rmsnorm_quantize(x, 64, 1e-5, w)
    q2, s2 = O.quantize(O.rmsnorm(x, 1e-5, w), 64)
    assert torch.equal(q, q2) and torch.equal(s, s2)
    q, s = O.silu_mul_quantize(x, u, 64)
    q2, s2 = O.quantize(O.silu_mul(x, u), 64)
    assert torch.equal(q, q2) and torch.equal(s, s2)
