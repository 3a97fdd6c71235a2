"""The module layer on the GPU: autograd function, BlockInt8Linear, replace_linear_with_blockwise_int8."""
import pytest
import torch
import torch.nn as nn

from oracle import blockwise_int8_oracle as O
from tests.gpu_util import DEV, assert_clean_device, bf16_ulp_distance, set_config
from tests.helpers import golden_names, load_golden

pytestmark = pytest.mark.gpu


def _assert_bf16_close(got, ref, identical=0.99):
    """bf16 results of the layer against the oracle's: at least 99 % bit-identical, and no element further away than one
    bf16 step at the magnitude of the largest output (the error of an element is set by the size of its terms, not of
    their sum; the per-term bound is tested on the GEMM itself)."""
    d = bf16_ulp_distance(got, ref)
    same = (d == 0).float().mean().item()
    assert same >= identical, f"only {same:.4f} identical"
    err = (got.float() - ref.float()).abs().max().item()
    assert err <= 2.0 ** -7 * ref.float().abs().max().item(), err


def _close_fp32(got, ref, rel=2e-5):
    scale = ref.abs().max().item() + 1e-30
    assert (got.cpu() - ref).abs().max().item() <= rel * scale, (got.cpu() - ref).abs().max().item() / scale


@pytest.mark.parametrize("name", golden_names("autograd_"))
def test_autograd_against_reference_run(name):
    """fp32 I/O (the configuration of the reference's own smoke script): forward, dX, dW, dbias against the values
    produced by the reference's autograd function."""
    from block_linear import blockwise_int8_linear
    g = load_golden(name)
    set_config(g["block"], torch.float32)
    x = g["x"].to(DEV).requires_grad_(True)
    w = g["w"].to(DEV).requires_grad_(True)
    b = g["b"].to(DEV).requires_grad_(True) if "b" in g else None
    y = blockwise_int8_linear.apply(x, w, b)
    y.backward(g["gy"].to(DEV))
    _close_fp32(y.detach(), g["y"])
    _close_fp32(x.grad, g["gx"])
    _close_fp32(w.grad, g["gw"])
    if b is not None:
        assert torch.allclose(b.grad.cpu(), g["gb"], rtol=1e-5, atol=1e-5)
    assert_clean_device()
    set_config(64)


def test_training_step_bf16_vs_oracle():
    from block_linear import BlockInt8Linear
    set_config(64, torch.bfloat16)
    torch.manual_seed(0)
    lin = BlockInt8Linear(256, 384, bias=True, device=DEV, dtype=torch.bfloat16)
    x = O.synthetic((4, 96, 256), 41).to(DEV).requires_grad_(True)
    gy = O.synthetic((4, 96, 384), 42, outlier_frac=0).to(DEV)
    lin.train()
    y = lin(x)
    y.backward(gy)
    w, b = lin.weight.detach().cpu(), lin.bias.detach().cpu()
    y_ref = O.linear_forward(x.detach().cpu(), w, b, 64)
    gx_ref, gw_ref, gb_ref = O.linear_backward(x.detach().cpu(), w, gy.cpu(), 64)
    for got, ref in ((y.detach(), y_ref), (x.grad, gx_ref), (lin.weight.grad, gw_ref)):
        _assert_bf16_close(got.cpu().reshape(ref.shape), ref)
    assert torch.allclose(lin.bias.grad.float().cpu(), gb_ref.float(), rtol=2e-2, atol=2e-2)
    assert_clean_device()


def test_eval_path_and_state_dict():
    from block_linear import BlockInt8Linear
    set_config(64, torch.bfloat16)
    torch.manual_seed(1)
    lin = BlockInt8Linear(512, 320, bias=True, device=DEV, dtype=torch.bfloat16).eval()
    x = O.synthetic((3, 40, 512), 43).to(DEV)
    with torch.no_grad():
        y = lin(x)
    assert tuple(y.shape) == (3, 40, 320) and y.dtype == torch.bfloat16
    y_ref = O.linear_forward(x.cpu(), lin.weight.detach().cpu(), lin.bias.detach().cpu(), 64)
    _assert_bf16_close(y.cpu(), y_ref)
    sd = lin.state_dict()
    assert sd["W_int8"].dtype == torch.int8 and tuple(sd["W_int8"].shape) == (320, 512)
    assert sd["state_W"].dtype == torch.float32 and tuple(sd["state_W"].shape) == (8, 320)
    wq_ref, ws_ref = O.quantize(lin.weight.detach().cpu(), 64)
    assert torch.equal(sd["W_int8"].cpu(), wq_ref) and torch.equal(sd["state_W"].cpu(), ws_ref)
    fresh = BlockInt8Linear(512, 320, bias=True, device=DEV, dtype=torch.bfloat16).eval()
    fresh.load_state_dict(sd)
    with torch.no_grad():
        assert torch.equal(fresh(x), y)


def test_replace_linear_in_model():
    from block_linear import BlockInt8Linear, replace_linear_with_blockwise_int8
    set_config(64, torch.bfloat16)

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.up = nn.Linear(128, 256)
            self.act = nn.GELU()
            self.down = nn.Linear(256, 128, bias=False)
            self.inner = nn.Sequential(nn.Linear(128, 128))

        def forward(self, x):
            return self.inner(self.down(self.act(self.up(x))))

    torch.manual_seed(2)
    m = MLP().to(DEV).to(torch.bfloat16)
    w_up = m.up.weight
    replace_linear_with_blockwise_int8(m)
    assert isinstance(m.up, BlockInt8Linear) and isinstance(m.down, BlockInt8Linear)
    assert not isinstance(m.inner[0], BlockInt8Linear)            # direct children only, like the reference
    assert m.up.weight.data_ptr() == w_up.data_ptr()              # storage shared
    m.apply(replace_linear_with_blockwise_int8)
    assert isinstance(m.inner[0], BlockInt8Linear)
    x = torch.randn(8, 128, device=DEV, dtype=torch.bfloat16)
    ref = (x.float() @ m.up.weight.float().t() + m.up.bias.float())
    m.train()
    out = m.up(x)
    assert ((out.float() - ref).norm() / ref.norm()).item() < 0.05
    loss = m(x).float().pow(2).mean()
    loss.backward()
    assert m.up.weight.grad is not None and torch.isfinite(m.up.weight.grad.float()).all()
    m.eval()
    with torch.no_grad():
        y = m(x)
    assert torch.isfinite(y.float()).all()
    assert_clean_device()


def test_config0_single_forward():
    """BASELINE config: x [256,1024], W [1024,1024] bf16 with outliers, block 64; checked against the fp32 product."""
    from block_linear import BlockInt8Linear
    set_config(64, torch.bfloat16)
    x = O.synthetic((256, 1024), 1234)
    w = O.synthetic((1024, 1024), 1235)
    lin = BlockInt8Linear(1024, 1024, bias=False, device=DEV, dtype=torch.bfloat16).eval()
    lin.weight.data.copy_(w.to(DEV))
    with torch.no_grad():
        y = lin(x.to(DEV))
    ref = x.float() @ w.float().t()
    rel = ((y.float().cpu() - ref).norm() / ref.norm()).item()
    assert rel < 0.03, rel
    _assert_bf16_close(y.cpu(), O.linear_forward(x, w, None, 64))


def test_fast_matmul_helpers():
    from block_linear import fast_matmul
    from triton_functions import fast_matmulT
    set_config(64, torch.bfloat16)
    a = O.synthetic((64, 256), 51)
    b = O.synthetic((128, 256), 52)
    ref = O.linear_forward(a, b, None, 64)
    _assert_bf16_close(fast_matmulT(a.to(DEV), b.to(DEV)).cpu(), ref)
    _assert_bf16_close(fast_matmul(a.to(DEV), b.t().contiguous().to(DEV)).cpu(), ref)


def test_int8_resident_weight_and_state_dict_round_trip():
    """prepare_for_eval(drop_weight=True): inference runs from the int8 buffers alone, and the state dict written
    afterwards (empty `weight`, `W_int8`, `state_W`) loads into a fresh module that gives the same outputs."""
    import io
    from block_linear import BlockInt8Linear
    set_config(64, torch.bfloat16)
    torch.manual_seed(3)
    lin = BlockInt8Linear(512, 320, bias=True, device=DEV, dtype=torch.bfloat16).eval()
    x = O.synthetic((130, 512), 44).to(DEV)
    with torch.no_grad():
        y = lin(x)
    full_bytes = lin.weight.numel() * 2
    lin.prepare_for_eval(drop_weight=True)
    assert lin.weight.numel() == 0 and full_bytes == 512 * 320 * 2
    with torch.no_grad():
        assert torch.equal(lin(x), y)
    buf = io.BytesIO()
    torch.save(lin.state_dict(), buf)
    buf.seek(0)
    sd = torch.load(buf)
    assert set(sd) == {"weight", "bias", "W_int8", "state_W"} and sd["weight"].numel() == 0
    fresh = BlockInt8Linear(512, 320, bias=True, device=DEV, dtype=torch.bfloat16).eval()
    fresh.load_state_dict(sd)
    assert fresh.weight.numel() == 0
    with torch.no_grad():
        assert torch.equal(fresh(x), y)
    fresh.train()
    with pytest.raises(RuntimeError):
        fresh(x)
    # the knob does the same on the first eval forward
    import block_linear_config as cfg
    cfg.DROP_WEIGHT_IN_EVAL = True
    try:
        torch.manual_seed(3)
        lazy = BlockInt8Linear(512, 320, bias=True, device=DEV, dtype=torch.bfloat16).eval()
        with torch.no_grad():
            assert torch.equal(lazy(x), y)
        assert lazy.weight.numel() == 0
    finally:
        cfg.DROP_WEIGHT_IN_EVAL = False


def test_cached_quantized_weights_in_training():
    """CACHE_QUANTIZED_WEIGHTS: micro-steps between weight updates reuse both int8 copies of the weight; results are
    bit-identical to the uncached path, and an in-place update of the weight invalidates the copies."""
    import block_linear_config as cfg
    from block_linear import BlockInt8Linear
    set_config(64, torch.bfloat16)
    torch.manual_seed(4)
    lin = BlockInt8Linear(256, 192, bias=True, device=DEV, dtype=torch.bfloat16).train()
    xs = [O.synthetic((96, 256), 50 + i).to(DEV) for i in range(3)]
    gys = [O.synthetic((96, 192), 60 + i, outlier_frac=0).to(DEV) for i in range(3)]

    def micro_steps():
        outs = []
        for x, gy in zip(xs, gys):
            x = x.clone().requires_grad_(True)
            lin.weight.grad = None
            y = lin(x)
            y.backward(gy)
            outs.append((y.detach().clone(), x.grad.clone(), lin.weight.grad.clone()))
        return outs

    ref = micro_steps()
    cfg.CACHE_QUANTIZED_WEIGHTS = True
    try:
        got = micro_steps()
        cache = lin.weight._bi8_quantized
        assert "row" in cache and "col" in cache
        for a, b in zip(ref, got):
            assert all(torch.equal(u, v) for u, v in zip(a, b))
        with torch.no_grad():
            lin.weight.mul_(1.5)                      # what an optimizer step does: an in-place update
        got2 = micro_steps()
        assert lin.weight._bi8_quantized is not cache
        cfg.CACHE_QUANTIZED_WEIGHTS = False
        ref2 = micro_steps()
        for a, b in zip(ref2, got2):
            assert all(torch.equal(u, v) for u, v in zip(a, b))
        assert not torch.equal(ref[0][0], ref2[0][0])
    finally:
        cfg.CACHE_QUANTIZED_WEIGHTS = False
    assert_clean_device()


@pytest.mark.parametrize("shape", [(4, 96, 256, 384), (1, 130, 200, 72)])
def test_fused_dual_quantize_changes_no_result(shape):
    """X and G read once for both of their quantizations (the default) against the separate quantizers: y, dX, dW and db
    must be bit-identical, with a frozen weight and with a frozen input as well, for shapes the one-pass kernel takes and
    for shapes that fall back to the two single kernels."""
    import block_linear_config as cfg
    from block_linear import BlockInt8Linear
    b, t, k, n = shape
    set_config(64, torch.bfloat16)
    lin = BlockInt8Linear(k, n, bias=True, device=DEV, dtype=torch.bfloat16)
    g = torch.Generator(device=DEV).manual_seed(3)
    go = torch.randn((b, t, n), device=DEV, generator=g).to(torch.bfloat16)
    results = {}
    try:
        for fused in (True, False):
            cfg.FUSE_DUAL_QUANTIZE = fused
            for x_grad, w_grad in ((True, True), (False, True), (True, False)):
                x = torch.randn((b, t, k), device=DEV, generator=torch.Generator(device=DEV).manual_seed(5)).to(torch.bfloat16)
                x.requires_grad_(x_grad)
                lin.weight.requires_grad_(w_grad)
                lin.weight.grad = lin.bias.grad = None
                y = lin(x)
                y.backward(go)
                results[(fused, x_grad, w_grad)] = (y.detach().clone(), None if x.grad is None else x.grad.clone(),
                                                    None if lin.weight.grad is None else lin.weight.grad.clone(),
                                                    lin.bias.grad.clone())
    finally:
        cfg.FUSE_DUAL_QUANTIZE = True
        lin.weight.requires_grad_(True)
    for x_grad, w_grad in ((True, True), (False, True), (True, False)):
        for a, c in zip(results[(True, x_grad, w_grad)], results[(False, x_grad, w_grad)]):
            assert (a is None) == (c is None)
            if a is not None:
                assert torch.equal(a, c)
    assert_clean_device()
