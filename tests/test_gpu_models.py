"""The model drivers in examples/ at toy size on the GPU, every linear layer checked against the CPU oracle.

* Llama-architecture inference driver (2 layers, d = 256, 4 heads, FFN 704 = 11 blocks of 64, vocab 512): the same
  network is evaluated twice, once with the library's layers and once with every linear layer replaced by the oracle
  (CPU restatement of the reference) on the same quantized weights; logits must agree within the bf16 tolerance of the
  layer tests, relaxed for the depth of the network (a one-step difference of a hidden activation propagates).
* GPT-2-architecture training driver (2 layers, d = 128): one forward/backward; for every replaced linear layer the output,
  the input gradient and the weight gradient are compared with the oracle evaluated on that layer's own inputs.
"""
import argparse
import importlib.util
import os

import pytest
import torch

from oracle import blockwise_int8_oracle as O
from tests.gpu_util import DEV, assert_clean_device, bf16_ulp_distance, set_config

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "examples", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _close(got, ref, identical, rel):
    same = (bf16_ulp_distance(got, ref) == 0).float().mean().item()
    err = (got.float() - ref.float()).abs().max().item()
    assert same >= identical, f"only {same:.4f} identical"
    assert err <= rel * ref.float().abs().max().item(), err


def _toy_llama_args():
    return argparse.Namespace(layers=2, hidden=256, heads=4, head_dim=64, ffn=704, vocab=512, batch=2, prompt=24, decode=6, block=64)


def test_llama_driver_logits_against_oracle_linears():
    import block_linear_config as cfg
    L = _load("llama_infer")
    set_config(64, torch.bfloat16)
    a = _toy_llama_args()
    dev = torch.device(DEV)
    model = L.Llama(a, dev, rank=0, world=1)
    ids = torch.randint(0, a.vocab, (a.batch, a.prompt), generator=torch.Generator().manual_seed(4000)).to(dev)
    max_len = a.prompt + a.decode
    logits = model(ids, 0, max_len)
    assert tuple(logits.shape) == (a.batch, 1, a.vocab)

    # the same network with every linear layer evaluated by the oracle on the same int8 weights
    linears = [m for m in model.modules() if isinstance(m, L.Int8Linear)]
    assert len(linears) == 4 * a.layers + 1
    saved = []
    for m in linears:
        lin = m.lin
        saved.append((lin, lin.infer))

        def oracle_infer(x, lin=lin):
            X = x.reshape(-1, x.size(-1)).cpu()
            xq, xs = O.quantize(X, a.block)
            y = O.gemm(xq, lin.W_int8.cpu().t(), xs, lin.state_W.cpu(), None, a.block, cfg.INPUT_OUTPUT_TORCH_TYPE)
            return y.to(x.device).view(*x.size()[:-1], -1)

        def oracle_infer_pre(x, op="none", x2=None, norm_weight=None, eps=1e-5, residual=None, infer=oracle_infer):
            # the fused producer steps and the residual sum, restated on the CPU around the oracle's layer
            if op == "rmsnorm":
                inp = O.rmsnorm(x.cpu(), eps, None if norm_weight is None else norm_weight.cpu()).to(x.device)
            elif op == "silu_mul":
                inp = O.silu_mul(x.cpu(), x2.cpu()).to(x.device)
            else:
                inp = x
            y = infer(inp)
            return y if residual is None else residual + y

        lin.infer = oracle_infer
        lin.infer_pre = oracle_infer_pre
    for layer in model.layers:
        layer.kcache = layer.vcache = None
    ref = model(ids, 0, max_len)
    for lin, fn in saved:
        lin.infer = fn
        del lin.infer_pre                      # the instance attribute set above; the class's method shows again
    _close(logits.cpu(), ref.cpu(), identical=0.90, rel=2.0 ** -6)
    assert_clean_device()


def test_llama_driver_graph_decode_equals_eager_decode():
    """The decode step captured in a CUDA graph produces the tokens of the eager step (same kernels, same order)."""
    L = _load("llama_infer")
    set_config(64, torch.bfloat16)
    a = _toy_llama_args()
    r1 = L.run(a, rank=0, world=1, dev=torch.device(DEV), eager=False)
    r2 = L.run(a, rank=0, world=1, dev=torch.device(DEV), eager=True)
    assert r1["tokens"] == r2["tokens"]
    assert len(r1["tokens"][0]) == a.decode
    assert_clean_device()


def test_gpt2_driver_training_step_against_oracle():
    from block_linear import BlockInt8Linear, replace_linear_with_blockwise_int8
    G = _load("gpt2_train")
    set_config(64, torch.bfloat16)
    torch.manual_seed(0)
    model = G.GPT2(layers=2, d=128, heads=4, vocab=520, seq=64).to(DEV).to(torch.bfloat16)
    model.apply(replace_linear_with_blockwise_int8)
    model.train()
    layers = {n: m for n, m in model.named_modules() if isinstance(m, BlockInt8Linear)}
    assert len(layers) == 2 * 4 + 1
    seen = {}

    def fwd_hook(name):
        def hook(mod, inp, out):
            seen[name] = {"x": inp[0].detach().cpu(), "y": out.detach().cpu()}
            out.register_hook(lambda g, name=name: seen[name].__setitem__("gy", g.detach().cpu()))
            if inp[0].requires_grad:
                inp[0].register_hook(lambda g, name=name: seen[name].__setitem__("gx", g.detach().cpu()))
        return hook

    for n, m in layers.items():
        m.register_forward_hook(fwd_hook(n))
    ids = torch.randint(0, 520, (2, 65), generator=torch.Generator().manual_seed(5000)).to(DEV)
    logits = model(ids[:, :-1])
    loss = torch.nn.functional.cross_entropy(logits.float().view(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))
    loss.backward()
    assert torch.isfinite(loss)
    for n, m in layers.items():
        rec = seen[n]
        w = m.weight.detach().cpu()
        b = None if m.bias is None else m.bias.detach().cpu()
        y_ref = O.linear_forward(rec["x"], w, b, 64)
        _close(rec["y"].reshape(y_ref.shape), y_ref, identical=0.99, rel=2.0 ** -7)
        gx_ref, gw_ref, _ = O.linear_backward(rec["x"], w, rec["gy"], 64, need_bias=False)
        # every linear layer's input has no other consumer in this model, so the hook sees exactly the layer's dX
        if "gx" in rec:
            _close(rec["gx"].reshape(gx_ref.shape), gx_ref, identical=0.99, rel=2.0 ** -7)
        _close(m.weight.grad.cpu().reshape(gw_ref.shape), gw_ref, identical=0.99, rel=2.0 ** -7)
    assert_clean_device()


def test_hf_llama_with_every_linear_replaced_against_oracle():
    """An unmodified transformers LlamaForCausalLM (toy size, random weights) after
    model.apply(replace_linear_with_blockwise_int8): all 7 x layers + 1 nn.Linear modules become BlockInt8Linear, the model's
    own forward and generate run on them, and the logits agree with the same model whose linear layers are evaluated by the
    CPU oracle on the same int8 weights; the int8 model stays close to the bf16 model it was made from."""
    import block_linear_config as cfg
    from block_linear import BlockInt8Linear
    H = _load("hf_llama_infer")
    set_config(64, torch.bfloat16)
    a = argparse.Namespace(layers=2, hidden=256, heads=4, ffn=704, vocab=512, batch=2, prompt=24, decode=6, block=64, skip_dense=False)
    dev = torch.device(DEV)
    dense = H.build(a, dev)
    ids = torch.randint(0, a.vocab, (a.batch, a.prompt), generator=torch.Generator().manual_seed(4000)).to(dev)
    with torch.no_grad():
        dense_logits = dense(ids).logits
    res, model = H.run(a, dev)                                   # same seed: the same weights, swapped and quantized
    assert res["int8"]["linear_layers_replaced"] == 7 * a.layers + 1
    assert len(res["int8"]["first_tokens"]) == a.decode and len(res["bf16_dense"]["first_tokens"]) == a.decode
    assert not any(type(m) is torch.nn.Linear for m in model.modules())
    with torch.no_grad():
        logits = model(ids).logits
    # close to the bf16 model: per-layer int8 noise of about 1 % over two layers
    assert (logits.float() - dense_logits.float()).abs().max().item() <= 0.1 * dense_logits.float().abs().max().item()
    linears = [m for m in model.modules() if isinstance(m, BlockInt8Linear)]
    for lin in linears:
        def oracle_infer(x, lin=lin):
            X = x.reshape(-1, x.size(-1)).cpu()
            xq, xs = O.quantize(X, a.block)
            y = O.gemm(xq, lin.W_int8.cpu().t(), xs, lin.state_W.cpu(), None, a.block, cfg.INPUT_OUTPUT_TORCH_TYPE)
            return y.to(x.device).view(*x.size()[:-1], -1)
        lin.infer = oracle_infer
    with torch.no_grad():
        ref = model(ids).logits
    for lin in linears:
        del lin.infer
    _close(logits.cpu(), ref.cpu(), identical=0.90, rel=2.0 ** -6)
    assert_clean_device()
