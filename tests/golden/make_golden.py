"""Generate the golden vectors under tests/golden/ from the reference's own kernels.

Run once, where a checkout of the reference is available (it cannot travel with
this repository):

    python tests/golden/make_golden.py --reference /path/to/blockwise_int8_linear

The reference's three ``@triton.jit`` kernel bodies (``triton_functions.py:69-139``,
``382-406``, ``467-490``) are executed on CPU tensors by Triton's interpreter
(``TRITON_INTERPRET=1``).  Nothing of the reference is modified or copied; what is
needed to import it with a newer Triton is injected from here:

* stub modules for ``triton.ops.matmul_perf_model`` and ``torch_cublas_matmul_int8``
  (imported by the reference but not on the path);
* ``tl.math.llrint`` (gone from newer Triton) as numpy's round-half-even;
* ``torch.Any`` (an annotation in ``block_linear.py``; gone from newer torch) as ``typing.Any``;
* the autotuner is bypassed by calling the kernels' inner ``.fn`` with one fixed
  tile configuration (tile sizes do not change results with SPLIT_K=1).

The interpreter truncates fp32 -> bf16 on store instead of rounding, unlike a
GPU, so every kernel is run with fp32 outputs; bf16 results are the RNE cast of
these.  The autograd fixtures run the reference's ``blockwise_int8_linear``
(``block_linear.py:69-112``) unchanged, with its three functional ops bound to
the interpreter-backed wrappers below.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(path: str, block: int):
    ops = types.ModuleType("triton.ops")
    mpm = types.ModuleType("triton.ops.matmul_perf_model")
    mpm.early_config_prune = lambda configs, named_args, **kw: configs
    mpm.estimate_matmul_time = lambda **kw: 1.0
    ops.matmul_perf_model = mpm
    sys.modules["triton.ops"] = ops
    sys.modules["triton.ops.matmul_perf_model"] = mpm
    stub = types.ModuleType("torch_cublas_matmul_int8")
    stub.matmul_int8 = None
    sys.modules["torch_cublas_matmul_int8"] = stub
    sys.path.insert(0, path)
    for name in ("block_linear_config", "triton_functions", "block_linear"):
        sys.modules.pop(name, None)
    import block_linear_config

    block_linear_config.GROUP_SIZE = block          # BLOCK_K is frozen at import of triton_functions
    block_linear_config.INPUT_OUTPUT_TORCH_TYPE = torch.float32
    import triton_functions as tf

    from triton.runtime.interpreter import TensorHandle

    def _llrint(x):
        with np.errstate(invalid="ignore"):
            d = np.rint(x.handle.data).astype(np.int64)
        ty = tl.block_type(tl.int64, x.shape) if x.type.is_block() else tl.int64
        return tl.tensor(TensorHandle(d, tl.int64), ty)

    tl.math.llrint = _llrint
    return block_linear_config, tf


class Ref:
    """Interpreter-backed callers of the reference kernels for one block size."""

    def __init__(self, path: str, block: int):
        self.block = block
        self.cfg, self.tf = import_reference(path, block)

    def quantize(self, x):
        tf, B = self.tf, self.block
        m, k = x.shape
        out = torch.empty(m, k, dtype=torch.int8)
        st = torch.empty((tf.ceil_div(k, B), m), dtype=torch.float32)
        tf._quantize_block_rowwise.fn[(m,)](x, out, st, M=m, K=k, FBLOCK_SIZE=B, n_elements=out.numel())
        return out, st

    def dequantize(self, q, st):
        tf, B = self.tf, self.block
        m, k = q.shape
        out = torch.empty(m, k, dtype=torch.float32)
        tf._dequantize_block_rowwise.fn[(m,)](q, st, out, 1.0 / 127, K=k, M=m, FBLOCK_SIZE=B,
                                              n_elements=out.numel())
        return out

    def gemm(self, a, b, sx, sw, bias=None):
        tf, B = self.tf, self.block
        if a.stride(0) > 1 and a.stride(1) > 1:
            a = a.contiguous()
        if b.stride(0) > 1 and b.stride(1) > 1:
            b = b.contiguous()
        M, K = a.shape
        _, N = b.shape
        c = torch.empty(M, N, dtype=torch.float32)
        BM = BN = 16
        grid = (triton.cdiv(M, BM) * triton.cdiv(N, BN), 1)
        tf._int8_matmul_block64_rowwise_dequantize.fn[grid](
            a, b, c, bias, sx, sw, M, N, K, 1.0 / (127.0 * 127.0), 0 if bias is None else 1,
            a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1),
            GROUP_M=8, ACC_TYPE=tl.float32, BLOCK_M=BM, BLOCK_N=BN, BLOCK_K=B, SPLIT_K=1)
        return c


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).numpy().astype(np.uint16)


def op_case(ref: Ref, name: str, M: int, K: int, N: int, seed: int, *, zero_block=False,
            with_bias=False, outliers=False, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g) * scale
    w = torch.randn(N, K, generator=g) / scale
    if outliers:
        x = torch.where(torch.rand(M, K, generator=g) < 0.01, x * 20, x)
        w = torch.where(torch.rand(N, K, generator=g) < 0.01, w * 20, w)
    x = x.to(torch.bfloat16)
    w = w.to(torch.bfloat16)
    if zero_block:
        x[0, : ref.block] = 0
        w[1, -min(ref.block, K):] = 0
    bias = torch.randn(N, generator=g).to(torch.bfloat16) if with_bias else None
    xq, xs = ref.quantize(x)
    wq, ws = ref.quantize(w)
    xd = ref.dequantize(xq, xs)
    c = ref.gemm(xq, wq.t(), xs, ws, bias)
    out = {
        "block": np.int64(ref.block), "x_bf16": bf16_bits(x), "w_bf16": bf16_bits(w),
        "xq": xq.numpy(), "xs": xs.numpy(), "wq": wq.numpy(), "ws": ws.numpy(),
        "x_deq_f32": xd.numpy(), "c_f32": c.numpy(),
    }
    if bias is not None:
        out["bias_bf16"] = bf16_bits(bias)
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
    print("wrote", name, {k: getattr(v, "shape", v) for k, v in out.items()})


def autograd_case(ref: Ref, path: str, name: str, batch, K: int, N: int, seed: int, with_bias: bool):
    """forward + backward of the reference's autograd function, fp32 I/O
    (the configuration of its own smoke script, ``block_linear.py:173-175``)."""
    import typing

    if not hasattr(torch, "Any"):          # annotation used at block_linear.py:50,83; gone from newer torch
        torch.Any = typing.Any
    import block_linear as bl

    bl.quantize_block_rowwise = lambda x, fblock_size=None: ref.quantize(x)
    bl.int8_matmul_block64_rowwise_dequantize = lambda a, b, sx, sw, bias=None: ref.gemm(a, b, sx, sw, bias)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*batch, K, generator=g).requires_grad_(True)
    w = (torch.randn(N, K, generator=g) * 0.05).requires_grad_(True)
    b = torch.randn(N, generator=g).requires_grad_(True) if with_bias else None
    gy = torch.randn(*batch, N, generator=g)
    y = bl.blockwise_int8_linear.apply(x, w, b)
    y.backward(gy)
    out = {"block": np.int64(ref.block), "x": x.detach().numpy(), "w": w.detach().numpy(),
           "gy": gy.numpy(), "y": y.detach().numpy(), "gx": x.grad.numpy(), "gw": w.grad.numpy()}
    if with_bias:
        out["b"] = b.detach().numpy()
        out["gb"] = b.grad.numpy()
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
    print("wrote", name, {k: getattr(v, "shape", v) for k, v in out.items()})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    ap.add_argument("--block", type=int, default=0, help="generate only this block size (internal)")
    args = ap.parse_args()
    if args.block == 0:
        # BLOCK_K is frozen when the reference module is imported: one process per block size.
        import subprocess

        for b in (64, 32, 128):
            subprocess.check_call([sys.executable, os.path.abspath(__file__), "--reference", args.reference,
                                   "--block", str(b)])
        return
    ref = Ref(args.reference, args.block)
    B = args.block
    if B == 64:
        op_case(ref, "ops_b64_zero_block", 24, 192, 40, seed=0, zero_block=True)
        op_case(ref, "ops_b64_ktail_bias", 20, 150, 24, seed=1, with_bias=True)
        op_case(ref, "ops_b64_outliers", 48, 320, 72, seed=2, outliers=True, with_bias=True)
        op_case(ref, "ops_b64_odd_shapes", 129, 266, 75, seed=3, scale=5.0)     # triton_functions.py:584-586
        op_case(ref, "ops_b64_one_row", 1, 256, 48, seed=4)
        autograd_case(ref, args.reference, "autograd_b64", (2, 64), 128, 192, seed=10, with_bias=True)
        autograd_case(ref, args.reference, "autograd_b64_nobias", (128,), 128, 128, seed=11, with_bias=False)
    elif B == 32:
        op_case(ref, "ops_b32", 33, 160, 40, seed=5, with_bias=True, zero_block=True)
    elif B == 128:
        op_case(ref, "ops_b128", 40, 384, 56, seed=6, outliers=True)
        op_case(ref, "ops_b128_ktail", 17, 200, 24, seed=7, with_bias=True)
        autograd_case(ref, args.reference, "autograd_b128", (128,), 128, 128, seed=12, with_bias=False)


if __name__ == "__main__":
    main()
