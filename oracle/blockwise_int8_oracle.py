"""CPU restatement of the reference's blockwise-int8 linear path.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it.  The shipped path is
the CUDA library; nothing in the package imports this file.

What it restates (paths are inside the reference project):

* ``quantize``     follows ``triton_functions.py:382-406`` (kernel) and
  ``triton_functions.py:411-423`` (wrapper): per row, per block of ``B``
  contiguous elements, ``scale = max|x|`` in fp32; ``q = rint(127 * (x / scale))``
  with an fp32 divide followed by a separate fp32 multiply, round half to even,
  stored as int8; the K tail is treated as zeros; an all-zero block gives
  ``0/0 = NaN`` which the int8 store turns into 0; scales are stored transposed,
  ``[ceil(K/B), M]``.
* ``dequantize``   follows ``triton_functions.py:467-490`` / ``492-500``:
  ``out = (scale * q) * fl32(1/127)``, left to right in fp32, then cast.
* ``gemm``         follows ``triton_functions.py:69-139`` / ``142-168``: per K-block
  ``P = A_j . B_j`` exactly in int32, ``acc += sw * (sx * (float(P) * fl32(1/127^2)))``
  in fp32 with j ascending, cast to the output type, then ``+ bias`` in the
  output type.
* ``linear_forward`` / ``linear_backward`` follow ``block_linear.py:69-112``.

Pinning: the reference ships no tests or golden vectors.  The fixtures under
``tests/golden/`` were produced by executing the reference's own ``@triton.jit``
kernel bodies on CPU tensors with Triton's interpreter (script
``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks this
restatement against them bit for bit.  What stays unpinned is the behaviour of
the reference on a real GPU, whose fp32 ``/`` is Triton's approximate
``div.full.f32``: on a vanishing fraction of near-tie inputs it may differ by
one int8 step from any IEEE evaluation, in a compiler- and hardware-defined way.
"Bit-exact" therefore means bit-exact against this IEEE restatement.
"""
from __future__ import annotations

import torch

_F32 = torch.float32


def ceil_div(n: int, d: int) -> int:
    return -(n // -d)


def _pad_blocks(x: torch.Tensor, block: int) -> torch.Tensor:
    """Return x as fp32 [M, nb, block] with the K tail zero-filled
    (``triton_functions.py:398-401``: masked load, ``tl.where(mask, |x|, 0)``)."""
    m, k = x.shape
    nb = ceil_div(k, block)
    xf = x.to(_F32)
    if nb * block != k:
        xf = torch.nn.functional.pad(xf, (0, nb * block - k))
    return xf.reshape(m, nb, block)


def quantize(x: torch.Tensor, block: int):
    """``quantize_block_rowwise`` (``triton_functions.py:411-423``).

    Returns (q int8 [M, K], scales fp32 [ceil(K/block), M])."""
    assert x.dim() == 2
    m, k = x.shape
    xb = _pad_blocks(x, block)
    s = xb.abs().amax(dim=-1)                                   # fp32, exact
    y = xb / s.unsqueeze(-1)                                    # IEEE fp32 divide
    z = torch.round(y * torch.tensor(127.0, dtype=_F32))        # separate multiply, RNE
    z = torch.nan_to_num(z, nan=0.0)                            # 0/0 block -> 0
    q = z.to(torch.int8).reshape(m, -1)[:, :k].contiguous()
    return q, s.t().contiguous()


def rmsnorm(x: torch.Tensor, eps: float = 1e-5, weight: torch.Tensor = None) -> torch.Tensor:
    """The stored output of the normalisation that feeds a layer's q/k/v and gate/up projections:
    ``cast(x * rsqrt(mean(x^2) + eps) [* weight])``, fp32 arithmetic, one rounding to ``x.dtype``.  The reference has no
    such step of its own (its layers quantize whatever tensor they are given, ``block_linear.py:141``); this restates the
    model code around the layer.  The order of the sum of squares is torch's on CPU, so against a GPU kernel the last
    bit of ``rsqrt`` may differ: compare dequantized values, not bits."""
    xf = x.to(torch.float32)
    rstd = torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) / x.shape[-1] + eps)
    y = xf * rstd
    if weight is not None:
        y = y * weight.to(torch.float32)
    return y.to(x.dtype)


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``F.silu(gate) * up`` as two stored elementwise steps: ``cast(gate / (1 + exp(-gate)))``, then ``cast(. * up)``."""
    gf = gate.to(torch.float32)
    s = (gf / (1.0 + torch.exp(-gf))).to(gate.dtype)
    return (s.to(torch.float32) * up.to(torch.float32)).to(gate.dtype)


def rmsnorm_quantize(x: torch.Tensor, block: int, eps: float = 1e-5, weight: torch.Tensor = None):
    """``quantize(rmsnorm(x))``: what the fused normalise-and-quantize step must return."""
    return quantize(rmsnorm(x, eps, weight), block)


def silu_mul_quantize(gate: torch.Tensor, up: torch.Tensor, block: int):
    """``quantize(silu_mul(gate, up))``: what the fused activation-and-quantize step must return."""
    return quantize(silu_mul(gate, up), block)


def dequantize(q: torch.Tensor, scales: torch.Tensor, block: int,
               out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``dequantize_block_rowwise`` (``triton_functions.py:492-500``, kernel line 487)."""
    m, k = q.shape
    nb = ceil_div(k, block)
    qb = q.to(_F32)
    if nb * block != k:
        qb = torch.nn.functional.pad(qb, (0, nb * block - k))
    qb = qb.reshape(m, nb, block)
    inv127 = torch.tensor(1.0 / 127, dtype=_F32)
    out = (scales.t().to(_F32).unsqueeze(-1) * qb) * inv127
    return out.reshape(m, -1)[:, :k].to(out_dtype).contiguous()


def gemm_block_partials(a: torch.Tensor, b: torch.Tensor, block: int) -> torch.Tensor:
    """Exact int32 partial sums ``P[j] = a[:, jB:(j+1)B] @ b[jB:(j+1)B, :]``
    (``triton_functions.py:115``).  a is [M, K] int8, b is [K, N] int8."""
    m, k = a.shape
    n = b.shape[1]
    nb = ceil_div(k, block)
    out = torch.empty((nb, m, n), dtype=torch.int32)
    for j in range(nb):
        lo, hi = j * block, min((j + 1) * block, k)
        # |P| <= 127*127*block < 2**24 for block <= 1040: an fp32 matmul of the
        # integer-valued operands is exact and much faster than an integer one.
        if block <= 1024:
            p = a[:, lo:hi].to(_F32) @ b[lo:hi, :].to(_F32)
            out[j] = p.to(torch.int32)
        else:
            out[j] = (a[:, lo:hi].to(torch.int64) @ b[lo:hi, :].to(torch.int64)).to(torch.int32)
    return out


def gemm_acc(a, b, state_x, state_w, block: int) -> torch.Tensor:
    """The fp32 accumulator of the GEMM before the output cast
    (``triton_functions.py:107-124``), operation order as in line 120."""
    m, k = a.shape
    n = b.shape[1]
    nb = ceil_div(k, block)
    div = torch.tensor(1.0 / (127.0 * 127.0), dtype=_F32)
    acc = torch.zeros((m, n), dtype=_F32)
    for j in range(nb):
        lo, hi = j * block, min((j + 1) * block, k)
        p = a[:, lo:hi].to(_F32) @ b[lo:hi, :].to(_F32)
        acc += state_w[j].to(_F32)[None, :] * (state_x[j].to(_F32)[:, None] * (p * div))
    return acc


def gemm_term_abs_sum(a, b, state_x, state_w, block: int) -> torch.Tensor:
    """Sum over blocks of |term_j|: the magnitude the fp32 tolerance is scaled by."""
    m, k = a.shape
    n = b.shape[1]
    nb = ceil_div(k, block)
    div = torch.tensor(1.0 / (127.0 * 127.0), dtype=_F32)
    tot = torch.zeros((m, n), dtype=_F32)
    for j in range(nb):
        lo, hi = j * block, min((j + 1) * block, k)
        p = a[:, lo:hi].to(_F32) @ b[lo:hi, :].to(_F32)
        tot += (state_w[j].to(_F32)[None, :] * (state_x[j].to(_F32)[:, None] * (p * div))).abs()
    return tot


def gemm(a, b, state_x, state_w, bias=None, block: int = 64,
         out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``int8_matmul_block64_rowwise_dequantize`` (``triton_functions.py:142-168``)."""
    assert a.shape[1] == b.shape[0], "incompatible dimensions"
    c = gemm_acc(a, b, state_x, state_w, block).to(out_dtype)
    if bias is not None:
        c = c + bias.to(out_dtype)[None, :]                      # line 127-131: add in output type
    return c


def linear_forward(x3d, w, bias, block: int, out_dtype=torch.bfloat16):
    """``blockwise_int8_linear.forward`` (``block_linear.py:71-80``)."""
    x = x3d.reshape(-1, x3d.shape[-1])
    xq, sx = quantize(x, block)
    wq, sw = quantize(w, block)
    y = gemm(xq, wq.t(), sx, sw, bias, block, out_dtype)
    return y.reshape(*x3d.shape[:-1], -1)


def linear_backward(x3d, w, g3d, block: int, out_dtype=torch.bfloat16, need_bias=True):
    """``blockwise_int8_linear.backward`` (``block_linear.py:83-112``).

    Returns (grad_x, grad_w, grad_bias)."""
    x = x3d.reshape(-1, x3d.shape[-1])
    g = g3d.reshape(-1, g3d.shape[-1])
    # dX: contraction over N, both operands blocked along N (lines 92-95)
    gq, gs = quantize(g, block)
    wtq, wts = quantize(w.t().contiguous(), block)
    gx = gemm(gq, wtq.t(), gs, wts, None, block, out_dtype).reshape(*g3d.shape[:-1], -1)
    # dW: contraction over the token dimension (lines 100-104)
    xtq, xts = quantize(x.t().contiguous(), block)
    gtq, gts = quantize(g.t().contiguous(), block)
    gw = gemm(gtq, xtq.t(), gts, xts, None, block, out_dtype)
    gb = g.sum(dim=0) if need_bias else None                     # line 110
    return gx, gw, gb


def synthetic(shape, seed: int, std: float = 1.0, outlier_frac: float = 0.001,
              outlier_mul: float = 20.0, dtype=torch.bfloat16) -> torch.Tensor:
    """Seeded synthetic tensor: N(0, std) with a fraction of entries multiplied by
    ``outlier_mul``.  Generated on CPU so every consumer sees the same bits."""
    g = torch.Generator().manual_seed(seed)
    t = torch.randn(shape, generator=g) * std
    if outlier_frac > 0:
        mask = torch.rand(shape, generator=g) < outlier_frac
        t = torch.where(mask, t * outlier_mul, t)
    return t.to(dtype)
