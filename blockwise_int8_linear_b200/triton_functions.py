"""Functional operations of the blockwise-int8 linear layer.

Same names, signatures, return values and layouts as the reference's ``triton_functions.py``
(``quantize_block_rowwise`` 411-423, ``dequantize_block_rowwise`` 492-500,
``int8_matmul_block64_rowwise_dequantize`` 142-168, ``fast_matmulT`` 511-514); the module keeps
the reference's name although nothing here uses Triton: every function validates its arguments,
allocates its outputs with torch and calls one entry point of ``libbi8.so`` on the current CUDA
stream.  There is no CPU path and no fallback.

Layouts: quantized tensors are int8 ``[rows, K]``; block scales ("state") are float32
``[ceil(K/block), rows]``.  ``block`` is ``block_linear_config.GROUP_SIZE`` read at call time
unless ``fblock_size`` is given.
"""
from __future__ import annotations

import torch

from . import _lib
from . import block_linear_config

__all__ = [
    "ceil_div", "quantize_block_rowwise", "quantize_block_colwise", "quantize_block_dual", "dequantize_block_rowwise",
    "int8_matmul_block64_rowwise_dequantize", "quantize_matmul_block_rowwise_dequantize", "int8_matmul_block_partials",
    "fast_matmulT", "rmsnorm_quantize_block_rowwise", "silu_mul_quantize_block_rowwise", "pre_quantize_matmul_block_rowwise_dequantize",
]


def ceil_div(n, d):
    return -(n // -d)


def _block(fblock_size=None) -> int:
    b = int(fblock_size or block_linear_config.GROUP_SIZE)
    if b < 1:
        raise ValueError(f"block size must be positive, got {b}")
    return b


def _scale_dtype():
    if block_linear_config.SHARED_EXP_TORCH_TYPE != torch.float32:
        raise ValueError("block scales are float32 only (block_linear_config.SHARED_EXP_TORCH_TYPE)")
    return torch.float32


def _rows_contiguous(t: torch.Tensor) -> torch.Tensor:
    """2-D tensor whose last dimension is contiguous and whose row pitch covers a row."""
    if t.shape[1] != 1 and t.stride(1) != 1:
        return t.contiguous()
    if t.shape[0] > 1 and t.stride(0) < t.shape[1]:
        return t.contiguous()
    return t


def _pitch(t: torch.Tensor) -> int:
    return t.stride(0) if t.shape[0] > 1 else max(t.shape[1], 1)


def _pad16(x: torch.Tensor, block: int, rows: bool, cols: bool):
    """Zero-padded copy of a large 16-bit ``x [R, C]`` whose row or column count is not a multiple of 16 (GPT-2's 50257-wide
    logits and their gradient), or None when no padding is called for.

    The fast quantizers and the tensor-core GEMM want 16-byte aligned rows; the kernels for unaligned rows move two bytes
    per lane and run 5-8 x slower than one extra copy plus the fast kernel.  Padding with zeros changes no result: the
    pad stays inside the last block (block sizes here are multiples of 16), and zeros change neither a block's absmax nor
    the quantized values of its other elements."""
    r, c = x.shape
    if x.dtype not in (torch.bfloat16, torch.float16) or block % 16 != 0 or r * c < (1 << 22):
        return None
    rp = -(-r // 16) * 16 if rows else r
    cp = -(-c // 16) * 16 if cols else c
    if (rp, cp) == (r, c) or min(r, c) < 256:
        return None
    buf = torch.zeros((rp, cp), device=x.device, dtype=x.dtype) if rp != r else torch.empty((rp, cp), device=x.device, dtype=x.dtype)
    if rp == r:
        buf[:, c:].zero_()
    buf[:r, :c].copy_(x)
    return buf


class _on_device:
    """Makes the tensor's device current for the duration of a library call (no-op when it already is)."""

    def __init__(self, t: torch.Tensor):
        self.idx = t.device.index
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if self.idx is not None and self.idx != cur:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


def quantize_block_rowwise(x: torch.Tensor, fblock_size=None):
    """Quantize each row of ``x [M, K]`` in blocks of ``block`` elements (``triton_functions.py:411-423``).

    Returns ``(q, state)``: ``q`` int8 ``[M, K]``; ``state`` float32 ``[ceil(K/block), M]`` holding
    ``max|x|`` of each block.  ``q = rint(127 * (x / state))`` (fp32 divide, fp32 multiply, round half to
    even); an all-zero block gives state 0 and q 0.  For a large 16-bit ``x`` whose ``K`` is not a multiple of 16 the
    returned ``q`` is a view of a zero-padded buffer (row pitch rounded up to 16; same values), which the GEMM takes
    without a copy; call ``.contiguous()`` where a dense tensor is needed."""
    block = _block(fblock_size)
    m, k = x.shape
    assert x.is_cuda
    padded = _pad16(x, block, rows=False, cols=True) if x.dim() == 2 else None
    if padded is not None:
        # the result is a view with a 16-byte aligned row pitch, which the GEMM takes as it is
        q, state = quantize_block_rowwise(padded, block)
        return q[:, :k], state
    x = _rows_contiguous(x)
    code = _lib.dtype_code(x.dtype)
    output = torch.empty((m, k), device=x.device, dtype=torch.int8)
    output_maxs = torch.empty((ceil_div(k, block), m), device=x.device, dtype=_scale_dtype())
    with _on_device(x):
        rc = _lib.lib().bi8_quantize_rowwise(_lib.ptr(x), code, _pitch(x), _lib.ptr(output), _lib.ptr(output_maxs), m, k,
                                             block, _lib.stream_ptr())
    _lib.check(rc, "bi8_quantize_rowwise")
    return output, output_maxs


def quantize_block_colwise(x: torch.Tensor, fblock_size=None):
    """``quantize_block_rowwise(x.t().contiguous())`` without materialising the transpose
    (the pattern at ``block_linear.py:93-94`` and ``100-103``).  ``x`` is ``[R, C]``; returns int8 ``[C, R]``
    and state ``[ceil(R/block), C]``, bit-identical to the two-step form."""
    block = _block(fblock_size)
    r, c = x.shape
    assert x.is_cuda
    padded = _pad16(x, block, rows=True, cols=True) if x.dim() == 2 else None
    if padded is not None:
        q, state = quantize_block_colwise(padded, block)
        return q[:c, :r], state[:, :c]
    x = _rows_contiguous(x)
    code = _lib.dtype_code(x.dtype)
    output = torch.empty((c, r), device=x.device, dtype=torch.int8)
    output_maxs = torch.empty((ceil_div(r, block), c), device=x.device, dtype=_scale_dtype())
    with _on_device(x):
        rc = _lib.lib().bi8_quantize_colwise(_lib.ptr(x), code, _pitch(x), _lib.ptr(output), _lib.ptr(output_maxs), r, c,
                                             block, _lib.stream_ptr())
    _lib.check(rc, "bi8_quantize_colwise")
    return output, output_maxs


def quantize_block_dual(x: torch.Tensor, fblock_size=None):
    """``quantize_block_rowwise(x)`` and ``quantize_block_colwise(x)`` from one read of ``x`` ``[R, C]``: returns
    ``(q_row [R, C], state_row [ceil(C/block), R], q_col [C, R], state_col [ceil(R/block), C])``, each bit-identical to its
    single-purpose function.  The layer needs both for its input (forward GEMM and weight gradient,
    ``block_linear.py:78, 100-101``) and for the output gradient (``block_linear.py:92, 102-103``)."""
    block = _block(fblock_size)
    r, c = x.shape
    assert x.is_cuda
    padded = _pad16(x, block, rows=True, cols=True) if x.dim() == 2 else None
    if padded is not None:
        q_row, s_row, q_col, s_col = quantize_block_dual(padded, block)
        return q_row[:r, :c], s_row[:, :r], q_col[:c, :r], s_col[:, :c]
    x = _rows_contiguous(x)
    code = _lib.dtype_code(x.dtype)
    q_row = torch.empty((r, c), device=x.device, dtype=torch.int8)
    s_row = torch.empty((ceil_div(c, block), r), device=x.device, dtype=_scale_dtype())
    q_col = torch.empty((c, r), device=x.device, dtype=torch.int8)
    s_col = torch.empty((ceil_div(r, block), c), device=x.device, dtype=_scale_dtype())
    with _on_device(x):
        rc = _lib.lib().bi8_quantize_dual(_lib.ptr(x), code, _pitch(x), _lib.ptr(q_row), _lib.ptr(s_row), _lib.ptr(q_col),
                                          _lib.ptr(s_col), r, c, block, _lib.stream_ptr())
    _lib.check(rc, "bi8_quantize_dual")
    return q_row, s_row, q_col, s_col


def dequantize_block_rowwise(x: torch.Tensor, state_x: torch.Tensor, fblock_size=None):
    """``(state * q) * (1/127)`` cast to ``INPUT_OUTPUT_TORCH_TYPE`` (``triton_functions.py:492-500``)."""
    block = _block(fblock_size)
    m, k = x.shape
    assert x.is_cuda
    if x.dtype != torch.int8:
        raise ValueError(f"expected an int8 tensor, got {x.dtype}")
    if tuple(state_x.shape) != (ceil_div(k, block), m) or state_x.dtype != torch.float32:
        raise ValueError(f"state must be float32 [{ceil_div(k, block)}, {m}] for block {block}, got "
                         f"{state_x.dtype} {tuple(state_x.shape)}")
    x = x.contiguous()
    state_x = state_x.contiguous()
    out_dtype = block_linear_config.INPUT_OUTPUT_TORCH_TYPE
    output = torch.empty((m, k), device=x.device, dtype=out_dtype)
    with _on_device(x):
        rc = _lib.lib().bi8_dequantize_rowwise(_lib.ptr(x), _lib.ptr(state_x), _lib.ptr(output), _lib.dtype_code(out_dtype),
                                               m, k, block, _lib.stream_ptr())
    _lib.check(rc, "bi8_dequantize_rowwise")
    return output


def _gemm_operands(a: torch.Tensor, b: torch.Tensor):
    # same fix-ups as the reference (triton_functions.py:149-152), then bring both operands to the
    # K-contiguous form the library takes: a [M, K] row pitch lda, bt = b^T [N, K] row pitch ldb
    if a.stride(0) > 1 and a.stride(1) > 1:
        a = a.contiguous()
    if b.stride(0) > 1 and b.stride(1) > 1:
        b = b.contiguous()
    assert a.shape[1] == b.shape[0], "incompatible dimensions"
    if a.dtype != torch.int8 or b.dtype != torch.int8:
        raise ValueError(f"operands must be int8, got {a.dtype} and {b.dtype}")
    a = _rows_contiguous(a)
    bt = _rows_contiguous(b.t())
    # The tensor-core kernel needs 16-byte aligned operand rows.  For a large contraction length that is not a multiple
    # of 16 (GPT-2's 50257-wide dX contraction) re-pitch both operands once: the values are untouched, the row pitch becomes
    # the next multiple of 16 and the bytes between K and the pitch are never read.
    k = a.shape[1]
    if k % 16 != 0 and k >= 256 and a.shape[0] * bt.shape[0] >= 128 * 128:
        a, bt = _repitch(a), _repitch(bt)
    return a, bt


def _repitch(t: torch.Tensor) -> torch.Tensor:
    rows, k = t.shape
    if _pitch(t) % 16 == 0 and t.data_ptr() % 16 == 0:
        return t
    buf = torch.empty((rows, (k + 15) // 16 * 16), device=t.device, dtype=t.dtype)
    view = buf[:, :k]
    view.copy_(t)
    return view


def int8_matmul_block64_rowwise_dequantize(a, b, state_x, state_w, bias=None, *, flags: int = 0):
    """Block GEMM with fused dequantize (``triton_functions.py:142-168``).

    ``a`` int8 ``[M, K]``; ``b`` int8 ``[K, N]`` (on the layer's path the ``.t()`` view of a row-major
    ``[N, K]`` tensor); ``state_x [ceil(K/block), M]``, ``state_w [ceil(K/block), N]`` float32; optional
    ``bias [N]``.  Returns a new ``[M, N]`` tensor of ``INPUT_OUTPUT_TORCH_TYPE``:
    ``sum_j state_w[j,n] * state_x[j,m] * (a_j . b_j) / 127**2`` accumulated in fp32, cast, then
    ``+ bias`` in the output type.  ``flags`` selects a kernel variant (see ``include/bi8.h``)."""
    block = _block()
    assert a.is_cuda
    a, bt = _gemm_operands(a, b)
    m, k = a.shape
    n = bt.shape[0]
    nb = ceil_div(k, block)
    for name, st, rows in (("state_x", state_x, m), ("state_w", state_w, n)):
        if tuple(st.shape) != (nb, rows) or st.dtype != torch.float32:
            raise ValueError(f"{name} must be float32 [{nb}, {rows}] for block {block}, got {st.dtype} {tuple(st.shape)}")
    state_x = state_x.contiguous()
    state_w = state_w.contiguous()
    out_dtype = block_linear_config.INPUT_OUTPUT_TORCH_TYPE
    c = torch.empty((m, n), device=a.device, dtype=out_dtype)
    bias_code = 0
    if bias is not None:
        if bias.numel() != n:
            raise ValueError(f"bias must have {n} elements, got {bias.numel()}")
        bias = bias.reshape(n).contiguous()
        if bias.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            bias = bias.float()
        bias_code = _lib.dtype_code(bias.dtype)
    L = _lib.lib()
    with _on_device(a):
        ws_bytes = L.bi8_gemm_workspace_bytes(m, n, k, block)
        ws = _lib.workspace(a.device, ws_bytes)
        rc = L.bi8_gemm_dequant(_lib.ptr(a), _pitch(a), _lib.ptr(bt), _pitch(bt), _lib.ptr(state_x), _lib.ptr(state_w),
                                _lib.ptr(bias), bias_code, _lib.ptr(c), n, _lib.dtype_code(out_dtype), m, n, k, block,
                                _lib.ptr(ws), ws_bytes, flags, _lib.stream_ptr())
    _lib.check(rc, "bi8_gemm_dequant")
    return c


def quantize_matmul_block_rowwise_dequantize(x, b, state_w, bias=None, *, flags: int = 0):
    """``int8_matmul_block64_rowwise_dequantize(*quantize_block_rowwise(x), ...)`` in one library call: the two steps
    of the layer's forward (``block_linear.py:141-143``).  ``x [M, K]`` floating point, ``b [K, N]`` int8 (the ``.t()``
    view of the ``[N, K]`` weights), ``state_w [ceil(K/block), N]``.  For ``M <= 64`` a decode quantizer runs
    overlapped with the start of the weight-streaming GEMM; the result is bit-identical to the two separate calls either way."""
    block = _block()
    assert x.is_cuda
    if x.dim() != 2:
        raise ValueError(f"expected a 2-D tensor, got {tuple(x.shape)}")
    x = _rows_contiguous(x)
    if b.stride(0) > 1 and b.stride(1) > 1:
        b = b.contiguous()
    assert x.shape[1] == b.shape[0], "incompatible dimensions"
    if b.dtype != torch.int8:
        raise ValueError(f"weights must be int8, got {b.dtype}")
    bt = b.t()
    if bt.shape[1] != 1 and bt.stride(1) != 1:
        bt = bt.contiguous()
    m, k = x.shape
    n = bt.shape[0]
    nb = ceil_div(k, block)
    if tuple(state_w.shape) != (nb, n) or state_w.dtype != torch.float32:
        raise ValueError(f"state_w must be float32 [{nb}, {n}] for block {block}, got {state_w.dtype} {tuple(state_w.shape)}")
    state_w = state_w.contiguous()
    out_dtype = block_linear_config.INPUT_OUTPUT_TORCH_TYPE
    c = torch.empty((m, n), device=x.device, dtype=out_dtype)
    bias_code = 0
    if bias is not None:
        if bias.numel() != n:
            raise ValueError(f"bias must have {n} elements, got {bias.numel()}")
        bias = bias.reshape(n).contiguous()
        if bias.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            bias = bias.float()
        bias_code = _lib.dtype_code(bias.dtype)
    xq = torch.empty((m, k), device=x.device, dtype=torch.int8)
    sx = torch.empty((nb, m), device=x.device, dtype=torch.float32)
    L = _lib.lib()
    with _on_device(x):
        ws_bytes = L.bi8_gemm_workspace_bytes(m, n, k, block)
        ws = _lib.workspace(x.device, ws_bytes)
        rc = L.bi8_gemm_dequant_fused_quant(_lib.ptr(x), _lib.dtype_code(x.dtype), _pitch(x), _lib.ptr(xq), _lib.ptr(sx),
                                            _lib.ptr(bt), _pitch(bt), _lib.ptr(state_w), _lib.ptr(bias), bias_code, _lib.ptr(c),
                                            n, _lib.dtype_code(out_dtype), m, n, k, block, _lib.ptr(ws), ws_bytes, flags,
                                            _lib.stream_ptr())
    _lib.check(rc, "bi8_gemm_dequant_fused_quant")
    return c


def _pre_operands(op: str, x, x2, norm_weight):
    """Checks the operands of a fused producer step: returns (code, x, x2, weight) with shared row pitch and dtype."""
    if op not in ("none", "rmsnorm", "silu_mul"):
        raise ValueError(f"unknown producer step {op!r}: expected 'none', 'rmsnorm' or 'silu_mul'")
    assert x.is_cuda
    if x.dim() != 2:
        raise ValueError(f"expected a 2-D tensor, got {tuple(x.shape)}")
    x = _rows_contiguous(x)
    if op == "silu_mul":
        if x2 is None or tuple(x2.shape) != tuple(x.shape) or x2.dtype != x.dtype or x2.device != x.device:
            raise ValueError("silu_mul needs a second operand with x's shape, dtype and device")
        x2 = _rows_contiguous(x2)
        if _pitch(x2) != _pitch(x):         # e.g. one of the two was copied: give both the same row pitch
            x, x2 = x.contiguous(), x2.contiguous()
    else:
        x2 = None
    if op == "rmsnorm" and norm_weight is not None:
        if norm_weight.numel() != x.shape[1]:
            raise ValueError(f"norm weight must have {x.shape[1]} elements, got {norm_weight.numel()}")
        norm_weight = norm_weight.reshape(-1).to(x.dtype).contiguous()
    else:
        norm_weight = None
    return {"none": _lib.PRE_NONE, "rmsnorm": _lib.PRE_RMSNORM, "silu_mul": _lib.PRE_SILU_MUL}[op], x, x2, norm_weight


def _quantize_pre(op, x, x2, norm_weight, eps, fblock_size):
    block = _block(fblock_size)
    code, x, x2, norm_weight = _pre_operands(op, x, x2, norm_weight)
    m, k = x.shape
    q = torch.empty((m, k), device=x.device, dtype=torch.int8)
    state = torch.empty((ceil_div(k, block), m), device=x.device, dtype=_scale_dtype())
    with _on_device(x):
        rc = _lib.lib().bi8_quantize_rowwise_pre(code, _lib.ptr(x), _lib.ptr(x2), _lib.dtype_code(x.dtype), _pitch(x),
                                                 _lib.ptr(norm_weight), float(eps), _lib.ptr(q), _lib.ptr(state), m, k, block,
                                                 _lib.stream_ptr())
    _lib.check(rc, "bi8_quantize_rowwise_pre")
    return q, state


def rmsnorm_quantize_block_rowwise(x: torch.Tensor, eps: float = 1e-5, weight: torch.Tensor = None, fblock_size=None):
    """``quantize_block_rowwise(y)`` for ``y = (x * rsqrt(mean(x^2, -1) + eps) [* weight]).to(x.dtype)`` without writing
    ``y``: the normalisation in front of a layer's q/k/v and gate/up projections fused into their quantizer (the
    reference quantizes a tensor another kernel stored just before, ``block_linear.py:141``).  fp32 arithmetic, one
    rounding to ``x.dtype``, then the quantizer's own arithmetic; the row's sum of squares is taken in a fixed order."""
    return _quantize_pre("rmsnorm", x, None, weight, eps, fblock_size)


def silu_mul_quantize_block_rowwise(gate: torch.Tensor, up: torch.Tensor, fblock_size=None):
    """``quantize_block_rowwise(F.silu(gate) * up)`` without writing the product (the gated activation in front of a
    layer's down projection): ``silu`` in fp32 rounded to the activation type, the product rounded again, as the two
    separate kernels would, then quantized; bit-identical to the three-step form."""
    return _quantize_pre("silu_mul", gate, up, None, 0.0, fblock_size)


def pre_quantize_matmul_block_rowwise_dequantize(op: str, x, b, state_w, bias=None, *, x2=None, norm_weight=None, eps: float = 1e-5,
                                                 residual=None, out=None, flags: int = 0):
    """``quantize_matmul_block_rowwise_dequantize`` with the producer step ``op`` ('none', 'rmsnorm', 'silu_mul') fused
    in front of the quantizer and an optional ``residual [M, N]`` (of the output type) added to the result in the output
    type, the way a transformer layer's ``x + proj(act(...))`` does.  ``out`` may be given (it may be ``residual``
    itself: updated in place, directly on the decode path, through a temporary elsewhere).  For ``M <= 64`` this is
    quantizer + weight-streaming GEMM (+ its reduction), with the residual added by the kernel that writes the result."""
    block = _block()
    code, x, x2, norm_weight = _pre_operands(op, x, x2, norm_weight)
    if b.stride(0) > 1 and b.stride(1) > 1:
        b = b.contiguous()
    assert x.shape[1] == b.shape[0], "incompatible dimensions"
    if b.dtype != torch.int8:
        raise ValueError(f"weights must be int8, got {b.dtype}")
    bt = b.t()
    if bt.shape[1] != 1 and bt.stride(1) != 1:
        bt = bt.contiguous()
    m, k = x.shape
    n = bt.shape[0]
    nb = ceil_div(k, block)
    if tuple(state_w.shape) != (nb, n) or state_w.dtype != torch.float32:
        raise ValueError(f"state_w must be float32 [{nb}, {n}] for block {block}, got {state_w.dtype} {tuple(state_w.shape)}")
    state_w = state_w.contiguous()
    out_dtype = block_linear_config.INPUT_OUTPUT_TORCH_TYPE
    if out is None:
        out = torch.empty((m, n), device=x.device, dtype=out_dtype)
    elif tuple(out.shape) != (m, n) or out.dtype != out_dtype or out.stride(1) != 1 or out.device != x.device:
        raise ValueError(f"out must be {out_dtype} [{m}, {n}] with contiguous rows on {x.device}")
    if residual is not None:
        if tuple(residual.shape) != (m, n) or residual.dtype != out_dtype or residual.stride(1) != 1 or residual.device != x.device:
            raise ValueError(f"residual must be {out_dtype} [{m}, {n}] with contiguous rows on {x.device}")
    bias_code = 0
    if bias is not None:
        if bias.numel() != n:
            raise ValueError(f"bias must have {n} elements, got {bias.numel()}")
        bias = bias.reshape(n).contiguous()
        if bias.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            bias = bias.float()
        bias_code = _lib.dtype_code(bias.dtype)
    final = None
    if residual is not None and out.data_ptr() == residual.data_ptr() and not (
            m <= 64 and bias is None and n % 4 == 0 and k % 16 == 0 and _pitch(out) == _pitch(residual)):
        final, out = out, torch.empty((m, n), device=x.device, dtype=out_dtype)    # not the path that may update in place
    xq = torch.empty((m, k), device=x.device, dtype=torch.int8)
    sx = torch.empty((nb, m), device=x.device, dtype=torch.float32)
    L = _lib.lib()
    with _on_device(x):
        ws_bytes = L.bi8_gemm_workspace_bytes(m, n, k, block)
        ws = _lib.workspace(x.device, ws_bytes)
        rc = L.bi8_gemm_dequant_fused_pre(code, _lib.ptr(x), _lib.ptr(x2), _lib.dtype_code(x.dtype), _pitch(x), _lib.ptr(norm_weight),
                                          float(eps), _lib.ptr(xq), _lib.ptr(sx), _lib.ptr(bt), _pitch(bt), _lib.ptr(state_w),
                                          _lib.ptr(bias), bias_code, _lib.ptr(residual), _pitch(residual) if residual is not None else 0,
                                          _lib.ptr(out), _pitch(out), _lib.dtype_code(out_dtype), m, n, k, block, _lib.ptr(ws), ws_bytes,
                                          flags, _lib.stream_ptr())
    _lib.check(rc, "bi8_gemm_dequant_fused_pre")
    if final is not None:
        final.copy_(out)
        return final
    return out


def int8_matmul_block_partials(a, b, fblock_size=None, *, flags: int = 0):
    """Exact int32 block partial sums ``P[j] = a[:, jB:(j+1)B] @ b[jB:(j+1)B, :]`` as ``[ceil(K/B), M, N]``,
    produced by the same loads and tensor-core instructions as the GEMM (``triton_functions.py:115``)."""
    block = _block(fblock_size)
    assert a.is_cuda
    a, bt = _gemm_operands(a, b)
    m, k = a.shape
    n = bt.shape[0]
    out = torch.zeros((ceil_div(k, block), m, n), device=a.device, dtype=torch.int32)
    with _on_device(a):
        rc = _lib.lib().bi8_gemm_block_partials(_lib.ptr(a), _pitch(a), _lib.ptr(bt), _pitch(bt), _lib.ptr(out), m, n, k,
                                                block, flags, _lib.stream_ptr())
    _lib.check(rc, "bi8_gemm_block_partials")
    return out


def fast_matmulT(a, b):
    """``a [M, K] @ b[N, K]^T`` with both operands quantized on the fly (``triton_functions.py:511-514``)."""
    a_int8, a_state = quantize_block_rowwise(a)
    b_int8, b_state = quantize_block_rowwise(b)
    return int8_matmul_block64_rowwise_dequantize(a_int8, b_int8.t(), a_state, b_state)
