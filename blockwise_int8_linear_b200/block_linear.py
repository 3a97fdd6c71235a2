"""The blockwise-int8 linear layer: autograd function, ``nn.Linear`` replacement and model patcher.

Mirrors the reference's ``block_linear.py``: ``replace_linear_with_blockwise_int8`` (16-32),
``fast_matmul`` (34-40), ``blockwise_int8_linear`` (69-112) and ``BlockInt8Linear`` (114-152).
``BlockLinear`` and ``BlockLinearConfig`` are convenience aliases that the reference does not have.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import block_linear_config
from .triton_functions import (
    dequantize_block_rowwise,
    int8_matmul_block64_rowwise_dequantize,
    quantize_block_colwise,
    pre_quantize_matmul_block_rowwise_dequantize,
    quantize_block_dual,
    quantize_block_rowwise,
    quantize_matmul_block_rowwise_dequantize,
)

__all__ = [
    "replace_linear_with_blockwise_int8", "fast_matmul", "blockwise_int8_linear", "BlockInt8Linear", "BlockLinear",
    "BlockLinearConfig",
]


def replace_linear_with_blockwise_int8(model: nn.Module) -> nn.Module:
    """Swap every direct-child ``nn.Linear`` of ``model`` for a ``BlockInt8Linear`` sharing its weight and
    bias storage (``block_linear.py:16-32``).  Not recursive: use ``model.apply(replace_linear_with_blockwise_int8)``
    to patch a whole tree, as with the reference."""
    names = [name for name, child in model.named_children() if type(child) is nn.Linear or
             (isinstance(child, nn.Linear) and not isinstance(child, BlockInt8Linear))]
    for name in names:
        old = model._modules[name]
        new = BlockInt8Linear(old.in_features, old.out_features, old.bias is not None, old.weight.device,
                              old.weight.dtype, _skip_init=True)
        new.weight.data = old.weight.data
        if old.bias is not None:
            new.bias.data = old.bias.data
        new.train(old.training)
        model._modules[name] = new
    return model


def fast_matmul(a, b):
    """``a [M, K] @ b [K, N]`` with both operands quantized on the fly (``block_linear.py:34-40``, without its
    debug prints)."""
    b_int8, b_state = quantize_block_colwise(b)            # == quantize(b.t().contiguous())
    a_int8, a_state = quantize_block_rowwise(a)
    return int8_matmul_block64_rowwise_dequantize(a_int8, b_int8.t(), a_state, b_state)


def _weight_cache(W):
    """The int8 copies of a weight that are still valid, or None when caching is off.

    With ``block_linear_config.CACHE_QUANTIZED_WEIGHTS`` the K-blocked copy (forward) and the N-blocked copy (dX) of a
    weight are kept on the tensor object until the weight changes: the key holds the tensor's version counter, which
    every in-place update (an optimizer step) advances, its storage address, shape, dtype and the block size.  Several
    micro-steps between optimizer steps, or evaluation passes in train mode, then quantize the weight once instead of
    twice per call (the reference re-quantizes in every call, ``block_linear.py:79,93-94``)."""
    if not getattr(block_linear_config, "CACHE_QUANTIZED_WEIGHTS", False):
        return None
    key = (W._version, W.data_ptr(), tuple(W.shape), W.dtype, block_linear_config.GROUP_SIZE)
    cache = getattr(W, "_bi8_quantized", None)
    if cache is None or cache.get("key") != key:
        cache = {"key": key}
        try:
            W._bi8_quantized = cache
        except AttributeError:
            return None
    return cache


class blockwise_int8_linear(torch.autograd.Function):
    """``y = x @ W^T + bias`` with every GEMM (forward, dX, dW) done in blockwise int8
    (``block_linear.py:69-112``).  X and W are re-quantized on every call, as in the reference (unless
    ``CACHE_QUANTIZED_WEIGHTS`` is set); the transposed operands of the backward GEMMs are quantized straight from
    the row-major tensors by the fused column-wise quantizer, which is bit-identical to ``t().contiguous()`` +
    row-wise quantize.  With ``FUSE_DUAL_QUANTIZE`` (default) X and G are each read once for both of their
    quantizations, and the backward pass keeps X as its transposed int8 copy; every result is unchanged."""

    @staticmethod
    def forward(ctx, X_3D, W, bias):
        X = X_3D.reshape(-1, X_3D.size(-1))
        ctx.has_bias = bias is not None
        ctx.wcache = cache = _weight_cache(W)
        if ctx.needs_input_grad[1] and getattr(block_linear_config, "FUSE_DUAL_QUANTIZE", True):
            # the weight gradient needs X blocked along the tokens (block_linear.py:100-101): both quantizations come
            # from one read of X, and the backward pass keeps the int8 transposed copy instead of X itself
            X_int8, state_X, Xt_int8, state_Xt = quantize_block_dual(X)
            ctx.save_for_backward(Xt_int8, state_Xt, W)
            ctx.x_quantized = True
            ctx.block = block_linear_config.GROUP_SIZE
        else:
            X_int8, state_X = quantize_block_rowwise(X)
            ctx.save_for_backward(X, W)
            ctx.x_quantized = False
        if cache is not None and "row" in cache:
            W_int8, state_W = cache["row"]
        else:
            W_int8, state_W = quantize_block_rowwise(W)
            if cache is not None:
                cache["row"] = (W_int8, state_W)
        out = int8_matmul_block64_rowwise_dequantize(X_int8, W_int8.t(), state_X, state_W, bias)
        return out.view(*X_3D.size()[:-1], -1)

    @staticmethod
    def backward(ctx, G_3D):
        G = G_3D.reshape(-1, G_3D.size(-1))
        if ctx.x_quantized:
            if ctx.block != block_linear_config.GROUP_SIZE:
                raise RuntimeError("GROUP_SIZE changed between the forward and the backward pass of a BlockInt8Linear")
            x_int8, x_state, W = ctx.saved_tensors
        else:
            X, W = ctx.saved_tensors
        grad_X = grad_W = grad_bias = None
        gt_int8 = None
        if ctx.needs_input_grad[0] and ctx.needs_input_grad[1] and getattr(block_linear_config, "FUSE_DUAL_QUANTIZE", True):
            # G is needed blocked along N (for dX) and along the tokens (for dW): one read
            g_int8, g_state, gt_int8, gt_state = quantize_block_dual(G)
        elif ctx.needs_input_grad[0]:
            g_int8, g_state = quantize_block_rowwise(G)
        if ctx.needs_input_grad[0]:
            # contraction over N: both operands blocked along N (block_linear.py:92-95)
            cache = ctx.wcache         # still valid: autograd refuses to run backward on a weight modified since forward
            if cache is not None and "col" in cache:
                Wt_int8, w_state = cache["col"]
            else:
                Wt_int8, w_state = quantize_block_colwise(W)                 # [K, N], state [N/B, K]
                if cache is not None:
                    cache["col"] = (Wt_int8, w_state)
            grad_X = int8_matmul_block64_rowwise_dequantize(g_int8, Wt_int8.t(), g_state, w_state)
            grad_X = grad_X.view(*G_3D.size()[:-1], -1)
        if ctx.needs_input_grad[1]:
            # contraction over the tokens: both operands blocked along M (block_linear.py:100-104)
            if not ctx.x_quantized:
                x_int8, x_state = quantize_block_colwise(X)                  # [K, M], state [M/B, K]
            if gt_int8 is None:
                gt_int8, gt_state = quantize_block_colwise(G)                # [N, M], state [M/B, N]
            grad_W = int8_matmul_block64_rowwise_dequantize(gt_int8, x_int8.t(), gt_state, x_state)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_bias = G.sum(dim=0)
        return grad_X, grad_W, grad_bias


class BlockInt8Linear(nn.Linear):
    """Drop-in ``nn.Linear`` (``block_linear.py:114-152``).

    Training mode runs ``blockwise_int8_linear``.  Eval mode quantizes the weight once on the first forward
    (buffers ``W_int8`` int8 ``[out, in]`` and ``state_W`` float32 ``[ceil(in/block), out]``, which become part of
    ``state_dict()``), then quantizes the activation and runs the fused GEMM on every call."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 _skip_init: bool = False):
        if _skip_init:
            # the caller rebinds weight/bias storage right away: skip the random init of nn.Linear
            nn.Module.__init__(self)
            self.in_features, self.out_features = in_features, out_features
            kw = {"device": device, "dtype": dtype}
            self.weight = nn.Parameter(torch.empty((0,), **kw))
            if bias:
                self.bias = nn.Parameter(torch.empty((0,), **kw))
            else:
                self.register_parameter("bias", None)
        else:
            super().__init__(in_features, out_features, bias, device, dtype)

    def prepare_for_eval(self, drop_weight: bool = None):
        """Quantizes the weight into the buffers ``W_int8`` / ``state_W`` (``block_linear.py:125-128``).  With
        ``drop_weight`` (default: ``block_linear_config.DROP_WEIGHT_IN_EVAL``, off like the reference) the floating-point
        weight is released afterwards: the parameter stays in place with zero elements, so ``state_dict()`` keeps its
        key, and inference runs from the int8 copy alone (a 7B model then holds 6.7 GB instead of 20 GB).  Training, or
        changing ``GROUP_SIZE``, needs the weight back: load a state dict that carries it."""
        if self.weight.numel() == 0:
            if not hasattr(self, "W_int8"):
                raise RuntimeError("BlockInt8Linear has neither a floating-point weight nor int8 buffers")
            return
        W_int8, state_W = quantize_block_rowwise(self.weight.detach())
        self.register_buffer("W_int8", W_int8)
        self.register_buffer("state_W", state_W)
        if drop_weight is None:
            drop_weight = getattr(block_linear_config, "DROP_WEIGHT_IN_EVAL", False)
        if drop_weight:
            self.weight.data = torch.empty(0, device=self.weight.device, dtype=self.weight.dtype)

    def dequantized_weight(self):
        """The weight after a quantize/dequantize round trip, in ``INPUT_OUTPUT_TORCH_TYPE`` (the working part of
        the reference's ``weight_quant_training``, ``block_linear.py:130-135``)."""
        W_int8, state_W = quantize_block_rowwise(self.weight.detach())
        return dequantize_block_rowwise(W_int8, state_W)

    def infer(self, x):
        if not hasattr(self, "W_int8"):
            self.prepare_for_eval()
        X = x.reshape(-1, x.size(-1))
        if X.size(0) <= 64:
            # decode-sized batches: the same two steps in one library call whose kernels overlap
            return quantize_matmul_block_rowwise_dequantize(X, self.W_int8.t(), self.state_W, self.bias).view(*x.size()[:-1], -1)
        X_int8, state_X = quantize_block_rowwise(X)
        return int8_matmul_block64_rowwise_dequantize(
            X_int8, self.W_int8.t(), state_X, self.state_W, self.bias
        ).view(*x.size()[:-1], -1)

    def infer_pre(self, x, op="none", x2=None, norm_weight=None, eps=1e-5, residual=None):
        """``infer`` with the elementwise step that produces this projection's input fused into the quantizer, and the
        residual sum that consumes its output fused behind the GEMM (neither exists in the reference, whose ``infer``
        quantizes a stored tensor, ``block_linear.py:141``):

        ``op='rmsnorm'``   ``infer(rms_norm(x, eps) [* norm_weight])``
        ``op='silu_mul'``  ``infer(F.silu(x) * x2)``
        ``residual``       ``residual + infer(...)`` in the activation type; ``residual`` has the output's shape."""
        if not hasattr(self, "W_int8"):
            self.prepare_for_eval()
        X = x.reshape(-1, x.size(-1))
        X2 = x2.reshape(-1, x2.size(-1)) if x2 is not None else None
        R = residual.reshape(-1, residual.size(-1)) if residual is not None else None
        out = pre_quantize_matmul_block_rowwise_dequantize(op, X, self.W_int8.t(), self.state_W, self.bias, x2=X2,
                                                           norm_weight=norm_weight, eps=eps, residual=R)
        return out.view(*x.size()[:-1], -1)

    def forward(self, x):
        if not self.training:
            return self.infer(x)
        if self.weight.numel() == 0:
            raise RuntimeError("this BlockInt8Linear dropped its floating-point weight for inference; training needs it")
        return blockwise_int8_linear.apply(x, self.weight, self.bias)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        # a checkpoint saved after the first eval forward carries W_int8/state_W: make room for them
        for name in ("W_int8", "state_W"):
            key = prefix + name
            if key in state_dict and not hasattr(self, name):
                self.register_buffer(name, torch.empty_like(state_dict[key], device=self.weight.device))
        # a checkpoint saved after the floating-point weight was dropped carries an empty `weight` (and the other way
        # round): take the shape the checkpoint has
        key = prefix + "weight"
        if key in state_dict and state_dict[key].shape != self.weight.shape:
            self.weight.data = torch.empty_like(state_dict[key], device=self.weight.device, dtype=self.weight.dtype)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)


BlockLinear = BlockInt8Linear


class BlockLinearConfig:
    """Attribute-style view of the module-level knobs in ``block_linear_config`` (the reference has only the
    globals, ``block_linear_config.py:3-5``).  Reading and assigning go straight to those globals; used as a
    context manager it restores the previous values on exit."""

    _FIELDS = {"group_size": "GROUP_SIZE", "scale_dtype": "SHARED_EXP_TORCH_TYPE", "io_dtype": "INPUT_OUTPUT_TORCH_TYPE"}

    def __init__(self, group_size=None, io_dtype=None, scale_dtype=None):
        object.__setattr__(self, "_pending", {k: v for k, v in
                                              (("group_size", group_size), ("io_dtype", io_dtype), ("scale_dtype", scale_dtype))
                                              if v is not None})
        object.__setattr__(self, "_saved", None)

    def __getattr__(self, name):
        if name in self._FIELDS:
            return getattr(block_linear_config, self._FIELDS[name])
        raise AttributeError(name)

    def __setattr__(self, name, value):
        if name not in self._FIELDS:
            raise AttributeError(name)
        setattr(block_linear_config, self._FIELDS[name], value)

    def apply(self):
        for k, v in self._pending.items():
            setattr(self, k, v)
        return self

    def __enter__(self):
        object.__setattr__(self, "_saved", {k: getattr(self, k) for k in self._FIELDS})
        return self.apply()

    def __exit__(self, *exc):
        for k, v in self._saved.items():
            setattr(self, k, v)
        return False
