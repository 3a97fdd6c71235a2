"""Model-side helpers for a decode step that sit between two of the library's kernels (the reference has no model code).

``rope_cache_append`` takes what a fused q/k/v ``BlockInt8Linear`` leaves for one new token per sequence, rotates q and k by
the position's angle and appends k and v to the caches in one launch (``bi8_rope_cache_append``); written with tensor
operations the same step is five launches per layer.
"""
from __future__ import annotations

import torch

from . import _lib

__all__ = ["rope_cache_append"]


def rope_cache_append(qkv: torch.Tensor, cis: torch.Tensor, pos: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor) -> torch.Tensor:
    """``qkv [B, 3, H, D]`` (bf16 / fp16, contiguous): q, k, v of one new token per sequence.  ``cis [D/2]`` complex64 (or
    ``[D/2, 2]`` float32: cos, sin) of the step's position, ``pos`` an int64 device tensor with one element (the cache row),
    ``kcache`` / ``vcache [B, H, max_len, D]`` contiguous.  Returns the rotated q as ``[B, H, 1, D]``; row ``pos`` of the caches
    receives the rotated k and v.  Feature pairs are (even, odd) neighbours: ``(x0 + i x1) * cis``."""
    assert qkv.is_cuda
    b, three, h, d = qkv.shape
    if three != 3 or d % 2:
        raise ValueError(f"expected [B, 3, H, D] with even D, got {tuple(qkv.shape)}")
    if not qkv.is_contiguous():
        qkv = qkv.contiguous()
    if cis.is_complex():
        cis = torch.view_as_real(cis)
    cis = cis.reshape(-1, 2)
    if cis.shape[0] != d // 2 or cis.dtype != torch.float32 or not cis.is_contiguous():
        raise ValueError(f"cis must hold {d // 2} contiguous (cos, sin) float32 pairs")
    if pos.dtype != torch.int64 or pos.numel() != 1 or pos.device != qkv.device:
        raise ValueError("pos must be an int64 tensor with one element on the activations' device")
    max_len = kcache.shape[2]
    for c in (kcache, vcache):
        if tuple(c.shape) != (b, h, max_len, d) or c.dtype != qkv.dtype or not c.is_contiguous() or c.device != qkv.device:
            raise ValueError(f"caches must be contiguous {qkv.dtype} [{b}, {h}, max_len, {d}] on {qkv.device}")
    q = torch.empty((b, h, 1, d), device=qkv.device, dtype=qkv.dtype)
    with torch.cuda.device(qkv.device):
        rc = _lib.lib().bi8_rope_cache_append(_lib.ptr(qkv), _lib.dtype_code(qkv.dtype), _lib.ptr(cis), _lib.ptr(pos), _lib.ptr(q),
                                              _lib.ptr(kcache), _lib.ptr(vcache), b, h, d, max_len, _lib.stream_ptr())
    _lib.check(rc, "bi8_rope_cache_append")
    return q
