"""Sharding of the blockwise-int8 linear layer over the GPUs of one node (``torch.distributed``).

The reference is single-GPU; these helpers add the three ways its layer shards:

* tokens (data parallel): every rank runs the whole layer on its own rows — no collective on the forward path;
  training averages gradients with ``allreduce_gradients``.
* output features (column parallel): rank r holds ``W[n_lo:n_hi, :]`` with its scales; its output columns are
  bit-identical to the same columns of the unsharded layer; ``all_gather`` concatenates them when asked.
* input features (row parallel): rank r holds ``W[:, k_lo:k_hi]`` with ``k_lo`` a multiple of the block size, so
  blocks and scales are those of the unsharded layer; each rank produces an fp32 partial result over its blocks
  and one ``all_reduce`` sums them (equal to the unsharded result up to fp32 summation order).

The functional ops are looked up in an ``ops`` namespace (default: this package's CUDA-backed
``triton_functions``), which lets the host-side logic be exercised on CPU ranks with any stand-in that has the same
three functions.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from . import block_linear_config


def _default_ops():
    from . import triton_functions
    return triton_functions


def block_aligned_bounds(total: int, parts: int, block: int) -> List[Tuple[int, int]]:
    """Split ``range(total)`` into ``parts`` contiguous pieces whose boundaries are multiples of ``block``, sizes
    differing by at most one block (e.g. 11008 = 172 blocks of 64 over 8 ranks -> 4 x 22 + 4 x 21 blocks).
    Trailing ranks get empty pieces when there are fewer blocks than parts."""
    if total < 0 or parts < 1 or block < 1:
        raise ValueError("block_aligned_bounds: bad arguments")
    nblocks = -(total // -block)
    base, extra = divmod(nblocks, parts)
    out, lo = [], 0
    for r in range(parts):
        n = base + (1 if r < extra else 0)
        hi = min(total, lo + n * block)
        out.append((lo, hi))
        lo = hi
    return out


def shard_columns(weight: torch.Tensor, bias: Optional[torch.Tensor], rank: int, world: int, block: Optional[int] = None):
    """Rows ``[n_lo:n_hi]`` of ``weight [N, K]`` (output features) for column-parallel use."""
    block = block or block_linear_config.GROUP_SIZE
    lo, hi = block_aligned_bounds(weight.shape[0], world, block)[rank]
    return weight[lo:hi].contiguous(), (None if bias is None else bias[lo:hi].contiguous()), (lo, hi)


def shard_rows(weight: torch.Tensor, rank: int, world: int, block: Optional[int] = None):
    """Columns ``[k_lo:k_hi]`` of ``weight [N, K]`` (input features) for row-parallel use; block aligned."""
    block = block or block_linear_config.GROUP_SIZE
    lo, hi = block_aligned_bounds(weight.shape[1], world, block)[rank]
    return weight[:, lo:hi].contiguous(), (lo, hi)


def column_parallel_forward(x: torch.Tensor, w_int8: torch.Tensor, state_w: torch.Tensor, bias: Optional[torch.Tensor],
                            group=None, gather: bool = True, sizes: Optional[List[int]] = None, ops=None):
    """``x [M, K]`` replicated; ``w_int8 [N_r, K]``, ``state_w [K/B, N_r]`` this rank's shard.  Returns the local
    ``[M, N_r]`` block, or with ``gather`` the full ``[M, N]`` (``sizes`` = N_r of every rank when they differ)."""
    ops = ops or _default_ops()
    xq, sx = ops.quantize_block_rowwise(x)
    y = ops.int8_matmul_block64_rowwise_dequantize(xq, w_int8.t(), sx, state_w, bias)
    if not gather or group is None and not dist.is_initialized():
        return y
    world = dist.get_world_size(group)
    if world == 1:
        return y
    sizes = sizes or [y.shape[1]] * world
    parts = [torch.empty((y.shape[0], n), dtype=y.dtype, device=y.device) for n in sizes]
    if len(set(sizes)) == 1:
        dist.all_gather(parts, y.contiguous(), group=group)
    else:
        # uneven shards: pad to the widest, gather, trim
        width = max(sizes)
        padded = torch.zeros((y.shape[0], width), dtype=y.dtype, device=y.device)
        padded[:, : y.shape[1]] = y
        bufs = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(bufs, padded, group=group)
        parts = [b[:, :n] for b, n in zip(bufs, sizes)]
    return torch.cat(parts, dim=1)


def row_parallel_forward(x_shard: torch.Tensor, w_int8: torch.Tensor, state_w: torch.Tensor, bias: Optional[torch.Tensor],
                         group=None, ops=None):
    """``x_shard [M, K_r]`` = this rank's block-aligned slice of the input features; ``w_int8 [N, K_r]``,
    ``state_w [K_r/B, N]``.  Partial sums are produced in fp32, summed over ranks, cast to the configured output
    type, and the bias is added once, after the cast, as in the unsharded layer."""
    ops = ops or _default_ops()
    out_dtype = block_linear_config.INPUT_OUTPUT_TORCH_TYPE
    xq, sx = ops.quantize_block_rowwise(x_shard)
    block_linear_config.INPUT_OUTPUT_TORCH_TYPE = torch.float32
    try:
        part = ops.int8_matmul_block64_rowwise_dequantize(xq, w_int8.t(), sx, state_w, None)
    finally:
        block_linear_config.INPUT_OUTPUT_TORCH_TYPE = out_dtype
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(part, op=dist.ReduceOp.SUM, group=group)
    y = part.to(out_dtype)
    if bias is not None:
        y = y + bias.to(out_dtype)
    return y


def allreduce_gradients(params, group=None, bucket_bytes: int = 64 << 20) -> int:
    """Average ``.grad`` of ``params`` over the ranks of ``group`` with bucketed flat all-reduces (buckets are sized for
    launch latency, not link count: NVSwitch gives every pair full bandwidth).  Returns the number of collectives."""
    if not dist.is_initialized():
        return 0
    world = dist.get_world_size(group)
    if world == 1:
        return 0
    grads = [p.grad for p in params if p.grad is not None]
    calls = 0
    by_dtype = {}
    for g in grads:
        by_dtype.setdefault(g.dtype, []).append(g)
    for dtype, gs in by_dtype.items():
        bucket, size = [], 0
        def flush():
            nonlocal bucket, size, calls
            if not bucket:
                return
            flat = torch.cat([g.reshape(-1) for g in bucket])
            dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
            flat.div_(world)
            off = 0
            for g in bucket:
                n = g.numel()
                g.copy_(flat[off:off + n].view_as(g))
                off += n
            calls += 1
            bucket, size = [], 0
        for g in gs:
            bucket.append(g)
            size += g.numel() * g.element_size()
            if size >= bucket_bytes:
                flush()
        flush()
    return calls
