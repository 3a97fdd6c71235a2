"""Sum of the fp32 partial results of a row-parallel ``BlockInt8Linear`` over NVLink peer memory.

The reference has no multi-GPU path; a Llama MLP sharded the usual way (``gate_up`` by columns, ``down`` by input
features, ``block_linear.py:141-143`` per shard) ends every layer half with a sum of ``[M, hidden]`` fp32 partial results
over the ranks.  ``PeerAllReduce`` does that sum with the library's own kernel (``bi8_peer_allreduce``: plain stores into
every rank's exchange buffer, a flag per chunk and rank, a bounded wait, the sum in rank order) instead of an NCCL call,
so that a decode step can be captured in one CUDA graph per rank with no host work between its kernels.

The exchange buffers come from ``torch.distributed._symmetric_memory`` (one allocation per rank, mapped by all ranks of
the group); only this library's kernel ever reads or writes them.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib, block_linear_config

__all__ = ["PeerAllReduce", "PeerAllReduceLarge"]

_CHUNK = 1024


def _exchange_buffers(nbytes: int, device, world: int, group, local: bool):
    """One zero-filled buffer of `nbytes` per rank, mapped by all ranks of the group: returns (tensors kept alive, symmetric
    memory handle or None, the eight device addresses the library's calls take).  With one rank, or `local` (a test hook:
    `world` buffers on this one device), the buffers are ordinary device memory."""
    if world == 1 or local:
        bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
        handle, ptrs = None, [b.data_ptr() for b in bufs]
    else:
        # plain peer mappings are all this needs: keep the allocation off NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        pg = group if group is not None else dist.group.WORLD
        name = pg.group_name
        enable = getattr(symm, "enable_symm_mem_for_group", None)
        if enable is not None:
            try:
                enable(name)
            except Exception:       # newer torch versions need no registration
                pass
        buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
        buf.zero_()
        handle = symm.rendezvous(buf, name)
        bufs = [buf]
        ptrs = [int(p) for p in handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group)         # every rank's buffer is zeroed before anybody's first kernel writes into it
    return bufs, handle, (ctypes.c_void_p * 8)(*(ptrs + [ptrs[0]] * (8 - len(ptrs))))


class PeerAllReduce:
    """``PeerAllReduce(capacity, device, group)(partial, bias)`` -> ``cast(sum over ranks of partial) + bias``.

    ``capacity``: largest ``M * N`` (fp32 values) one call will carry.  ``wait_limit_us``: how long a call waits for the
    other ranks before it gives up with ``BI8_ERR_TIMEOUT`` in the device status (ranks that reach the call seconds apart,
    e.g. right after capturing their graphs, need more than the default second).  With a group of one rank (or no
    process group) the buffer is ordinary device memory and the call is a cast + bias."""

    def __init__(self, capacity: int, device, group=None, wait_limit_us: int = 0, _local_world: int = 0):
        self.device = torch.device(device)
        self.wait_limit_us = int(wait_limit_us)          # default limit of the flag waits (0 = the library's one second)
        self.capacity = -(-int(capacity) // _CHUNK) * _CHUNK
        if _local_world:
            # test hook: `_local_world` exchange buffers on this one device, this object acting as rank 0 of them
            self.rank, self.world = 0, _local_world
        elif dist.is_initialized() and dist.get_world_size(group) > 1:
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        if self.world > 8:
            raise ValueError("PeerAllReduce supports at most 8 ranks")
        L = _lib.lib()
        nbytes = L.bi8_peer_allreduce_buffer_bytes(self.world, self.capacity)
        if nbytes == 0:
            raise ValueError(f"bad exchange buffer geometry: world {self.world}, capacity {self.capacity}")
        self._bufs, self._handle, self._ptrs = _exchange_buffers(nbytes, self.device, self.world, group, bool(_local_world))

    @staticmethod
    def _addend(bias, residual, m, n, out_dtype):
        """The one operand the kernels add after the cast: a bias [N], or a residual [M, N] of the output type."""
        if residual is not None:
            if bias is not None:
                raise ValueError("bias and residual cannot be combined in the peer-memory reduction")
            if residual.numel() != m * n or residual.dtype != out_dtype or not residual.is_contiguous():
                raise ValueError(f"residual must be a contiguous {out_dtype} tensor of {m} x {n} elements")
            return residual, _lib.dtype_code(residual.dtype) | _lib.ADDEND_FULL
        if bias is not None:
            bias = bias.reshape(n).contiguous()
            return bias, _lib.dtype_code(bias.dtype)
        return None, 0

    def __call__(self, partial: torch.Tensor, bias: torch.Tensor = None, out: torch.Tensor = None, wait_limit_us: int = None,
                 residual: torch.Tensor = None):
        """``cast(sum over ranks of partial) + bias`` or ``... + residual`` (a ``[M, N]`` tensor of the output type, e.g. the
        layer's input stream; it may be ``out``)."""
        if partial.dtype != torch.float32 or not partial.is_contiguous():
            raise ValueError("partial must be a contiguous float32 tensor")
        n = partial.shape[-1]
        m = partial.numel() // n
        out_dtype = block_linear_config.INPUT_OUTPUT_TORCH_TYPE
        if out is None:
            out = torch.empty(partial.shape, dtype=out_dtype, device=partial.device)
        addend, code = self._addend(bias, residual, m, n, out.dtype)
        if wait_limit_us is None:
            wait_limit_us = self.wait_limit_us
        with torch.cuda.device(partial.device):
            rc = _lib.lib().bi8_peer_allreduce(self._ptrs, self.rank, self.world, self.capacity, _lib.ptr(partial), m, n,
                                               _lib.ptr(addend), code, _lib.ptr(out), _lib.dtype_code(out.dtype),
                                               int(wait_limit_us), _lib.stream_ptr())
        _lib.check(rc, "bi8_peer_allreduce")
        return out

    def row_parallel_linear(self, x: torch.Tensor, w_int8: torch.Tensor, state_w: torch.Tensor, bias: torch.Tensor = None,
                            wait_limit_us: int = None, *, op: str = "none", x2: torch.Tensor = None, norm_weight: torch.Tensor = None,
                            eps: float = 1e-5, residual: torch.Tensor = None):
        """The whole row-parallel layer in one library call: ``x [..., K_r]`` is this rank's slice of the input features,
        ``w_int8 [N, K_r]`` / ``state_w [ceil(K_r/block), N]`` this rank's weight slice.  Returns
        ``cast(sum over ranks of pre(x_r) @ W_r^T) + bias`` (or ``+ residual``, a tensor of the output's shape and type).
        ``op`` / ``x2`` / ``norm_weight`` / ``eps``: the producer step fused into the quantizer, as in
        ``pre_quantize_matmul_block_rowwise_dequantize`` ('silu_mul' for a gated MLP's down projection; 'rmsnorm' would
        normalise over this rank's slice only and is rejected).  For decode-sized batches (at most 64 rows) the kernel that
        finishes the weight-streaming GEMM exchanges its sums with the other ranks itself; the result equals
        ``self(partial)`` on the fp32 output of ``quantize_matmul_block_rowwise_dequantize``."""
        from .triton_functions import _block, _pitch, _pre_operands, ceil_div
        if op == "rmsnorm" and self.world > 1:
            raise ValueError("a row-parallel layer holds a slice of the features: normalise before the slice is taken")
        block = _block()
        lead = x.shape[:-1]
        code, x2d, x2_2d, norm_weight = _pre_operands(op, x.reshape(-1, x.shape[-1]),
                                                      None if x2 is None else x2.reshape(-1, x2.shape[-1]), norm_weight)
        m, k = x2d.shape
        n = w_int8.shape[0]
        if w_int8.dtype != torch.int8 or w_int8.shape[1] != k or w_int8.stride(1) != 1:
            raise ValueError("w_int8 must be int8 [N, K] with contiguous rows")
        nb = ceil_div(k, block)
        if tuple(state_w.shape) != (nb, n) or state_w.dtype != torch.float32:
            raise ValueError(f"state_w must be float32 [{nb}, {n}] for block {block}")
        state_w = state_w.contiguous()
        out_dtype = block_linear_config.INPUT_OUTPUT_TORCH_TYPE
        dev = x2d.device
        out = torch.empty((m, n), dtype=out_dtype, device=dev)
        partial = torch.empty((m, n), dtype=torch.float32, device=dev)
        xq = torch.empty((m, k), dtype=torch.int8, device=dev)
        sx = torch.empty((nb, m), dtype=torch.float32, device=dev)
        addend, addend_code = self._addend(bias, None if residual is None else residual.reshape(m, n), m, n, out_dtype)
        if wait_limit_us is None:
            wait_limit_us = self.wait_limit_us
        L = _lib.lib()
        with torch.cuda.device(dev):
            ws_bytes = L.bi8_gemm_workspace_bytes(m, n, k, block)
            ws = _lib.workspace(dev, ws_bytes)
            rc = L.bi8_row_parallel_linear_pre(code, _lib.ptr(x2d), _lib.ptr(x2_2d), _lib.dtype_code(x2d.dtype), _pitch(x2d),
                                               _lib.ptr(norm_weight), float(eps), _lib.ptr(xq), _lib.ptr(sx), _lib.ptr(w_int8),
                                               _pitch(w_int8), _lib.ptr(state_w), _lib.ptr(partial), m, n, k, block, _lib.ptr(ws),
                                               ws_bytes, self._ptrs, self.rank, self.world, self.capacity, _lib.ptr(addend),
                                               addend_code, _lib.ptr(out), _lib.dtype_code(out_dtype), int(wait_limit_us), 0,
                                               _lib.stream_ptr())
        _lib.check(rc, "bi8_row_parallel_linear_pre")
        return out.view(*lead, n)


class PeerAllReduceLarge:
    """The same sum for prefill-sized results (``bi8_peer_allreduce_large``): every rank owns one chunk in ``world`` of the
    result, loads that chunk of every rank's partial result over NVLink, adds in rank order, casts, adds bias or residual
    and stores the chunk into every rank's output — reduce-scatter by peer loads, all-gather by peer stores, one kernel.

    The partial results and the output live inside the exchange buffer: ``partial(m, n)`` is the fp32 view the GEMM should
    write into (``pre_quantize_matmul_block_rowwise_dequantize(..., out=...)`` with a float32 output type), ``reduce(m, n)``
    returns the ``[m, n]`` view of the output region, valid until the next ``reduce``."""

    def __init__(self, capacity: int, device, group=None, wait_limit_us: int = 0, _local_world: int = 0):
        self.device = torch.device(device)
        self.wait_limit_us = int(wait_limit_us)
        self.capacity = -(-int(capacity) // _CHUNK) * _CHUNK
        if _local_world:
            self.rank, self.world = 0, _local_world
        elif dist.is_initialized() and dist.get_world_size(group) > 1:
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        if self.world > 8:
            raise ValueError("PeerAllReduceLarge supports at most 8 ranks")
        L = _lib.lib()
        nbytes = L.bi8_peer_allreduce_large_buffer_bytes(self.world, self.capacity)
        if nbytes == 0:
            raise ValueError(f"bad exchange buffer geometry: world {self.world}, capacity {self.capacity}")
        self._bufs, self._handle, self._ptrs = _exchange_buffers(nbytes, self.device, self.world, group, bool(_local_world))
        own = self._bufs[0]
        p_off, o_off = L.bi8_peer_allreduce_large_partial_offset(), L.bi8_peer_allreduce_large_out_offset(self.capacity)
        self._partial = own[p_off:p_off + 4 * self.capacity].view(torch.float32)
        self._out_bytes = own[o_off:o_off + 4 * self.capacity]

    def partial(self, m: int, n: int) -> torch.Tensor:
        """This rank's ``[m, n]`` float32 partial region (write the GEMM's result here, then call ``reduce``)."""
        if m * n > self.capacity:
            raise ValueError(f"{m} x {n} exceeds the capacity {self.capacity}")
        return self._partial[: m * n].view(m, n)

    def reduce(self, m: int, n: int, bias: torch.Tensor = None, residual: torch.Tensor = None, wait_limit_us: int = None) -> torch.Tensor:
        """``cast(sum over ranks of partial(m, n)) + bias`` (or ``+ residual``, ``[m, n]`` of the output type, which may be
        the previous result's view): a view of the output region in ``block_linear_config.INPUT_OUTPUT_TORCH_TYPE``."""
        if m * n > self.capacity or n % 4:
            raise ValueError(f"{m} x {n}: exceeds the capacity {self.capacity} or n is not a multiple of 4")
        out_dtype = block_linear_config.INPUT_OUTPUT_TORCH_TYPE
        addend, code = PeerAllReduce._addend(bias, residual, m, n, out_dtype)
        if wait_limit_us is None:
            wait_limit_us = self.wait_limit_us
        with torch.cuda.device(self.device):
            rc = _lib.lib().bi8_peer_allreduce_large(self._ptrs, self.rank, self.world, self.capacity, m, n, _lib.ptr(addend), code,
                                                     _lib.dtype_code(out_dtype), int(wait_limit_us), _lib.stream_ptr())
        _lib.check(rc, "bi8_peer_allreduce_large")
        esz = torch.empty((), dtype=out_dtype).element_size()
        return self._out_bytes[: m * n * esz].view(out_dtype).view(m, n)
