"""ctypes binding of libbi8.so (declared in include/bi8.h).

There is no fallback: if the library cannot be loaded, or a call returns an error status, an
exception is raised.  Tensors are passed as raw device pointers plus sizes; the current torch
CUDA stream is passed to every call.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbi8.so")

BI8_BF16, BI8_F32, BI8_F16 = 0, 1, 2
GEMM_DEFAULT, GEMM_FORCE_GENERIC, GEMM_FORCE_TC, GEMM_NO_SEED, GEMM_FORCE_SMALLM, GEMM_FORCE_SKINNY = 0, 1, 2, 4, 8, 16
GEMM_QUANT_IN_KERNEL = 32

_DTYPE_CODE = {torch.bfloat16: BI8_BF16, torch.float32: BI8_F32, torch.float16: BI8_F16}

EXPORTS = [
    "bi8_version", "bi8_last_error_string", "bi8_device_status", "bi8_quantize_rowwise", "bi8_quantize_colwise", "bi8_quantize_dual", "bi8_peer_allreduce", "bi8_peer_allreduce_buffer_bytes", "bi8_row_parallel_linear",
    "bi8_dequantize_rowwise", "bi8_gemm_dequant", "bi8_gemm_workspace_bytes", "bi8_gemm_block_partials",
    "bi8_gemm_dequant_fused_quant", "bi8_mma_peak_probe", "bi8_gemm_dequant_static", "bi8_gemm_static_scratch_bytes",
    "bi8_gemm_wait_selftest", "bi8_stream_capture_id", "bi8_quantize_rowwise_pre", "bi8_gemm_dequant_fused_pre",
    "bi8_row_parallel_linear_pre", "bi8_peer_allreduce_large", "bi8_peer_allreduce_large_buffer_bytes",
    "bi8_peer_allreduce_large_partial_offset", "bi8_peer_allreduce_large_out_offset", "bi8_rope_cache_append",
]
ADDEND_FULL = 0x100
PRE_NONE, PRE_RMSNORM, PRE_SILU_MUL = 0, 1, 2

_lib = None


class Bi8Error(RuntimeError):
    """A libbi8 entry point returned a non-zero status."""


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m blockwise_int8_linear_b200.build` "
                "(there is no non-CUDA fallback)")
        L = ctypes.CDLL(LIB_PATH)
        c = ctypes
        vp, i64, i32, sz = c.c_void_p, c.c_int64, c.c_int, c.c_size_t
        L.bi8_version.restype = i32
        L.bi8_last_error_string.restype = c.c_char_p
        L.bi8_device_status.argtypes = [c.POINTER(i32)]
        L.bi8_quantize_rowwise.argtypes = [vp, i32, i64, vp, vp, i64, i64, i32, vp]
        L.bi8_quantize_colwise.argtypes = [vp, i32, i64, vp, vp, i64, i64, i32, vp]
        L.bi8_quantize_dual.argtypes = [vp, i32, i64, vp, vp, vp, vp, i64, i64, i32, vp]
        L.bi8_dequantize_rowwise.argtypes = [vp, vp, vp, i32, i64, i64, i32, vp]
        L.bi8_peer_allreduce_buffer_bytes.argtypes = [i32, i64]
        L.bi8_peer_allreduce_buffer_bytes.restype = sz
        L.bi8_row_parallel_linear.argtypes = [vp, i32, i64, vp, vp, vp, i64, vp, vp, i64, i64, i64, i32, vp, sz, c.POINTER(vp), i32, i32,
                                              i64, vp, i32, vp, i32, c.c_uint, i32, vp]
        L.bi8_row_parallel_linear_pre.argtypes = [i32, vp, vp, i32, i64, vp, c.c_float, vp, vp, vp, i64, vp, vp, i64, i64, i64, i32, vp, sz,
                                                  c.POINTER(vp), i32, i32, i64, vp, i32, vp, i32, c.c_uint, i32, vp]
        L.bi8_peer_allreduce_large.argtypes = [c.POINTER(vp), i32, i32, i64, i64, i64, vp, i32, i32, c.c_uint, vp]
        L.bi8_peer_allreduce_large_buffer_bytes.argtypes = [i32, i64]
        L.bi8_peer_allreduce_large_buffer_bytes.restype = sz
        L.bi8_peer_allreduce_large_partial_offset.argtypes = []
        L.bi8_peer_allreduce_large_partial_offset.restype = sz
        L.bi8_peer_allreduce_large_out_offset.argtypes = [i64]
        L.bi8_peer_allreduce_large_out_offset.restype = sz
        L.bi8_rope_cache_append.argtypes = [vp, i32, vp, vp, vp, vp, vp, i64, i64, i64, i64, vp]
        L.bi8_peer_allreduce.argtypes = [c.POINTER(vp), i32, i32, i64, vp, i64, i64, vp, i32, vp, i32, c.c_uint, vp]
        L.bi8_gemm_dequant.argtypes = [vp, i64, vp, i64, vp, vp, vp, i32, vp, i64, i32, i64, i64, i64, i32, vp, sz, i32, vp]
        L.bi8_gemm_workspace_bytes.argtypes = [i64, i64, i64, i32]
        L.bi8_gemm_workspace_bytes.restype = sz
        L.bi8_gemm_block_partials.argtypes = [vp, i64, vp, i64, vp, i64, i64, i64, i32, i32, vp]
        L.bi8_gemm_dequant_fused_quant.argtypes = [vp, i32, i64, vp, vp, vp, i64, vp, vp, i32, vp, i64, i32, i64, i64, i64, i32, vp,
                                                   sz, i32, vp]
        L.bi8_quantize_rowwise_pre.argtypes = [i32, vp, vp, i32, i64, vp, c.c_float, vp, vp, i64, i64, i32, vp]
        L.bi8_gemm_dequant_fused_pre.argtypes = [i32, vp, vp, i32, i64, vp, c.c_float, vp, vp, vp, i64, vp, vp, i32, vp, i64, vp, i64, i32,
                                                 i64, i64, i64, i32, vp, sz, i32, vp]
        L.bi8_gemm_wait_selftest.argtypes = [vp, i64, vp, i64, vp, vp, vp, i64, i32, i64, i64, i64, i32, c.c_uint, i32, vp]
        L.bi8_stream_capture_id.argtypes = [vp, c.POINTER(c.c_ulonglong)]
        L.bi8_mma_peak_probe.argtypes = [i32, c.POINTER(c.c_float), c.POINTER(i32)]
        for name in EXPORTS:
            fn = getattr(L, name)
            if name not in ("bi8_last_error_string", "bi8_gemm_workspace_bytes", "bi8_gemm_static_scratch_bytes",
                            "bi8_peer_allreduce_buffer_bytes", "bi8_peer_allreduce_large_buffer_bytes",
                            "bi8_peer_allreduce_large_partial_offset", "bi8_peer_allreduce_large_out_offset"):
                fn.restype = i32
        _lib = L
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().bi8_last_error_string().decode(errors="replace")
        raise Bi8Error(f"{what} failed with status {status}: {msg}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}: expected bfloat16, float16 or float32") from None


def ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_workspaces: dict = {}       # (device, stream handle) -> buffer, eager launches
_capture_ws: dict = {}       # (device, capture id) -> buffer, launches recorded into the CUDA graph being captured


def _capture_id(stream) -> int:
    cid = ctypes.c_ulonglong(0)
    check(lib().bi8_stream_capture_id(ctypes.c_void_p(stream.cuda_stream), ctypes.byref(cid)), "bi8_stream_capture_id")
    return int(cid.value)


def workspace(device: torch.device, nbytes: int):
    """GEMM workspace of at least ``nbytes`` for (device, current stream), or None for 0 bytes.

    The workspace is scratch for split-K partial results.  Eager launches: one buffer per stream is reused by all GEMMs
    queued on that stream (they run one after the other), which saves an allocator round trip per call; a larger request
    replaces the buffer.  While the stream is being captured, the buffer's address is baked into the CUDA graph, so every
    capture gets a buffer of its own (keyed by the capture's sequence number): two graphs never share scratch and may be
    replayed on different streams.  All GEMMs of one graph share its buffer, which is correct because a graph's kernels
    run in capture order.  The buffer is allocated from the capture's memory pool, which keeps it reserved for the graph's
    lifetime; this module drops its own reference when it sees the next capture (or an eager call)."""
    if nbytes <= 0:
        return None
    stream = torch.cuda.current_stream(device)
    cid = _capture_id(stream) if torch.cuda.is_current_stream_capturing() else 0
    for k in [k for k in _capture_ws if k != (device.index, cid)]:
        del _capture_ws[k]
    table, key = (_capture_ws, (device.index, cid)) if cid else (_workspaces, (device.index, stream.cuda_stream))
    ws = table.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 2 * ws.numel() if ws is not None else 0), dtype=torch.uint8, device=device)
        table[key] = ws
    return ws


def device_status() -> int:
    """Synchronises and returns the device-side status word (0 = clean); raises on a recorded timeout."""
    detail = ctypes.c_int(0)
    rc = lib().bi8_device_status(ctypes.byref(detail))
    check(rc, "bi8_device_status")
    return rc
