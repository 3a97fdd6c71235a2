"""ctypes front-end of the plain-C restatement (bi8_oracle.c).  TEST INFRASTRUCTURE ONLY.

``build()`` compiles ``libbi8_oracle.so`` next to this file with the Makefile;
the functions take and return CPU torch tensors.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libbi8_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "bi8_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libbi8_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
    return _lib


def _p(t: torch.Tensor):
    return ctypes.c_void_p(t.data_ptr())


def _dt(dtype) -> int:
    if dtype == torch.bfloat16:
        return 0
    if dtype == torch.float32:
        return 1
    raise ValueError(f"C oracle handles bf16 and fp32, not {dtype}")


def quantize(x: torch.Tensor, block: int):
    x = x.contiguous()
    m, k = x.shape
    nb = -(k // -block)
    q = torch.empty((m, k), dtype=torch.int8)
    s = torch.empty((nb, m), dtype=torch.float32)
    _load().bi8o_quantize_rowwise(_p(x), _dt(x.dtype), _p(q), _p(s), ctypes.c_long(m), ctypes.c_long(k),
                                  ctypes.c_long(block))
    return q, s


def dequantize(q: torch.Tensor, s: torch.Tensor, block: int, out_dtype=torch.bfloat16):
    q = q.contiguous()
    s = s.contiguous()
    m, k = q.shape
    out = torch.empty((m, k), dtype=out_dtype)
    _load().bi8o_dequantize_rowwise(_p(q), _p(s), _p(out), _dt(out_dtype), ctypes.c_long(m), ctypes.c_long(k),
                                    ctypes.c_long(block))
    return out


def gemm_acc(a: torch.Tensor, bt: torch.Tensor, sx: torch.Tensor, sw: torch.Tensor, block: int):
    """a [M,K] int8, bt [N,K] int8 (row-major; the GEMM's B operand is bt.t())."""
    a = a.contiguous()
    bt = bt.contiguous()
    m, k = a.shape
    n = bt.shape[0]
    acc = torch.empty((m, n), dtype=torch.float32)
    _load().bi8o_gemm_acc(_p(a), _p(bt), _p(sx.contiguous()), _p(sw.contiguous()), _p(acc), ctypes.c_long(m),
                          ctypes.c_long(n), ctypes.c_long(k), ctypes.c_long(block))
    return acc


def gemm_partials(a: torch.Tensor, bt: torch.Tensor, block: int):
    a = a.contiguous()
    bt = bt.contiguous()
    m, k = a.shape
    n = bt.shape[0]
    nb = -(k // -block)
    out = torch.empty((nb, m, n), dtype=torch.int32)
    _load().bi8o_gemm_partials(_p(a), _p(bt), _p(out), ctypes.c_long(m), ctypes.c_long(n), ctypes.c_long(k),
                               ctypes.c_long(block))
    return out
