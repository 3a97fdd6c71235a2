"""Host-side checks that need no GPU: the library loads, exports what the header declares, validates its
arguments before touching CUDA, and the Python surface mirrors the reference's names."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from blockwise_int8_linear_b200 import build, _lib
    build.build()
    return _lib.lib()


def test_library_exports_every_declared_symbol(L):
    header = open(os.path.join(ROOT, "include", "bi8.h")).read()
    declared = sorted(set(re.findall(r"BI8_API[^;]*?\b(bi8_\w+)\s*\(", header)))
    assert len(declared) >= 13
    for name in declared:
        assert hasattr(L, name), name
    from blockwise_int8_linear_b200 import _lib
    assert sorted(_lib.EXPORTS) == declared
    assert L.bi8_version() == 100


def test_argument_validation_happens_before_cuda(L):
    vp = ctypes.c_void_p
    one = vp(256)          # a non-null, aligned, never dereferenced address
    err = lambda: L.bi8_last_error_string().decode()
    assert L.bi8_quantize_rowwise(one, 7, 64, one, one, 4, 64, 64, None) == -1 and "dtype" in err()
    assert L.bi8_quantize_rowwise(one, 0, 64, one, one, 4, 64, 0, None) == -2
    assert L.bi8_quantize_rowwise(one, 0, 32, one, one, 4, 64, 64, None) == -4      # pitch < K
    assert L.bi8_quantize_rowwise(None, 0, 64, one, one, 4, 64, 64, None) == -8
    assert L.bi8_quantize_rowwise(vp(257), 0, 64, one, one, 4, 64, 64, None) == -3
    assert L.bi8_quantize_rowwise(None, 0, 64, None, None, 0, 64, 64, None) == 0      # empty: nothing to do
    assert L.bi8_quantize_colwise(one, 0, 8, one, one, 4, 64, 64, None) == -4
    assert L.bi8_dequantize_rowwise(one, one, one, 9, 4, 64, 64, None) == -1
    assert L.bi8_dequantize_rowwise(one, one, None, 0, 4, 64, 64, None) == -8
    g = lambda **kw: L.bi8_gemm_dequant(kw.get("A", one), kw.get("lda", 64), one, 64, one, one, None, 0, kw.get("C", one),
                                        kw.get("ldc", 64), kw.get("dt", 0), kw.get("M", 8), 64, 64, kw.get("block", 64),
                                        None, 0, 0, None)
    assert g(M=-1) == -4
    assert g(block=0) == -2
    assert g(A=None) == -8
    assert g(lda=8) == -4
    assert g(dt=5) == -1
    assert g(C=None) == -8
    assert g(ldc=8) == -4
    assert g(M=0) == 0
    assert L.bi8_gemm_workspace_bytes(128, 128, 128, 64) == 0


def test_fused_entry_point_validates_and_flags_match_the_header(L):
    from blockwise_int8_linear_b200 import _lib
    header = open(os.path.join(ROOT, "include", "bi8.h")).read()
    flags = {name: int(value) for name, value in re.findall(r"#define BI8_GEMM_(\w+)\s+(\d+)", header)}
    assert flags == {"DEFAULT": 0, "FORCE_GENERIC": 1, "FORCE_TC": 2, "NO_SEED": 4, "FORCE_SMALLM": 8, "FORCE_SKINNY": 16,
                     "QUANT_IN_KERNEL": 32}
    assert (_lib.GEMM_FORCE_GENERIC, _lib.GEMM_FORCE_TC, _lib.GEMM_NO_SEED, _lib.GEMM_FORCE_SMALLM, _lib.GEMM_FORCE_SKINNY,
            _lib.GEMM_QUANT_IN_KERNEL) == (1, 2, 4, 8, 16, 32)
    vp = ctypes.c_void_p
    one = vp(256)
    f = lambda **kw: L.bi8_gemm_dequant_fused_quant(one, kw.get("xdt", 0), 64, kw.get("xq", one), kw.get("sx", one), one, 64, one,
                                                    None, 0, one, 64, 0, kw.get("M", 8), 64, 64, 64, None, 0, 0, None)
    assert f(xdt=9) == -1
    # without a GPU (or a workspace) the one-kernel form does not apply, so the scratch is required
    assert f(xq=None) == -7 and "scratch" in L.bi8_last_error_string().decode()
    assert f(M=0) == 0


def test_new_entry_points_validate_before_cuda(L):
    """The entry points around the layer (fused producer steps, residual, prefill-sized peer sum, rotary/cache helper):
    every argument check runs before the first CUDA call, so it can be exercised without a GPU."""
    from blockwise_int8_linear_b200 import _lib
    header = open(os.path.join(ROOT, "include", "bi8.h")).read()
    pre = {name: int(value) for name, value in re.findall(r"#define BI8_PRE_(\w+)\s+(\d+)", header)}
    assert pre == {"NONE": 0, "RMSNORM": 1, "SILU_MUL": 2}
    assert (_lib.PRE_NONE, _lib.PRE_RMSNORM, _lib.PRE_SILU_MUL) == (0, 1, 2)
    assert int(re.search(r"#define BI8_ADDEND_FULL\s+(0x[0-9a-fA-F]+)", header).group(1), 16) == _lib.ADDEND_FULL
    vp = ctypes.c_void_p
    one = vp(256)
    err = lambda: L.bi8_last_error_string().decode()
    q = lambda **kw: L.bi8_quantize_rowwise_pre(kw.get("op", 1), kw.get("x", one), kw.get("x2", None), kw.get("dt", 0), kw.get("ldx", 64),
                                                None, 1e-5, one, one, kw.get("M", 4), 64, 64, None)
    assert q(dt=9) == -1
    assert q(op=5) == -4 and "operation" in err()
    assert q(ldx=8) == -4
    assert q(x=None) == -8
    assert q(op=2) == -8                                   # the gated activation needs its second operand
    assert q(x=vp(257)) == -3
    assert q(M=0) == 0
    f = lambda **kw: L.bi8_gemm_dequant_fused_pre(kw.get("op", 1), one, None, 0, 64, None, 1e-5, kw.get("xq", one), one, one, 64, one,
                                                  None, 0, kw.get("res", None), kw.get("ldr", 64), kw.get("C", one), 64, kw.get("dt", 0),
                                                  kw.get("M", 8), 64, 64, 64, None, 0, 0, None)
    assert f(xq=None) == -7
    assert f(res=one, ldr=8) == -4
    assert f(dt=7) == -1
    assert f(res=vp(257)) == -3
    assert f(res=vp(256 + 64), C=vp(256)) == -4 and "overlap" in err()      # overlapping, not the same tensor
    assert f(M=0) == 0
    assert L.bi8_peer_allreduce_large_buffer_bytes(2, 1000) == 0            # capacity must be a multiple of 1024
    assert L.bi8_peer_allreduce_large_buffer_bytes(9, 1024) == 0
    n = L.bi8_peer_allreduce_large_buffer_bytes(2, 4096)
    assert n == L.bi8_peer_allreduce_large_out_offset(4096) + 4 * 4096
    assert L.bi8_peer_allreduce_large_out_offset(4096) == L.bi8_peer_allreduce_large_partial_offset() + 4 * 4096
    bufs = (vp * 8)(*([256] * 8))
    big = lambda **kw: L.bi8_peer_allreduce_large(bufs, kw.get("rank", 0), kw.get("world", 2), kw.get("cap", 4096), kw.get("M", 4),
                                                  kw.get("N", 64), None, 0, kw.get("dt", 0), 0, None)
    assert big(dt=9) == -1
    assert big(rank=2) == -4
    assert big(cap=1000) == -4
    assert big(N=6) == -4                                  # N a multiple of 4
    assert big(M=100) == -4                                # does not fit the capacity
    r = lambda **kw: L.bi8_rope_cache_append(kw.get("qkv", one), kw.get("dt", 0), one, one, one, one, one, kw.get("B", 2), 4,
                                             kw.get("D", 64), kw.get("max_len", 16), None)
    assert r(dt=1) == -1                                   # 16-bit activations only
    assert r(D=63) == -4
    assert r(max_len=0) == -4
    assert r(qkv=None) == -8
    assert r(qkv=vp(258)) == -3
    assert r(B=0) == 0


def test_python_surface_mirrors_reference_names():
    import block_linear
    import block_linear_config
    import triton_functions
    import blockwise_int8_linear_b200 as pkg

    assert block_linear_config is pkg.block_linear_config
    for name in ("quantize_block_rowwise", "dequantize_block_rowwise", "int8_matmul_block64_rowwise_dequantize",
                 "fast_matmulT", "ceil_div"):
        assert callable(getattr(triton_functions, name))
    for name in ("replace_linear_with_blockwise_int8", "fast_matmul", "blockwise_int8_linear", "BlockInt8Linear"):
        assert hasattr(block_linear, name)
    # additions without a counterpart in the reference
    for name in ("quantize_block_colwise", "quantize_block_dual", "quantize_matmul_block_rowwise_dequantize",
                 "rmsnorm_quantize_block_rowwise", "silu_mul_quantize_block_rowwise", "pre_quantize_matmul_block_rowwise_dequantize"):
        assert callable(getattr(triton_functions, name))
    assert callable(block_linear.BlockInt8Linear.infer_pre)
    from blockwise_int8_linear_b200 import decode_ops, peer
    assert callable(decode_ops.rope_cache_append) and hasattr(peer, "PeerAllReduce") and hasattr(peer, "PeerAllReduceLarge")
    assert block_linear.BlockLinear is block_linear.BlockInt8Linear
    assert issubclass(block_linear.BlockInt8Linear, torch.nn.Linear)
    # defaults of the reference (block_linear_config.py:3-5)
    import importlib
    fresh = importlib.reload(block_linear_config)
    assert fresh.GROUP_SIZE == 128 and fresh.SHARED_EXP_TORCH_TYPE == torch.float32
    assert fresh.INPUT_OUTPUT_TORCH_TYPE == torch.bfloat16


def test_config_knobs_are_read_at_call_time():
    import block_linear_config as cfg
    from blockwise_int8_linear_b200.block_linear import BlockLinearConfig
    from blockwise_int8_linear_b200 import triton_functions as tf

    old = cfg.GROUP_SIZE
    cfg.GROUP_SIZE = 64
    assert tf._block() == 64 and tf._block(32) == 32
    with BlockLinearConfig(group_size=32, io_dtype=torch.float32) as c:
        assert cfg.GROUP_SIZE == 32 and c.group_size == 32 and cfg.INPUT_OUTPUT_TORCH_TYPE == torch.float32
    assert cfg.GROUP_SIZE == 64 and cfg.INPUT_OUTPUT_TORCH_TYPE == torch.bfloat16
    cfg.SHARED_EXP_TORCH_TYPE = torch.float16
    with pytest.raises(ValueError):
        tf._scale_dtype()
    cfg.SHARED_EXP_TORCH_TYPE = torch.float32
    cfg.GROUP_SIZE = old


def test_cpu_tensors_are_rejected_like_the_reference():
    import triton_functions as tf
    with pytest.raises(AssertionError):
        tf.quantize_block_rowwise(torch.zeros(4, 64, dtype=torch.bfloat16))
    with pytest.raises(AssertionError):
        tf.dequantize_block_rowwise(torch.zeros(4, 64, dtype=torch.int8), torch.zeros(1, 4))


def test_replace_linear_on_cpu_module_structure():
    import torch.nn as nn
    from block_linear import BlockInt8Linear, replace_linear_with_blockwise_int8

    m = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4, bias=False))
    w0 = m[0].weight.data_ptr()
    replace_linear_with_blockwise_int8(m)
    assert isinstance(m[0], BlockInt8Linear) and isinstance(m[2], BlockInt8Linear)
    assert m[0].weight.data_ptr() == w0 and m[2].bias is None
    assert m[0].in_features == 8 and m[0].out_features == 16 and tuple(m[0].weight.shape) == (16, 8)


def test_product_code_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "blockwise_int8_linear_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, f"{f} mentions the oracle"
