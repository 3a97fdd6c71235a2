"""Helpers shared by the GPU parity tests: every comparison is CUDA library result vs CPU oracle."""
import torch

from oracle import blockwise_int8_oracle as O

DEV = "cuda"


def set_config(block, io_dtype=torch.bfloat16):
    import block_linear_config as cfg

    cfg.GROUP_SIZE = block
    cfg.INPUT_OUTPUT_TORCH_TYPE = io_dtype
    cfg.SHARED_EXP_TORCH_TYPE = torch.float32


def assert_clean_device():
    from blockwise_int8_linear_b200 import _lib

    assert _lib.device_status() == 0


def randn_bf16(shape, seed, std=1.0, outliers=0.001):
    return O.synthetic(shape, seed, std=std, outlier_frac=outliers)


def quantized_pair(m, k, n, block, seed, std_w=1.0):
    """CPU-quantized operands (so that the GEMM tests do not depend on the GPU quantizer)."""
    x = randn_bf16((m, k), seed)
    w = randn_bf16((n, k), seed + 1, std=std_w)
    xq, xs = O.quantize(x, block)
    wq, ws = O.quantize(w, block)
    return xq, xs, wq, ws


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in units of bf16 steps between two bf16 tensors (monotone integer mapping of the bit patterns)."""
    def key(t):
        i = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return (key(a) - key(b)).abs()
