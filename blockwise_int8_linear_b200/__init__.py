"""Blockwise-int8 linear layer for NVIDIA B200 (sm_100a): hand-written CUDA kernels behind the
reference project's Python interface.  See ``include/bi8.h`` for the C ABI underneath."""
from . import block_linear_config
from .block_linear import (BlockInt8Linear, BlockLinear, BlockLinearConfig, blockwise_int8_linear, fast_matmul,
                           replace_linear_with_blockwise_int8)
from .triton_functions import (dequantize_block_rowwise, fast_matmulT, int8_matmul_block64_rowwise_dequantize,
                               int8_matmul_block_partials, quantize_block_colwise, quantize_block_rowwise)

__all__ = [
    "block_linear_config", "BlockInt8Linear", "BlockLinear", "BlockLinearConfig", "blockwise_int8_linear", "fast_matmul",
    "fast_matmulT", "replace_linear_with_blockwise_int8", "quantize_block_rowwise", "quantize_block_colwise",
    "dequantize_block_rowwise", "int8_matmul_block64_rowwise_dequantize", "int8_matmul_block_partials",
]
