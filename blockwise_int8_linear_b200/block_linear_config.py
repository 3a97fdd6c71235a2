"""Configuration knobs of the blockwise-int8 linear layer.

Mirrors the reference's ``block_linear_config.py:3-5``: three module-level values that
callers change by assignment (``block_linear_config.GROUP_SIZE = 64``).  All three are read
at call time by every operation of this package, so one assignment takes effect everywhere
(the reference froze the GEMM's block size at import, ``triton_functions.py:30,43-56``, which
let the quantizer and the GEMM disagree after a later assignment).

Three more knobs belong to this package alone (the reference keeps the floating-point weight in eval mode,
re-quantizes the weight in every training call and quantizes X and G twice each, once per blocking,
``block_linear.py:78-79,92-94,100-103,125-128``).  The first two default to the reference's behaviour; the third changes no
result (the fused quantizer is bit-identical to the two separate ones) and is on.
"""
import torch

GROUP_SIZE = 128                              # elements per quantisation block along the contraction axis
SHARED_EXP_TORCH_TYPE = torch.float32         # dtype of the block scales; only float32 is supported
INPUT_OUTPUT_TORCH_TYPE = torch.bfloat16      # dtype of GEMM / dequantize outputs: bfloat16, float16 or float32
DROP_WEIGHT_IN_EVAL = False                   # prepare_for_eval() releases the floating-point weight (int8-resident inference)
CACHE_QUANTIZED_WEIGHTS = False               # training: keep both int8 blockings of a weight until the weight changes
FUSE_DUAL_QUANTIZE = True                     # training: read X and G once for their row-wise and column-wise quantizations
