"""Single-kernel timings of the library (CUDA events, L2 flushed before every launch).

    python -m blockwise_int8_linear_b200.microbench quantize 8192 8192
    python -m blockwise_int8_linear_b200.microbench dequantize 8192 8192
    python -m blockwise_int8_linear_b200.microbench colwise 8192 8192
    python -m blockwise_int8_linear_b200.microbench rmsnorm 4096 4096             # normalise + quantize in one kernel
    python -m blockwise_int8_linear_b200.microbench silu_mul 4096 11008           # silu(gate) * up + quantize in one kernel
    python -m blockwise_int8_linear_b200.microbench gemm 4096 4096 11008          # M K N, int8 operands given
    python -m blockwise_int8_linear_b200.microbench gemm 16 4096 4096 --block 64

One kernel and a few launches per invocation, so the command is also suitable for a profiler capture.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["quantize", "dequantize", "colwise", "dual", "rmsnorm", "silu_mul", "gemm"])
    ap.add_argument("dims", type=int, nargs="+")
    ap.add_argument("--block", type=int, default=64)
    ap.add_argument("--reps", type=int, default=7)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--flags", type=int, default=0, help="GEMM kernel selection flags (BI8_GEMM_* in include/bi8.h)")
    a = ap.parse_args()
    from blockwise_int8_linear_b200 import block_linear_config as cfg
    from blockwise_int8_linear_b200 import triton_functions as F

    cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE = a.block, torch.bfloat16
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(1)
    if a.op == "gemm":
        m, k, n = a.dims
        nb = -(k // -a.block)
        xq = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev, generator=g)
        wq = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev, generator=g)
        xs = torch.rand((nb, m), device=dev, generator=g) + 0.5
        ws = torch.rand((nb, n), device=dev, generator=g) + 0.5
        fn = lambda: F.int8_matmul_block64_rowwise_dequantize(xq, wq.t(), xs, ws, flags=a.flags)
        work = 2.0 * m * n * k
        nbytes = m * k + n * k + 4 * (m + n) * nb + 2 * m * n
    else:
        m, k = a.dims
        x = torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16)
        q, s = F.quantize_block_rowwise(x)
        gu = torch.randn((m, 2 * k), device=dev, generator=g).to(torch.bfloat16) if a.op == "silu_mul" else None
        fn = {"quantize": lambda: F.quantize_block_rowwise(x), "dequantize": lambda: F.dequantize_block_rowwise(q, s),
              "colwise": lambda: F.quantize_block_colwise(x), "dual": lambda: F.quantize_block_dual(x),
              "rmsnorm": lambda: F.rmsnorm_quantize_block_rowwise(x),
              "silu_mul": lambda: F.silu_mul_quantize_block_rowwise(gu[:, :k], gu[:, k:])}[a.op]
        work = 0.0
        nbytes = m * k * ((4 if a.op == "silu_mul" else 2) + (2 if a.op == "dual" else 1) * (1 + 4.0 / a.block))
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(a.warmup):
        fn()
    ts = []
    for _ in range(a.reps):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    ms = ts[len(ts) // 2]
    line = f"{a.op} {a.dims} block {a.block}: median {ms * 1e3:.1f} us over {a.reps} launches, {nbytes / ms / 1e6:.0f} GB/s algorithmic"
    if work:
        line += f", {work / ms / 1e9:.1f} TOP/s"
    print(line)


if __name__ == "__main__":
    main()
