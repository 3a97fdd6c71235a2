"""Benchmark of the blockwise-int8 linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one forward of the layer on one batch: block-quantize the bf16 activations
(x [M, K]) and run the int8 block GEMM with fused dequantize against pre-quantized weights
(W [N, K]) into a bf16 output.  The default workload is the largest Llama-2-7B projection of
the benchmark configuration (M = 8192 tokens, K = 4096, N = 11008, block 64); the metric is the
reference's own (``triton_functions.py:565``): 2*M*N*K / time, in tera-ops per second.

With N > 1 (launched by torchrun, one rank per GPU) every rank runs the same step on its own
batch of tokens: the layer is data-parallel in the token dimension, there is no collective on the
path, so scaling is weak and ``value`` is the sum over ranks divided by the slowest rank's time.
The partitionings that do communicate are measured beside it at the same N (``roofline.tp``,
``roofline.models``): the Llama MLP pair sharded column-/row-parallel with its NCCL all-reduce and with the
library's own peer-memory sums in its place (``peer_reduce``, ``peer_reduce_fused`` for decode, ``peer_reduce_large``
for prefill), the Llama-architecture inference driver (tensor parallel) and the GPT-2 training driver (data parallel).

Prints ONE JSON line.  Besides the headline it carries
  roofline      the GEMM kernel alone (CUDA events around its launches inside the timed region), and inside it
                kernels (memory-bound kernels and the small-M GEMM rows against the HBM roof), sustained (the GEMM
                back to back for two seconds), cublas_bf16_ms (torch.matmul on the same shape, comparator only),
                fused_producers (the quantizers with RMSNorm / SiLU*mul fused in front and the residual sum behind,
                against the separate kernels), tp and models (see above)
  e2e           the same step through the public Python API with host buffers (pinned H2D of x, D2H of y)
  cpu_baseline  the CPU restatement of the reference timed on this host on a bounded sample (rank 0, N = 1)
  extra         the full sweep tables the rows in roofline.kernels are taken from
``--impl reference`` times the CPU restatement only (the reference has no CPU path of its own and
cannot be imported without a GPU and Triton 2.3; the restatement is pinned to its kernels by golden vectors).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

BLOCK = 64
WORKLOADS = {
    # name: (M, K, N)
    "llama7b_up_proj_m8192": (8192, 4096, 11008),
    "llama7b_attn_proj_m8192": (8192, 4096, 4096),
    "llama7b_down_proj_m8192": (8192, 11008, 4096),
    "llama7b_up_proj_m2048": (2048, 4096, 11008),
}
DEFAULT_WORKLOAD = "llama7b_up_proj_m8192"
INT8_NOMINAL_TOPS = 4500.0
NSETS = 3            # rotating input/output sets of the timed step
HBM_FALLBACK, BF16_FALLBACK = 6650.0, 1590.0


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return HBM_FALLBACK, BF16_FALLBACK, "fallback"


def ncu_traffic(key: str):
    p = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    if os.path.exists(p):
        return json.load(open(p)).get(key)
    return None


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.rows = []          # (arrival time, fields) of every sample line, appended by the reader thread
        self.thread = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [x.strip() for x in line.split(",")]))

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "25", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True, bufsize=1)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def count_since(self, t0: float) -> int:
        return sum(1 for t, f in list(self.rows) if t >= t0 and len(f) >= 9)

    def stop(self, since: float = None):
        """Summary of the samples that arrived from `since` (a time.perf_counter() value) on; all of them without it."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        if since is None:
            time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t_arr, f in list(self.rows):
            if len(f) < 9 or (since is not None and t_arr < since):
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def bench_config(workload: str, world: int):
    """The `config` object of the JSON line; both arms print the same one."""
    M, K, N = WORKLOADS[workload]
    return {"workload": workload, "M_per_gpu": M, "K": K, "N": N, "block": BLOCK, "in": "bf16", "out": "bf16",
            "step": "block-quantize x + int8 block GEMM with fused dequantize (weights pre-quantized)",
            "l2": f"{NSETS} rotating input/output sets of {(M * K * 2 + M * N * 2) >> 20} MiB each (larger than L2)",
            "parallelism": f"dp{world} over tokens, no collective"}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ---------------------------------------------------------------------------------------------------------
# CPU restatement (reference arm and cpu_baseline)
# ---------------------------------------------------------------------------------------------------------
def cpu_step(O, x, wq, ws):
    xq, xs = O.quantize(x, BLOCK)
    return O.gemm(xq, wq.t(), xs, ws, None, BLOCK, torch.bfloat16)


def cpu_baseline(workload: str, budget_s: float = 12.0):
    """Times the CPU restatement on a bounded row sample of the workload; returns the cpu_baseline object."""
    from oracle import blockwise_int8_oracle as O
    M, K, N = WORKLOADS[workload]
    torch.set_num_threads(os.cpu_count() or 1)
    w = O.synthetic((N, K), 3100, std=0.02, outlier_frac=0.0)
    wq, ws = O.quantize(w, BLOCK)
    x = O.synthetic((256, K), 3000, outlier_frac=0.0)
    cpu_step(O, x[:64], wq, ws)                  # warm the thread pool
    t0 = time.perf_counter()
    cpu_step(O, x, wq, ws)
    t256 = time.perf_counter() - t0
    rows = int(max(64, min(M, 256 * budget_s / max(t256, 1e-3) / 2)))
    rows -= rows % 64
    x = O.synthetic((rows, K), 3001, outlier_frac=0.0)
    cpu_step(O, x, wq, ws)                       # warm
    t0 = time.perf_counter()
    cpu_step(O, x, wq, ws)
    dt = time.perf_counter() - t0
    tops = 2.0 * rows * N * K / dt / 1e12
    return {"value": tops, "unit": "TOP/s", "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(),
            "kind": "port", "sample": f"{rows} of {M} rows of {workload} (quantize x + block GEMM, weights pre-quantized), "
                                      f"{dt:.2f} s, torch CPU fp32 restatement"}, rows


def run_reference(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from oracle import blockwise_int8_oracle as O
    M, K, N = WORKLOADS[args.workload]
    torch.set_num_threads(os.cpu_count() or 1)
    w = O.synthetic((N, K), 3100, std=0.02, outlier_frac=0.0)
    wq, ws = O.quantize(w, BLOCK)
    # one step is the whole batch when warmup + steps of it fit in about 200 s, else a bounded row sample
    x = O.synthetic((256, K), 3000, outlier_frac=0.0)
    cpu_step(O, x[:64], wq, ws)                  # warm the thread pool
    t0 = time.perf_counter()
    cpu_step(O, x, wq, ws)
    t256 = time.perf_counter() - t0
    budget = 200.0 / max(1, args.steps + args.warmup)
    rows = int(max(64, min(M, 256 * budget / max(t256, 1e-3))))
    rows -= rows % 64
    x = O.synthetic((rows, K), 3001, outlier_frac=0.0)
    for _ in range(args.warmup):
        cpu_step(O, x, wq, ws)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(O, x, wq, ws)
    dt = (time.perf_counter() - t0) / args.steps
    tops = 2.0 * rows * N * K / dt / 1e12
    sample = (f"{rows} of {M} rows per step of {args.workload} (throughput does not depend on the row count); torch CPU fp32 "
              f"restatement of the reference kernels")
    line = {
        "impl": "reference", "metric": "int8_block_gemm_tops", "value": tops, "unit": "TOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": bench_config(args.workload, args.gpus),
        "cpu_baseline": {"value": tops, "unit": "TOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "rows_per_step": rows,
        "note": "the reference has no CPU implementation (its wrappers assert CUDA tensors); this arm times the CPU "
                "restatement that the golden vectors pin to the reference's kernels",
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------
def time_kernel(fn, reps: int, flush) -> float:
    """Median milliseconds of fn() over reps launches, L2 flushed before each (the flush is not timed)."""
    ts = []
    for _ in range(reps):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def time_graph(fn, reps: int) -> float:
    """Median milliseconds per launch of fn(i), i = 0..reps-1, captured once in a CUDA graph and replayed 5 times.
    The caller rotates its inputs over more bytes than L2 holds, so every launch starts cold; nothing but the launches is
    on the stream, so neither the host nor a flush kernel's dirty lines sit inside the timed region."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(reps):
            fn(i)
    ts = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b) / reps)
    ts.sort()
    del graph
    return ts[len(ts) // 2]


def extras(dev, hbm_gbs, flush):
    """Memory-bound kernels (quantize / dequantize sweep) and the other GEMM shapes, cold L2.

    "us" comes from CUDA-graph replays over rotating inputs that together exceed L2 (time_graph); "us_flushed" from events
    around single eager launches behind a 256 MB fill (time_kernel), which adds the launch latency and the write-back of
    the fill's dirty lines to a kernel of a few tens of microseconds."""
    import block_linear_config as cfg
    from triton_functions import (dequantize_block_rowwise, int8_matmul_block64_rowwise_dequantize,
                                  quantize_block_colwise, quantize_block_dual, quantize_block_rowwise,
                                  quantize_matmul_block_rowwise_dequantize)
    cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE = BLOCK, torch.bfloat16
    out = {"quantize": [], "dequantize": [], "quantize_colwise": [], "quantize_dual": [], "gemm": []}
    for n in (4096, 8192, 16384):
        copies = max(2, -(-(300 << 20) // (n * n * 2)) + 1)
        xs, qs, ss = [], [], []
        for c in range(copies):
            g = torch.Generator(device=dev).manual_seed(2000 + n + c)
            x = torch.randn((n, n), device=dev, dtype=torch.float32, generator=g)
            x = torch.where(torch.rand((n, n), device=dev, generator=g) < 0.001, x * 20, x).to(torch.bfloat16)
            q, s = quantize_block_rowwise(x)
            xs.append(x)
            qs.append(q)
            ss.append(s)
        nbytes = n * n * (2 + 1 + 4 / BLOCK)
        reps = 2 * copies
        # the dual quantizer reads the input once and writes both int8 results: 2 + 2 * (1 + 4/block) bytes per element
        dual_bytes = n * n * (2 + 2 * (1 + 4 / BLOCK))
        for key, fn, nb_ in (("quantize", lambda i: quantize_block_rowwise(xs[i % copies]), nbytes),
                             ("dequantize", lambda i: dequantize_block_rowwise(qs[i % copies], ss[i % copies]), nbytes),
                             ("quantize_colwise", lambda i: quantize_block_colwise(xs[i % copies]), nbytes),
                             ("quantize_dual", lambda i: quantize_block_dual(xs[i % copies]), dual_bytes)):
            ms = time_graph(fn, reps)
            ms_flushed = time_kernel(lambda: fn(0), 7, flush)
            out[key].append({"shape": [n, n], "us": ms * 1e3, "gbs": nb_ / ms / 1e6, "frac_hbm": nb_ / ms / 1e6 / hbm_gbs,
                             "us_flushed": ms_flushed * 1e3, "frac_hbm_flushed": nb_ / ms_flushed / 1e6 / hbm_gbs})
        del xs, qs, ss
    # Llama-7B projection shapes.  "us" times the GEMM on pre-quantized activations, "us_linear" the layer's forward from
    # bf16 activations (quantize + GEMM: for M <= 64 one library call whose kernels overlap).  Launches of a few
    # microseconds are timed as CUDA-graph replays of 16 launches that rotate over enough weight copies to exceed L2
    # (an eager loop would time the host); the large ones with events around one launch after an L2 flush.
    for (k, n) in ((4096, 4096), (4096, 11008), (11008, 4096)):
        copies = max(2, -(-(256 << 20) // (n * k)))
        wqs, wss = [], []
        for c in range(copies):
            w = (torch.randn((n, k), device=dev, generator=torch.Generator(device=dev).manual_seed(n + k + c)) * 0.02).to(torch.bfloat16)
            wq, ws = quantize_block_rowwise(w)
            wqs.append(wq)
            wss.append(ws)
            del w
        for m in (1, 16, 128, 2048, 8192):
            x = torch.randn((m, k), device=dev, generator=torch.Generator(device=dev).manual_seed(m)).to(torch.bfloat16)
            xq, xs = quantize_block_rowwise(x)

            def gemm(i):
                return int8_matmul_block64_rowwise_dequantize(xq, wqs[i % copies].t(), xs, wss[i % copies])

            def linear(i):
                if m <= 64:
                    return quantize_matmul_block_rowwise_dequantize(x, wqs[i % copies].t(), wss[i % copies])
                q, st = quantize_block_rowwise(x)
                return int8_matmul_block64_rowwise_dequantize(q, wqs[i % copies].t(), st, wss[i % copies])

            times = {}
            for name, fn in (("us", gemm), ("us_linear", linear)):
                if m <= 128:
                    times[name] = time_graph(fn, max(16, copies))
                else:
                    for i in range(3):
                        fn(i)
                    times[name] = time_kernel(lambda: fn(0), 7, flush)
            ms = times["us"]
            ops = 2.0 * m * n * k
            nbytes = m * k + n * k + 4 * (m + n) * k / BLOCK + 2 * m * n
            out["gemm"].append({"M": m, "K": k, "N": n, "us": ms * 1e3, "us_linear": times["us_linear"] * 1e3,
                                "timing": "graph replay" if m <= 128 else "events, L2 flushed",
                                "tops": ops / ms / 1e9, "gbs": nbytes / ms / 1e6,
                                "frac_int8_nominal": ops / ms / 1e9 / INT8_NOMINAL_TOPS, "frac_hbm": nbytes / ms / 1e6 / hbm_gbs})
        del wqs, wss
    try:
        out["fused_producers"] = fused_producers(dev, hbm_gbs, flush)
    except Exception as e:                # comparison table only
        out["fused_producers"] = {"error": f"{type(e).__name__}: {e}"}
    return out


def fused_producers(dev, hbm_gbs, flush):
    """The quantizers with the producing elementwise step fused in front, and the layer call with the residual sum fused
    behind, against the same steps as separate kernels: the stand-alone quantizers at M = 4096 (HBM-bound: algorithmic
    bytes = input + int8 + scales) and the MLP half of a Llama-7B layer at M = 8 (rms_norm -> gate_up -> silu * up ->
    down -> residual sum), both forms producing identical tensors except for the last bit of the normalisation."""
    import block_linear_config as cfg
    import torch.nn.functional as F
    from triton_functions import (pre_quantize_matmul_block_rowwise_dequantize as pre_mm, quantize_block_rowwise,
                                  quantize_matmul_block_rowwise_dequantize as q_mm, rmsnorm_quantize_block_rowwise,
                                  silu_mul_quantize_block_rowwise)
    cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE = BLOCK, torch.bfloat16
    res = {"quantizers": [], "mlp_half_decode": None}
    m, h, f = 4096, 4096, 11008
    g = torch.Generator(device=dev).manual_seed(77)
    copies = 5                                                   # 5 x (32 + 180) MB of inputs: larger than L2
    xs = [torch.randn((m, h), device=dev, generator=g).to(torch.bfloat16) for _ in range(copies)]
    gus = [torch.randn((m, 2 * f), device=dev, generator=g).to(torch.bfloat16) for _ in range(copies)]
    rows = (("rmsnorm_quantize", lambda i: rmsnorm_quantize_block_rowwise(xs[i % copies]),
             lambda i: quantize_block_rowwise(F.rms_norm(xs[i % copies], (h,), eps=1e-5)), m * h * (2 + 1 + 4 / BLOCK), [m, h]),
            ("silu_mul_quantize", lambda i: silu_mul_quantize_block_rowwise(gus[i % copies][:, :f], gus[i % copies][:, f:]),
             lambda i: quantize_block_rowwise(F.silu(gus[i % copies][:, :f]) * gus[i % copies][:, f:]), m * f * (4 + 1 + 4 / BLOCK), [m, f]))
    for name, fused, separate, nbytes, shape in rows:
        ms_f, ms_s = time_graph(fused, 2 * copies), time_graph(separate, 2 * copies)
        res["quantizers"].append({"name": name, "shape": shape, "us": ms_f * 1e3, "frac_hbm": nbytes / ms_f / 1e6 / hbm_gbs,
                                  "us_separate_kernels": ms_s * 1e3})
    del xs, gus
    m = 8
    wcopies = 3                                                  # 3 x 135 MB of weights
    gate_up, down = [], []
    for c in range(wcopies):
        w1 = (torch.randn((2 * f, h), device=dev, generator=g) * 0.02).to(torch.bfloat16)
        w2 = (torch.randn((h, f), device=dev, generator=g) * 0.02).to(torch.bfloat16)
        gate_up.append(quantize_block_rowwise(w1))
        down.append(quantize_block_rowwise(w2))
        del w1, w2
    x = torch.randn((m, h), device=dev, generator=g).to(torch.bfloat16)

    def separate(i):
        (w1, s1), (w2, s2) = gate_up[i % wcopies], down[i % wcopies]
        gu = q_mm(F.rms_norm(x, (h,), eps=1e-5), w1.t(), s1)
        return x + q_mm(F.silu(gu[:, :f]) * gu[:, f:], w2.t(), s2)

    def fused(i):
        (w1, s1), (w2, s2) = gate_up[i % wcopies], down[i % wcopies]
        gu = pre_mm("rmsnorm", x, w1.t(), s1, eps=1e-5)
        return pre_mm("silu_mul", gu[:, :f], w2.t(), s2, x2=gu[:, f:], residual=x)

    ms_f, ms_s = time_graph(fused, 12), time_graph(separate, 12)
    res["mlp_half_decode"] = {"M": m, "us": ms_f * 1e3, "us_separate_kernels": ms_s * 1e3, "launches": "6 against 10",
                              "timing": "CUDA-graph replays of 12 calls rotating over 3 weight copies (405 MB)"}
    return res


def kernel_rows(extra, hbm_gbs):
    """The rows of the sweep that stand against the HBM roof (quantizers, dequantizer, GEMM with M <= 128) and the
    tensor-bound GEMM rows, in the compact form kept under roofline.kernels."""
    rows = []
    for key, name in (("quantize", "quantize_rowwise"), ("quantize_colwise", "quantize_colwise"), ("dequantize", "dequantize_rowwise")):
        for r in extra.get(key, []):
            rows.append({"name": name, "shape": r["shape"], "us": round(r["us"], 2), "bound": "hbm", "frac": round(r["frac_hbm"], 3)})
    for r in extra.get("quantize_dual", []):
        rows.append({"name": "quantize_dual", "shape": r["shape"], "us": round(r["us"], 2), "bound": "hbm", "frac": round(r["frac_hbm"], 3)})
    fp = extra.get("fused_producers") or {}
    for r in fp.get("quantizers", []) if isinstance(fp, dict) else []:
        rows.append({"name": r["name"], "shape": r["shape"], "us": round(r["us"], 2), "bound": "hbm", "frac": round(r["frac_hbm"], 3)})
    for r in extra.get("gemm", []):
        hbm_bound = r["M"] <= 128
        rows.append({"name": "gemm", "shape": [r["M"], r["K"], r["N"]], "us": round(r["us"], 2), "bound": "hbm" if hbm_bound else "tensor",
                     "frac": round(r["frac_hbm"] if hbm_bound else r["frac_int8_nominal"], 3)})
    return rows


def k512_sweep(dev, flush):
    """The reference's own benchmark protocol (triton_functions.py:521-567): square M = N in 2048 .. 14336, K = 512,
    providers cuBLAS bf16 (torch.matmul), blockwise_int8 (the GEMM on pre-quantized operands) and blockwise_int8_quantise
    (both quantizers + the GEMM), in TFLOP/s = 2*M*N*K / t.  Events around one launch behind an L2 flush, median of 7."""
    import block_linear_config as cfg
    from triton_functions import int8_matmul_block64_rowwise_dequantize as mm, quantize_block_rowwise as qr
    cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE = BLOCK, torch.bfloat16
    rows = []
    K = 512
    for n in range(2048, 16 * 1024, 2048):
        g = torch.Generator(device=dev).manual_seed(n)
        a = torch.randn((n, K), device=dev, generator=g).to(torch.bfloat16)
        bt = torch.randn((n, K), device=dev, generator=g).to(torch.bfloat16)      # the reference's b.t().contiguous()
        aq, sa = qr(a)
        bq, sb = qr(bt)

        def quantise_and_multiply():
            x, sx = qr(a)
            w, sw = qr(bt)
            return mm(x, w.t(), sx, sw)

        ops = 2.0 * n * n * K
        t_cublas = time_kernel(lambda: torch.matmul(a, bt.t()), 7, flush)
        t_gemm = time_kernel(lambda: mm(aq, bq.t(), sa, sb), 7, flush)
        t_all = time_kernel(quantise_and_multiply, 7, flush)
        rows.append({"M": n, "N": n, "K": K, "cublas_bf16_tflops": round(ops / t_cublas / 1e9, 1),
                     "blockwise_int8_tops": round(ops / t_gemm / 1e9, 1), "blockwise_int8_quantise_tops": round(ops / t_all / 1e9, 1)})
        del a, bt, aq, bq
    return rows


def sustained_gemm(step_gemm, ops, local, seconds=2.0):
    """The GEMM back to back for `seconds` with the SM clock sampled: the number a long training or prefill run sees."""
    sampler = ClockSampler(local)
    for _ in range(3):
        step_gemm(0)
    torch.cuda.synchronize()
    sampler.start()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    n = 0
    while True:
        for i in range(50):
            step_gemm(n + i)
        n += 50
        torch.cuda.synchronize()
        if time.perf_counter() - t0 >= seconds:
            break
    e1.record()
    e1.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / n
    return {"seconds": round(time.perf_counter() - t0, 2), "launches": n, "gemm_ms": ms, "tops": ops / ms / 1e9,
            "frac_of_nominal_int8_4500": ops / ms / 1e9 / INT8_NOMINAL_TOPS, "sm_mhz_median": clocks.get("sm_mhz"),
            "reasons": clocks.get("reasons")}


def tp_bench(dev, rank, world, hbm_gbs):
    """The Llama-2-7B MLP pair sharded as blockwise_int8_linear_b200.parallel shards it: column-parallel gate_up
    (2 x 11008 / p output features per rank) -> SiLU * mul -> row-parallel down (block-aligned 11008 / p input features,
    fp32 partial result) -> NCCL all-reduce of [M, 4096] -> cast.  M = 4096 (prefill) and M = 8 (decode)."""
    import torch.distributed as dist
    import torch.nn.functional as F
    import block_linear_config as cfg
    from blockwise_int8_linear_b200.parallel import block_aligned_bounds
    from triton_functions import (int8_matmul_block64_rowwise_dequantize as mm, quantize_block_rowwise,
                                  quantize_matmul_block_rowwise_dequantize as qmm)
    d, f = 4096, 11008
    lo, hi = block_aligned_bounds(f, world, BLOCK)[rank]
    fr = hi - lo
    out = {"layer_pair": "gate_up [2*11008/p, 4096] column-parallel + down [4096, 11008/p] row-parallel, block 64",
           "ffn_columns_of_rank0": fr, "collective": "none" if world == 1 else "ncclAllReduce fp32 [M, 4096]"}
    for tag, M in (("prefill", 4096), ("decode", 8)):
        shard_bytes = 3 * fr * d
        copies = max(2, -(-(300 << 20) // shard_bytes)) if M <= 64 else 2
        gus, dns = [], []
        for c in range(copies):
            g = torch.Generator(device=dev).manual_seed(7100 + c)
            wgu = (torch.randn((2 * fr, d), device=dev, generator=g) * 0.02).to(torch.bfloat16)
            wdn = (torch.randn((d, fr), device=dev, generator=g) * 0.02).to(torch.bfloat16)
            gus.append(quantize_block_rowwise(wgu))
            dns.append(quantize_block_rowwise(wdn))
            del wgu, wdn
        x = torch.randn((M, d), device=dev, generator=torch.Generator(device=dev).manual_seed(7000)).to(torch.bfloat16)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]

        peer = None
        if world > 1 and M <= 64:
            from blockwise_int8_linear_b200.peer import PeerAllReduce
            try:
                peer = PeerAllReduce(M * d, dev, wait_limit_us=20_000_000)
            except Exception as e:       # no peer mapping on this machine: the NCCL figures stand alone
                print(f"peer-memory reduction unavailable ({type(e).__name__}: {e})", file=sys.stderr)
                peer = None
            flag = torch.tensor([1 if peer is not None else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if flag.item() == 0:
                peer = None

        large = None
        if world > 1 and M > 64:
            from blockwise_int8_linear_b200.peer import PeerAllReduceLarge
            from triton_functions import pre_quantize_matmul_block_rowwise_dequantize as pre_mm
            try:
                large = PeerAllReduceLarge(M * d, dev, wait_limit_us=20_000_000)
            except Exception as e:       # no peer mapping on this machine: the NCCL figures stand alone
                print(f"peer-memory prefill reduction unavailable ({type(e).__name__}: {e})", file=sys.stderr)
                large = None
            flag = torch.tensor([1 if large is not None else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if flag.item() == 0:
                large = None

        def pair(i, timed=False, use_peer=False):
            wq_gu, s_gu = gus[i % copies]
            wq_dn, s_dn = dns[i % copies]
            if timed:
                ev[0].record()
            cfg.INPUT_OUTPUT_TORCH_TYPE = torch.bfloat16
            if M <= 64:
                h = qmm(x, wq_gu.t(), s_gu)
            else:
                xq, sx = quantize_block_rowwise(x)
                h = mm(xq, wq_gu.t(), sx, s_gu)
            a = F.silu(h[:, :fr]) * h[:, fr:]
            if use_peer == 2:
                # the whole row-parallel layer in one call: the GEMM's reduction kernel exchanges its sums itself
                y = peer.row_parallel_linear(a, wq_dn, s_dn)
                if timed:
                    ev[1].record()
                    ev[2].record()
                return y
            if use_peer == 3:
                # prefill: the GEMM writes its fp32 partial result into the exchange buffer; one kernel per rank sums the ranks
                # (reduce-scatter by peer loads, all-gather by peer stores) and casts
                cfg.INPUT_OUTPUT_TORCH_TYPE = torch.float32
                try:
                    pre_mm("none", a, wq_dn.t(), s_dn, out=large.partial(M, d))
                finally:
                    cfg.INPUT_OUTPUT_TORCH_TYPE = torch.bfloat16
                if timed:
                    ev[1].record()
                y = large.reduce(M, d)
                if timed:
                    ev[2].record()
                return y
            cfg.INPUT_OUTPUT_TORCH_TYPE = torch.float32 if world > 1 else torch.bfloat16
            try:
                if M <= 64:
                    part = qmm(a, wq_dn.t(), s_dn)
                else:
                    aq, sa = quantize_block_rowwise(a)
                    part = mm(aq, wq_dn.t(), sa, s_dn)
            finally:
                cfg.INPUT_OUTPUT_TORCH_TYPE = torch.bfloat16
            if timed:
                ev[1].record()
            if world > 1 and use_peer:
                y = peer(part)
            elif world > 1:
                dist.all_reduce(part)
                y = part.to(torch.bfloat16)
            else:
                y = part
            if timed:
                ev[2].record()
            return y

        for i in range(5):
            pair(i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        tot, comp = [], []
        for i in range(15):
            if world > 1:
                dist.barrier()
            pair(i, timed=True)
            ev[2].synchronize()
            comp.append(ev[0].elapsed_time(ev[1]))
            tot.append(ev[0].elapsed_time(ev[2]))
        tot.sort()
        comp.sort()
        t = torch.tensor([tot[len(tot) // 2], comp[len(comp) // 2]], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_pair, ms_compute = t.tolist()
        ops = 2.0 * M * d * (2 * fr) + 2.0 * M * fr * d
        nbytes = 3 * fr * d + M * d * 2 + 2 * M * fr * 2 * 2 + M * d * 4
        roof_ms = max(ops / (INT8_NOMINAL_TOPS * 1e9), nbytes / (hbm_gbs * 1e6))
        out[tag] = {"M": M, "ms_per_pair": ms_pair, "ms_compute": ms_compute, "ms_allreduce": ms_pair - ms_compute,
                    "allreduce_share": (ms_pair - ms_compute) / ms_pair if ms_pair > 0 else None,
                    "tokens_per_s": M / (ms_pair * 1e-3), "rank_roofline_ms": roof_ms, "frac_of_rank_roofline": roof_ms / ms_pair,
                    "timing": "CUDA events, median of 15 eager steps, max over ranks; " +
                              ("weights rotate over copies larger than L2" if M <= 64 else "operands larger than L2")}
        if large is not None:
            for i in range(5):
                pair(i, use_peer=3)
            torch.cuda.synchronize()
            dist.barrier()
            tot, comp = [], []
            for i in range(15):
                dist.barrier()
                pair(i, timed=True, use_peer=3)
                ev[2].synchronize()
                comp.append(ev[0].elapsed_time(ev[1]))
                tot.append(ev[0].elapsed_time(ev[2]))
            tot.sort()
            comp.sort()
            t = torch.tensor([tot[len(tot) // 2], comp[len(comp) // 2]], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            # per rank and direction: it loads (world-1)/world of the fp32 result from its peers and receives (world-1)/world of
            # the bf16 result they store into its output; outwards it serves the same loads and issues the same stores
            nv = (world - 1) / world * M * d * (4 + 2)
            ms_red = (t[0] - t[1]).item()
            out[tag]["peer_reduce_large"] = {
                "kernel": "bi8_peer_allreduce_large (reduce-scatter by peer loads, all-gather by peer stores, one kernel per rank)",
                "ms_per_pair": t[0].item(), "ms_reduce": ms_red, "nvlink_bytes_per_direction_per_rank": nv,
                "nvlink_gbs_per_direction": nv / (ms_red * 1e-3) / 1e9 if ms_red > 0 else None,
                "frac_of_770_gbs_peer_copy": nv / (ms_red * 1e-3) / 1e9 / 770.0 if ms_red > 0 else None}
            from blockwise_int8_linear_b200 import _lib
            _lib.device_status()
            del large
        if peer is not None:
            # the same pair with the library's peer-memory reduction (one kernel, plain stores over NVLink) instead of NCCL
            for i in range(5):
                pair(i, use_peer=True)
            torch.cuda.synchronize()
            dist.barrier()
            tot, comp = [], []
            for i in range(15):
                dist.barrier()
                pair(i, timed=True, use_peer=True)
                ev[2].synchronize()
                comp.append(ev[0].elapsed_time(ev[1]))
                tot.append(ev[0].elapsed_time(ev[2]))
            tot.sort()
            comp.sort()
            t = torch.tensor([tot[len(tot) // 2], comp[len(comp) // 2]], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out[tag]["peer_reduce"] = {"kernel": "bi8_peer_allreduce (st.global to every rank's slots, flag per chunk, sum in rank order)",
                                       "ms_per_pair": t[0].item(), "ms_reduce": (t[0] - t[1]).item()}
            for i in range(5):
                pair(i, use_peer=2)
            torch.cuda.synchronize()
            dist.barrier()
            tot = []
            for i in range(15):
                dist.barrier()
                pair(i, timed=True, use_peer=2)
                ev[2].synchronize()
                tot.append(ev[0].elapsed_time(ev[2]))
            tot.sort()
            t = torch.tensor([tot[len(tot) // 2]], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out[tag]["peer_reduce_fused"] = {"kernel": "bi8_row_parallel_linear (the decode GEMM's reduction kernel sums tile parts and ranks)",
                                             "ms_per_pair": t[0].item()}
            from blockwise_int8_linear_b200 import _lib
            _lib.device_status()
        del gus, dns
    return out


def _load_example(name):
    import importlib.util
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "examples", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def models_bench(dev, rank, world, local):
    """The two model drivers of examples/ at this GPU count, bounded to a couple of minutes: Llama-2-7B architecture
    (tensor parallel over the ranks; full depth, 512-token prompt, 32 greedy steps) and GPT-2 small training (data parallel,
    6 timed steps), int8 layers and the same model with bf16 nn.Linear."""
    import gc
    out = {}
    L = _load_example("llama_infer")
    a = argparse.Namespace(layers=32, hidden=4096, heads=32, head_dim=128, ffn=11008, vocab=32000, batch=8, prompt=512,
                           decode=33, block=BLOCK)
    r = L.run(a, rank, world, dev)
    out["llama7b_infer"] = {k: r[k] for k in ("n_gpus", "batch", "prompt", "decode", "prefill_tokens_per_s", "decode_tokens_per_s",
                                              "decode_ms_per_step", "decode_mode", "first_tokens")}
    out["llama7b_infer"]["parallelism"] = f"tp{world}"
    del r
    gc.collect()
    torch.cuda.empty_cache()
    G = _load_example("gpt2_train")
    for tag, dense in (("gpt2_small_train_int8", False), ("gpt2_small_train_bf16_dense", True)):
        ga = argparse.Namespace(steps=6, warmup=2, batch=8, seq=1024, layers=12, block=BLOCK, dense=dense)
        r = G.run(ga, rank, world, local, dev)
        out[tag] = {k: r[k] for k in ("n_gpus", "batch_per_gpu", "steps", "tokens_per_s", "ms_per_step", "loss_first", "loss_last")}
        out[tag]["parallelism"] = f"dp{world} (DistributedDataParallel, NCCL gradient all-reduce)"
        gc.collect()
        torch.cuda.empty_cache()
    return out


def run_ours(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    import block_linear_config as cfg
    from block_linear import BlockInt8Linear
    from blockwise_int8_linear_b200 import _lib
    from triton_functions import int8_matmul_block64_rowwise_dequantize, quantize_block_rowwise

    cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE = BLOCK, torch.bfloat16
    M, K, N = WORKLOADS[args.workload]
    hbm_gbs, bf16_tf, peak_src = peaks()

    # Synthetic data of the benchmark configuration: activations N(0,1), weights N(0, 0.02), both bf16.
    # Three rotating buffer sets (x, y) so that consecutive steps do not find their inputs in the 126 MB L2.
    gen = torch.Generator(device=dev).manual_seed(3000 + rank)
    xs_dev = [torch.randn((M, K), device=dev, generator=gen).to(torch.bfloat16) for _ in range(NSETS)]
    w = (torch.randn((N, K), device=dev, generator=torch.Generator(device=dev).manual_seed(3100)) * 0.02).to(torch.bfloat16)
    wq, ws = quantize_block_rowwise(w)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flush = lambda: flush_buf.fill_(1)

    def step(i, ev=None):
        x = xs_dev[i % NSETS]
        xq, sx = quantize_block_rowwise(x)
        if ev is not None:
            ev[0].record()
        y = int8_matmul_block64_rowwise_dequantize(xq, wq.t(), sx, ws)
        if ev is not None:
            ev[1].record()
        return y

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
            torch.cuda.synchronize()

    # the sampler starts before the warm-up (nvidia-smi needs a few hundred milliseconds to deliver its first line); only
    # samples that arrive from the start of the timed region on are kept
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(args.warmup):
        step(i)
    barrier()
    gemm_events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_clock0 = time.perf_counter()
    t_start.record()
    for i in range(args.steps):
        step(i, gemm_events[i])
    t_end.record()
    barrier()
    clocks = None
    if rank == 0:
        # A timed region shorter than a few sample periods: the same loop keeps running, untimed, until three samples have
        # arrived under this load (one second at most).
        extra_steps = 0
        while sampler.proc is not None and sampler.count_since(t_clock0) < 3 and time.perf_counter() - t_clock0 < 1.0:
            for i in range(args.steps):
                step(i)
            torch.cuda.synchronize()
            extra_steps += args.steps
        clocks = sampler.stop(since=t_clock0)
        clocks["window"] = "timed region" if extra_steps == 0 else f"timed region + {extra_steps} further untimed steps of the same loop"
    barrier()
    ms_total = t_start.elapsed_time(t_end)
    gemm_ms = sum(a.elapsed_time(b) for a, b in gemm_events) / args.steps
    if world > 1:
        t = torch.tensor([ms_total, gemm_ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms_total, gemm_ms = t.tolist()
    ms_step = ms_total / args.steps
    ops_step = 2.0 * M * N * K
    value = world * ops_step / (ms_step * 1e-3) / 1e12
    _lib.device_status()

    # ---- end to end through the public API with host buffers ----
    # Every step copies its activations from pinned host memory, runs BlockInt8Linear.forward and copies the result back
    # to pinned host memory.  The three legs run on three streams with double buffers, so that the copy engines work on
    # the neighbouring steps while the kernels of one step run (the way a serving loop drives the layer); every byte of
    # every step still crosses PCIe inside the timed region.
    lin = BlockInt8Linear(K, N, bias=False, device=dev, dtype=torch.bfloat16).eval()
    lin.weight.data = w
    x_host = [xs_dev[i].cpu().pin_memory() for i in range(2)]
    y_host = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    x_dev2 = [torch.empty((M, K), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    y_dev2 = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_run = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        b = i % 2
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_free[b])                 # x_dev2[b] was consumed by the step that used it last
            x_dev2[b].copy_(x_host[b], non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in[b])
            s_run.wait_event(ev_out[b])                 # y_dev2[b] has been copied out
            with torch.no_grad():
                y_dev2[b].copy_(lin(x_dev2[b]))
            ev_free[b].record(s_run)
            ev_run[b].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_run[b])
            y_host[b].copy_(y_dev2[b], non_blocking=True)
            ev_out[b].record(s_out)

    for ev in ev_free + ev_out:
        ev.record()
    for i in range(max(3, args.warmup)):
        e2e_step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s_ in (s_in, s_run, s_out):
        s_.wait_event(e0)
    for i in range(args.steps):
        e2e_step(i)
    for s_ in (s_in, s_run, s_out):
        torch.cuda.current_stream().wait_stream(s_)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        e2e_ms = t.item()
    e2e_value = world * ops_step / (e2e_ms * 1e-3) / 1e12
    del lin, x_host, y_host, x_dev2, y_dev2

    # ---- the partitionings that communicate, at this GPU count (all ranks take part) ----
    del xs_dev
    torch.cuda.empty_cache()
    tp = models = None
    if not args.no_tp:
        try:
            tp = tp_bench(dev, rank, world, hbm_gbs)
        except Exception as e:            # the tensor-parallel pair must not take the headline down with it
            tp = {"error": f"{type(e).__name__}: {e}"}
    if not args.no_models:
        try:
            models = models_bench(dev, rank, world, local)
        except Exception as e:            # a model driver must not take the headline down with it
            models = {"error": f"{type(e).__name__}: {e}"}
    try:
        _lib.device_status()
    except Exception as e:                # a bounded wait that gave up in one of the extras: reported, not fatal
        (models if isinstance(models, dict) else {}).setdefault("device_status", str(e))

    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    # ---- rank 0: roofline, probe, sweeps, CPU baseline ----
    achieved = ops_step / (gemm_ms * 1e-3) / 1e12
    probe = None
    try:
        import ctypes
        ms_p, sms = ctypes.c_float(0), ctypes.c_int(0)
        iters = 1 << 16
        _lib.check(_lib.lib().bi8_mma_peak_probe(iters, ctypes.byref(ms_p), ctypes.byref(sms)), "bi8_mma_peak_probe")
        probe = sms.value * iters * 2.0 * 128 * 256 * 32 / (ms_p.value * 1e-3) / 1e12
    except Exception as e:  # the probe is informational
        probe = None
        print(f"mma probe failed: {e}", file=sys.stderr)
    peak = 2.0 * bf16_tf
    roofline = {
        "bound": "tensor", "kernel": "gemm_tc_kernel<64,0,seeded> (tcgen05 kind::i8, 128x160 tiles)", "achieved": achieved, "peak": peak,
        "unit": "TFLOP/s", "frac": achieved / peak,
        "peak_source": f"2 x {peak_src} cuBLAS bf16 burst ({bf16_tf} TF/s); int8 multiply-add counted as 2 ops",
        "frac_of_nominal_int8_4500": achieved / INT8_NOMINAL_TOPS,
        "mma_issue_probe_tops": probe, "frac_of_mma_issue_probe": (achieved / probe) if probe else None,
        "gemm_ms": gemm_ms, "algorithmic_ops_per_launch": ops_step,
        "traffic": ncu_traffic(f"gemm_tc:{args.workload}"),
    }
    # comparator only: the same (M, K, N) as one bf16 GEMM in cuBLAS, what the layer costs without quantization
    xb = torch.randn((M, K), device=dev, dtype=torch.bfloat16)
    for _ in range(3):
        torch.matmul(xb, w.t())
    roofline["cublas_bf16_ms"] = time_kernel(lambda: torch.matmul(xb, w.t()), 7, flush)
    roofline["int8_gemm_over_cublas_bf16"] = gemm_ms / roofline["cublas_bf16_ms"]
    del xb
    # the GEMM back to back for two seconds (pre-quantized activations, rotating outputs)
    xq_s, sx_s = quantize_block_rowwise(torch.randn((M, K), device=dev, generator=torch.Generator(device=dev).manual_seed(1)).to(torch.bfloat16))
    roofline["sustained"] = sustained_gemm(lambda i: int8_matmul_block64_rowwise_dequantize(xq_s, wq.t(), sx_s, ws), ops_step, local)
    del xq_s, sx_s
    extra = None
    if world == 1 and not args.no_extras:
        extra = extras(dev, hbm_gbs, flush)
        extra["hbm_peak_gbs"] = hbm_gbs
        extra["hbm_peak_source"] = peak_src
        extra["timing"] = ("us: CUDA-graph replays over rotating inputs larger than L2, median of 5 replays; us_flushed and the "
                           "GEMM rows marked so: CUDA events around one launch behind a 256 MB fill, median of 7")
        roofline["kernels"] = kernel_rows(extra, hbm_gbs)
        roofline["fused_producers"] = extra.get("fused_producers")
        try:
            roofline["k512_sweep"] = k512_sweep(dev, flush)
        except Exception as e:            # comparator table only
            roofline["k512_sweep"] = {"error": f"{type(e).__name__}: {e}"}
        roofline["kernels_note"] = (f"frac = fraction of the {peak_src} HBM copy bandwidth ({hbm_gbs} GB/s) for bound hbm, of the nominal "
                                    "4500 TOP/s for bound tensor; M <= 128 rows and the quantizers are CUDA-graph replays over rotating inputs")
    if tp is not None:
        roofline["tp"] = tp
    if models is not None:
        roofline["models"] = models
    cpu = None
    if world == 1 and not args.no_cpu:
        cpu, _ = cpu_baseline(args.workload)
    line = {
        "metric": "int8_block_gemm_tops", "value": value, "unit": "TOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": bench_config(args.workload, world),
        "roofline": roofline,
        "e2e": {"value": e2e_value, "unit": "TOP/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": M * K * 2,
                "d2h_bytes_per_step": M * N * 2, "api": "BlockInt8Linear.forward (eval) on pinned host buffers; H2D, kernels and D2H of neighbouring steps overlap on three streams"},
        "gpu_launches": world * args.steps * 2,          # quantize + GEMM per step in the device-timed region (the e2e leg launches the same two per step)
        "clocks": clocks,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if extra is not None and args.full_extra:
        line["extra"] = extra
    print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=DEFAULT_WORKLOAD)
    ap.add_argument("--no-extras", action="store_true", help="skip the quantize/dequantize/GEMM-shape sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel MLP pair")
    ap.add_argument("--no-models", action="store_true", help="skip the Llama inference / GPT-2 training drivers")
    ap.add_argument("--full-extra", action="store_true", help="also print the full sweep tables (the compact rows are in roofline.kernels)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
