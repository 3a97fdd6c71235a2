"""Llama-2-7B-architecture inference with every linear layer replaced by BlockInt8Linear.

The reference's example only quantizes one weight matrix of a downloaded checkpoint
(``examples/quantised_infer_llama.py/infer_llama.ipynb``); checkpoints are not available offline, so this driver
builds the architecture (32 layers, d = 4096, 32 heads, FFN 11008, vocab 32000) with seeded random weights
N(0, 0.02), runs a 512-token prompt for a batch of 8 and decodes 128 tokens greedily with a KV cache.

Single GPU:            python examples/llama_infer.py
Tensor parallel (N):   python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 examples/llama_infer.py

Tensor parallelism follows ``blockwise_int8_linear_b200.parallel``: q/k/v, gate/up and the LM head are split over output
features (bit-identical columns), o_proj and down_proj over input features on block boundaries (11008 = 172 blocks of 64 is
split 22/21 blocks for 8 ranks) with fp32 partial results summed once per layer half: by the library's peer-memory kernels
(``--reduce peer``, the default: the decode step is then one CUDA graph per rank, and the prefill's sums are a reduce-scatter
by peer loads and an all-gather by peer stores) or by NCCL (``--reduce nccl``).

The elementwise steps between the layer's kernels run inside the library's calls (``BlockInt8Linear.infer_pre``: RMSNorm and
``silu(gate) * up`` in the quantizer, the residual sum in the kernel that writes the GEMM's result; rotary embedding and
cache append of a decode step in one kernel); ``--no-fuse`` runs them as torch kernels, for comparison.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import block_linear_config as cfg  # noqa: E402
from block_linear import BlockInt8Linear  # noqa: E402
from blockwise_int8_linear_b200.decode_ops import rope_cache_append  # noqa: E402
from blockwise_int8_linear_b200.parallel import block_aligned_bounds  # noqa: E402
from triton_functions import pre_quantize_matmul_block_rowwise_dequantize  # noqa: E402


def seeded_weight(out_f, in_f, seed, dev, rows=None, cols=None):
    """N(0, 0.02) bf16 [out_f, in_f], generated from `seed` so that every rank sees the same full matrix, then sliced."""
    g = torch.Generator(device=dev).manual_seed(seed)
    w = (torch.randn((out_f, in_f), device=dev, generator=g) * 0.02).to(torch.bfloat16)
    if rows is not None:
        w = w[rows[0]:rows[1]]
    if cols is not None:
        w = w[:, cols[0]:cols[1]]
    return w.contiguous()


class Int8Linear(nn.Module):
    """A BlockInt8Linear holding this rank's shard of one or several projections that share their input.

    mode 'col': rows [lo,hi) of every weight in `out_fs` (q/k/v, or gate/up, are stored as one matrix, so the step runs one
    GEMM for them; each part keeps its own seed, so the model is the same function as with separate layers), local output.
    mode 'row': columns [lo,hi), fp32 partial output summed over the group."""

    def __init__(self, in_f, out_fs, seeds, dev, mode, rank, world, block, ops=None):
        super().__init__()
        self.mode, self.world, self.ops = mode, world, ops
        if mode == "col":
            parts = []
            for out_f, seed in zip(out_fs, seeds):
                lo, hi = block_aligned_bounds(out_f, world, block)[rank]
                parts.append(seeded_weight(out_f, in_f, seed, dev, rows=(lo, hi)))
            self.bounds = (lo, hi)
            self.widths = [p.shape[0] for p in parts]
            w = torch.cat(parts, dim=0) if len(parts) > 1 else parts[0]
        else:
            lo, hi = block_aligned_bounds(in_f, world, block)[rank]
            w = seeded_weight(out_fs[0], in_f, seeds[0], dev, cols=(lo, hi))
            self.bounds = (lo, hi)
            self.widths = [w.shape[0]]
        if ops is not None:
            # stand-in functional ops (the host-side sharding logic can then run on CPU ranks): same two calls as
            # BlockInt8Linear.infer on the int8 weights
            self.lin = None
            self.W_int8, self.state_W = ops.quantize_block_rowwise(w)
            return
        self.lin = BlockInt8Linear(w.shape[1], w.shape[0], bias=False, device=dev, dtype=torch.bfloat16)
        self.lin.weight.data = w
        self.lin.eval()
        self.lin.prepare_for_eval(drop_weight=True)                                  # keep only the int8 copy resident

    def _infer(self, x):
        if self.lin is not None:
            return self.lin.infer(x)
        X = x.reshape(-1, x.size(-1))
        xq, sx = self.ops.quantize_block_rowwise(X)
        return self.ops.int8_matmul_block64_rowwise_dequantize(xq, self.W_int8.t(), sx, self.state_W, None).view(*x.size()[:-1], -1)

    def partial(self, x):
        """This rank's contribution: the finished result for a column-parallel layer (or one rank), an fp32 partial sum for
        a row-parallel one (to be summed over the group by the caller)."""
        if self.mode == "col" or self.world == 1:
            return self._infer(x)
        prev = cfg.INPUT_OUTPUT_TORCH_TYPE
        cfg.INPUT_OUTPUT_TORCH_TYPE = torch.float32
        try:
            return self._infer(x)
        finally:
            cfg.INPUT_OUTPUT_TORCH_TYPE = prev

    def forward(self, x):
        part = self.partial(x)
        if self.mode == "col" or self.world == 1:
            return part
        dist.all_reduce(part)
        return part.to(cfg.INPUT_OUTPUT_TORCH_TYPE)

    def fusable(self):
        """Whether `fused` runs as one library call: a layer whose output needs no sum over ranks."""
        return FUSE and self.lin is not None and (self.mode == "col" or self.world == 1)

    def fused(self, x, op="none", x2=None, residual=None):
        """``residual + self(pre(x))`` with pre = rms_norm ('rmsnorm'), silu(x) * x2 ('silu_mul') or nothing ('none'):
        the producer step inside the layer's quantizer and the residual sum inside the kernel that writes its output
        where the layer's output is complete on this rank, the separate torch kernels otherwise."""
        if self.fusable():
            return self.lin.infer_pre(x, op, x2=x2, eps=NORM_EPS, residual=residual)
        inp = rms_norm(x) if op == "rmsnorm" else (F.silu(x) * x2 if op == "silu_mul" else x)
        y = self.forward(inp)
        return y if residual is None else residual + y

    def summed(self, x, op="none", x2=None, residual=None):
        """``residual + sum over the group of this row-parallel layer applied to pre(x)``, cast to the activation type: for
        decode-sized inputs with the peer-memory reduction installed, one library call whose first kernel applies `op` and
        quantizes and whose last kernel adds the GEMM's tile parts, the ranks and the residual."""
        peer = self.world > 1 and self.mode == "row" and PEER is not None and self.lin is not None
        if peer:
            rows = x.numel() // x.shape[-1]
            peer = rows <= 64 and rows * self.widths[0] <= PEER.capacity
        if peer and FUSE:
            return PEER.row_parallel_linear(x, self.lin.W_int8, self.lin.state_W, op=op, x2=x2, residual=residual)
        rows = x.numel() // x.shape[-1]
        if (not peer and self.world > 1 and self.mode == "row" and PEER_LARGE is not None and self.lin is not None
                and rows * self.widths[0] <= PEER_LARGE.capacity and self.widths[0] % 4 == 0):
            # prefill: the GEMM writes its fp32 partial result into the exchange buffer, one kernel per rank sums the ranks
            # (reduce-scatter by peer loads, all-gather by peer stores), casts and adds the residual
            n = self.widths[0]
            if not FUSE:
                x, x2, op = (rms_norm(x) if op == "rmsnorm" else (F.silu(x) * x2 if op == "silu_mul" else x)), None, "none"
            prev = cfg.INPUT_OUTPUT_TORCH_TYPE
            cfg.INPUT_OUTPUT_TORCH_TYPE = torch.float32
            try:
                pre_quantize_matmul_block_rowwise_dequantize(op, x.reshape(rows, -1), self.lin.W_int8.t(), self.lin.state_W,
                                                             x2=None if x2 is None else x2.reshape(rows, -1), eps=NORM_EPS,
                                                             out=PEER_LARGE.partial(rows, n))
            finally:
                cfg.INPUT_OUTPUT_TORCH_TYPE = prev
            res = residual.reshape(rows, n).contiguous() if residual is not None and FUSE else None
            y = PEER_LARGE.reduce(rows, n, residual=res).clone().view(*x.shape[:-1], n)    # the view lives until the next sum
            return y if residual is None or FUSE else residual + y
        inp = rms_norm(x) if op == "rmsnorm" else (F.silu(x) * x2 if op == "silu_mul" else x)
        if peer:
            y = PEER.row_parallel_linear(inp, self.lin.W_int8, self.lin.state_W)
        else:
            y = group_sum(self.partial(inp), cfg.INPUT_OUTPUT_TORCH_TYPE, self.world)
        return y if residual is None else residual + y


NORM_EPS = 1e-5
FUSE = True      # producer steps and residual sums inside the library's calls (Int8Linear.fused); --no-fuse runs them as torch kernels


def rms_norm(x, eps=NORM_EPS):
    return F.rms_norm(x, (x.shape[-1],), eps=eps)


def rope_table(max_len, d, dev, theta=10000.0):
    """cos/sin of every position as one complex table [max_len, d/2], built once."""
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=dev, dtype=torch.float32) / d))
    ang = torch.arange(max_len, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.polar(torch.ones_like(ang), ang)


def rope(x, cis):
    # x [B, T, G, H, D] (G = q and k) with (even, odd) feature pairs rotated by the position's angle; cis [T, D/2] complex
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    return torch.view_as_real(xc * cis[None, :, None, None]).flatten(-2).to(x.dtype)


class Layer(nn.Module):
    def __init__(self, i, a, dev, rank, world, ops=None):
        super().__init__()
        d, f, blk = a.hidden, a.ffn, a.block
        mk = lambda in_f, out_fs, seeds, mode: Int8Linear(in_f, out_fs, [1000 * i + s for s in seeds], dev, mode, rank, world, blk, ops)
        self.qkv = mk(d, (d, d, d), (1, 2, 3), "col")
        self.o = mk(d, (d,), (4,), "row")
        self.gate_up = mk(d, (f, f), (5, 6), "col")
        self.down = mk(f, (d,), (7,), "row")
        self.heads_local = self.qkv.widths[0] // a.head_dim
        self.head_dim = a.head_dim
        self.kcache = self.vcache = None

    def attn_partial(self, x, pos0, max_len, cis, mask=None, pos_dev=None, summed=False, residual=None):
        """Attention half of the layer up to the output projection; without `residual` also without the sum over ranks
        (unless `summed`) and the residual add, with it the half's complete output ``residual + o(att)``.
        Prefill: pos0 is a Python int and the cache is sliced.  Decode (pos_dev given, T == 1): the position is a device
        tensor, the cache is written with index_copy_ and attended in full under a mask, so that every shape is static and
        the step can be captured in a CUDA graph.  `cis` holds the rotary factors of this call's positions."""
        B, T, _ = x.shape
        hl, hd = self.heads_local, self.head_dim
        qkv = self.qkv.fused(x, "rmsnorm").view(B, T, 3, hl, hd)
        if pos_dev is not None and T == 1 and FUSE and self.qkv.lin is not None and self.kcache is not None:
            # decode: rotation of q and k and the append of k and v to the caches in one launch
            q = rope_cache_append(qkv.view(B, 3, hl, hd), cis, pos_dev, self.kcache, self.vcache)
            att = F.scaled_dot_product_attention(q, self.kcache, self.vcache, attn_mask=mask)
            att = att.transpose(1, 2).reshape(B, T, hl * hd)
            if residual is not None and self.o.fusable():
                return self.o.fused(att, "none", residual=residual)
            if residual is not None:
                return self.o.summed(att, residual=residual)
            return self.o.summed(att) if summed else self.o.partial(att)
        qk = rope(qkv[:, :, :2], cis)                                   # q and k in one pass: [B, T, 2, H, D]
        q, k, v = qk[:, :, 0].transpose(1, 2), qk[:, :, 1].transpose(1, 2), qkv[:, :, 2].transpose(1, 2)
        if self.kcache is None:
            self.kcache = torch.zeros((B, hl, max_len, hd), device=x.device, dtype=x.dtype)
            self.vcache = torch.zeros_like(self.kcache)
        if pos_dev is None:
            self.kcache[:, :, pos0:pos0 + T] = k
            self.vcache[:, :, pos0:pos0 + T] = v
            kk, vv = self.kcache[:, :, :pos0 + T], self.vcache[:, :, :pos0 + T]
            att = F.scaled_dot_product_attention(q, kk, vv, is_causal=(T > 1))
        else:
            self.kcache.index_copy_(2, pos_dev, k)
            self.vcache.index_copy_(2, pos_dev, v)
            att = F.scaled_dot_product_attention(q, self.kcache, self.vcache, attn_mask=mask)
        att = att.transpose(1, 2).reshape(B, T, hl * hd)
        if residual is not None and self.o.fusable():
            return self.o.fused(att, "none", residual=residual)
        if residual is not None:
            return self.o.summed(att, residual=residual)
        return self.o.summed(att) if summed else self.o.partial(att)

    def mlp_partial(self, x, summed=False, residual=None):
        gate, up = self.gate_up.fused(x, "rmsnorm").split(self.gate_up.widths, dim=-1)
        if residual is not None and self.down.fusable():
            return self.down.fused(gate, "silu_mul", x2=up, residual=residual)
        if residual is not None:
            return self.down.summed(gate, "silu_mul", x2=up, residual=residual)
        h = F.silu(gate) * up
        return self.down.summed(h) if summed else self.down.partial(h)

    def forward(self, x, pos0, max_len, cis, mask=None, pos_dev=None):
        x = self.attn_partial(x, pos0, max_len, cis, mask, pos_dev, residual=x)
        return self.mlp_partial(x, residual=x)


PEER = None      # a blockwise_int8_linear_b200.peer.PeerAllReduce while the decode step uses the library's own reduction
PEER_LARGE = None   # a PeerAllReduceLarge while the prefill's row-parallel layers are summed by the library's own kernel


def group_sum(part, dtype, world):
    """Sum of the ranks' row-parallel partial results, cast to the activation type: the library's peer-memory kernel
    when one is installed and the tensor fits its buffers (decode), else fp32 over NCCL (prefill)."""
    if world == 1:
        return part
    if PEER is not None and part.numel() <= PEER.capacity:
        return PEER(part.contiguous())
    dist.all_reduce(part)
    return part.to(dtype)


class Llama(nn.Module):
    def __init__(self, a, dev, rank, world, ops=None):
        """`ops`: optional namespace with quantize_block_rowwise / int8_matmul_block64_rowwise_dequantize that replaces the
        CUDA-backed functions (used to exercise the sharding on CPU ranks)."""
        super().__init__()
        g = torch.Generator(device=dev).manual_seed(7)
        self.emb = (torch.randn((a.vocab, a.hidden), device=dev, generator=g) * 0.02).to(torch.bfloat16)
        self.layers = nn.ModuleList(Layer(i, a, dev, rank, world, ops) for i in range(a.layers))
        self.head = Int8Linear(a.hidden, (a.vocab,), (99,), dev, "col", rank, world, a.block, ops)
        self.world, self.vocab, self.block = world, a.vocab, a.block
        self.cis = rope_table(a.prompt + a.decode + 16, a.head_dim, dev)
        self.positions = torch.arange(a.prompt + a.decode + 16, device=dev)

    def positions_of(self, ids, pos0, max_len, pos_dev):
        if pos_dev is None:
            return self.cis[pos0:pos0 + ids.shape[1]], None
        # an additive mask in the activation type, built once per step: given a boolean mask, every layer's attention call
        # would convert it again (two fills and a select per layer)
        keep = (self.positions[:max_len] <= pos_dev).view(1, 1, 1, max_len)
        mask = torch.zeros((1, 1, 1, max_len), device=ids.device, dtype=self.emb.dtype).masked_fill_(~keep, float("-inf"))
        return self.cis.index_select(0, pos_dev), mask

    def local_logits(self, x):
        """[B, 1, V_local] of this rank, padded with -inf to the widest shard (all_gather wants equal sizes)."""
        logits = self.head.fused(x[:, -1:], "rmsnorm")
        if self.world == 1:
            return logits
        sizes = [hi - lo for lo, hi in block_aligned_bounds(self.vocab, self.world, self.block)]
        pad = torch.full((logits.shape[0], 1, max(sizes)), float("-inf"), device=logits.device, dtype=logits.dtype)
        pad[..., : logits.shape[-1]] = logits
        return pad

    def join_logits(self, bufs):
        sizes = [hi - lo for lo, hi in block_aligned_bounds(self.vocab, self.world, self.block)]
        return torch.cat([b[..., :n] for b, n in zip(bufs, sizes)], dim=-1)

    @torch.no_grad()
    def forward(self, ids, pos0, max_len, pos_dev=None):
        x = self.emb[ids]
        cis, mask = self.positions_of(ids, pos0, max_len, pos_dev)
        for layer in self.layers:
            x = layer(x, pos0, max_len, cis, mask, pos_dev)
        logits = self.local_logits(x)                              # [B, 1, V_local]
        if self.world > 1:
            width = logits.shape[-1]
            if PEER is not None and logits.shape[0] * width * self.world <= PEER.capacity:
                # gather as a sum: every rank contributes its shard in place and zeros elsewhere
                full = torch.zeros((logits.shape[0], 1, width * self.world), device=logits.device, dtype=torch.float32)
                rank = dist.get_rank()
                full[..., rank * width:(rank + 1) * width] = torch.nan_to_num(logits.float(), neginf=-3.0e38)
                summed = PEER(full, out=torch.empty_like(full))
                bufs = list(summed.split(width, dim=-1))
            else:
                bufs = [torch.empty_like(logits) for _ in range(self.world)]
                dist.all_gather(bufs, logits)
            logits = self.join_logits(bufs)
        return logits

    @torch.no_grad()
    def decode_pieces(self, tok, pos_dev, max_len):
        """The decode step of a tensor-parallel group as a list of (compute, bind) pairs: every compute piece is free of
        communication and can be captured in a CUDA graph of its own, the NCCL calls run between the replays.  The
        pieces hand their tensors to each other through `st`; `bind()`, called right after its piece has been captured,
        returns the collective on exactly the tensors that piece produced (later pieces put new tensors under the same
        keys)."""
        st = {}
        dtype = self.emb.dtype

        def reduce_part():
            part = st["part"]
            return lambda: dist.all_reduce(part)

        def first():
            st["cis"], st["mask"] = self.positions_of(tok, 0, max_len, pos_dev)
            st["x"] = self.emb[tok]
            st["part"] = self.layers[0].attn_partial(st["x"], 0, max_len, st["cis"], st["mask"], pos_dev)

        pieces = [(first, reduce_part)]
        for i, layer in enumerate(self.layers):
            def mlp(layer=layer):
                st["x"] = st["x"] + st["part"].to(dtype)
                st["part"] = layer.mlp_partial(st["x"])

            pieces.append((mlp, reduce_part))
            if i + 1 < len(self.layers):
                def attn(nxt=self.layers[i + 1]):
                    st["x"] = st["x"] + st["part"].to(dtype)
                    st["part"] = nxt.attn_partial(st["x"], 0, max_len, st["cis"], st["mask"], pos_dev)

                pieces.append((attn, reduce_part))

        def head():
            st["logits"] = self.local_logits(st["x"] + st["part"].to(dtype))
            st["bufs"] = [torch.empty_like(st["logits"]) for _ in range(self.world)]

        def last():
            tok.copy_(self.join_logits(st["bufs"]).argmax(-1))
            pos_dev.add_(1)

        def gather_logits():
            bufs, logits = st["bufs"], st["logits"]
            return lambda: dist.all_gather(bufs, logits)

        pieces.append((head, gather_logits))
        pieces.append((last, None))
        return pieces


def run(a, rank, world, dev, eager=False):
    """Builds the model described by `a` (fields as the command line options below) on this rank, runs the prompt and
    the greedy decode, and returns the measurements and the generated tokens.  The process group, if any, is the
    caller's."""
    assert a.heads % world == 0, "heads must divide over the ranks"
    global FUSE
    FUSE = not getattr(a, "no_fuse", False)
    cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE = a.block, torch.bfloat16
    global PEER_LARGE
    PEER_LARGE = None
    if world > 1 and getattr(a, "reduce", "peer") == "peer":
        from blockwise_int8_linear_b200.peer import PeerAllReduceLarge
        try:
            PEER_LARGE = PeerAllReduceLarge(a.batch * a.prompt * a.hidden, dev, wait_limit_us=20_000_000)
        except Exception as e:                                  # no peer mapping on this machine: NCCL
            print(f"peer-memory prefill reduction unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
            PEER_LARGE = None
        flag = torch.tensor([1 if PEER_LARGE is not None else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)               # all ranks take the same path
        if flag.item() == 0:
            PEER_LARGE = None
    model = Llama(a, dev, rank, world)
    ids = torch.randint(0, a.vocab, (a.batch, a.prompt), generator=torch.Generator().manual_seed(4000)).to(dev)
    max_len = -(-(a.prompt + a.decode) // 16) * 16                # cache length: a multiple of 16, so that the attention call
    torch.cuda.synchronize()                                      # takes the additive mask as it is (no padded copy per layer)
    t0 = time.perf_counter()
    model(ids, 0, max_len)                                        # first call: lazy initialisation, allocator growth
    torch.cuda.synchronize()
    t_first = time.perf_counter() - t0
    t_prefill = float("inf")
    for _ in range(4):                                            # steady state (rewrites the same cache positions)
        t0 = time.perf_counter()
        logits = model(ids, 0, max_len)
        torch.cuda.synchronize()
        t_prefill = min(t_prefill, time.perf_counter() - t0)
    nxt = logits.argmax(-1)
    out = [nxt]
    # Decode: one step = ~450 small launches (quantize + GEMM per linear, attention, norms); eager launch latency would
    # dominate, so the step is captured once in a CUDA graph (static token / position buffers) and replayed.
    tok = nxt.clone()
    pos_dev = torch.full((1,), a.prompt, device=dev, dtype=torch.long)

    def decode_step():
        lg = model(tok, 0, max_len, pos_dev)
        tok.copy_(lg.argmax(-1))
        pos_dev.add_(1)

    global PEER
    PEER = None
    if world > 1 and not eager and getattr(a, "reduce", "peer") == "peer":
        from blockwise_int8_linear_b200.peer import PeerAllReduce
        widest = max(hi - lo for lo, hi in block_aligned_bounds(a.vocab, world, a.block))
        try:
            PEER = PeerAllReduce(max(a.batch * a.hidden, a.batch * widest * world), dev, wait_limit_us=20_000_000)
        except Exception as e:                                  # no peer mapping on this machine: NCCL between graphs
            print(f"peer-memory reduction unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
            PEER = None
        # all ranks take the same path
        flag = torch.tensor([1 if PEER is not None else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if flag.item() == 0:
            PEER = None
    graph, pieces = None, None
    if not eager:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):                                    # warm-up on a side stream (allocator, NCCL, lazy init)
                decode_step()
        torch.cuda.current_stream().wait_stream(side)
        tok.copy_(nxt)
        pos_dev.fill_(a.prompt)
        if world == 1 or PEER is not None:
            # one graph for the whole step: with the peer-memory reduction there is no host work between its kernels
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                decode_step()
        else:
            # Tensor parallel: NCCL stays outside the graphs.  The step is cut at its collectives (two sums per layer, one
            # gather of the logits); every communication-free piece is captured in a graph of its own (one shared memory
            # pool, so a piece reads the tensors the piece before it wrote) and the collectives are issued between the
            # replays.
            pieces, pool = [], None
            for compute, bind in model.decode_pieces(tok, pos_dev, max_len):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=pool):
                    compute()
                pool = g.pool()
                pieces.append((g, bind() if bind is not None else None))
        tok.copy_(nxt)                                            # the capture itself does not execute the step
        pos_dev.fill_(a.prompt)
    else:
        decode_step()                                             # warm-up
        tok.copy_(nxt)
        pos_dev.fill_(a.prompt)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()                                            # the ranks start the decode loop together
    t0 = time.perf_counter()
    for step in range(a.decode - 1):
        if graph is not None:
            graph.replay()
        elif pieces is not None:
            for g, collective in pieces:
                g.replay()
                if collective is not None:
                    collective()
        else:
            decode_step()
        out.append(tok.clone())
    torch.cuda.synchronize()
    t_decode = time.perf_counter() - t0
    toks = torch.cat(out, dim=1)
    if PEER is not None or PEER_LARGE is not None:
        from blockwise_int8_linear_b200 import _lib
        _lib.device_status()                                      # raises if a bounded flag wait gave up
        PEER = PEER_LARGE = None
    return {
        "model": f"llama-arch {a.layers}x{a.hidden} ffn {a.ffn} vocab {a.vocab}, random init N(0,0.02), BlockInt8Linear block {a.block}",
        "n_gpus": world, "batch": a.batch, "prompt": a.prompt, "decode": a.decode,
        "prefill_tokens_per_s": a.batch * a.prompt / t_prefill, "prefill_s": t_prefill, "first_prefill_s": t_first,
        "decode_tokens_per_s": a.batch * (a.decode - 1) / t_decode, "decode_ms_per_step": 1e3 * t_decode / max(1, a.decode - 1),
        "decode_mode": "eager" if eager else ("cuda graph" if world == 1 else
                                              "one cuda graph, peer-memory reductions" if graph is not None else
                                              "cuda graphs between the NCCL collectives"),
        "fused_producers": FUSE,
        "first_tokens": toks[0, :8].tolist(), "tokens": toks.tolist(),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--decode", type=int, default=128)
    ap.add_argument("--block", type=int, default=64)
    ap.add_argument("--eager", action="store_true", help="do not capture the decode step in a CUDA graph")
    ap.add_argument("--reduce", choices=["peer", "nccl"], default="peer",
                    help="tensor-parallel decode: the library's peer-memory reduction inside one CUDA graph, or NCCL between graphs")
    ap.add_argument("--no-fuse", dest="no_fuse", action="store_true",
                    help="run the normalisations, the gated activation and the residual sums as separate torch kernels")
    ap.add_argument("--out", default=None, help="also append the JSON line to this file")
    a = ap.parse_args()
    a.head_dim = a.hidden // a.heads
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    res = run(a, rank, world, dev, eager=a.eager)
    if rank == 0:
        res.pop("tokens")
        line = json.dumps(res)
        print(line)
        if a.out:
            with open(a.out, "a") as f:
                f.write(line + "\n")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
