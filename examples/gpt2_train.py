"""GPT-2-small training with BlockInt8Linear in forward and backward (dX and dW are blockwise-int8 GEMMs too).

The reference's training example (``examples/train_gpt2``) is an empty submodule and its dataset is unknown, so this driver
builds GPT-2 small (12 layers, d = 768, 12 heads, vocab 50257, sequence 1024) from ``nn.Linear`` layers, swaps them with
``replace_linear_with_blockwise_int8`` and trains on uniform random token ids: batch 8 per GPU, bf16 parameters and
activations, AdamW at 3e-4.  Data parallel over N GPUs with torch's DistributedDataParallel (NCCL gradient all-reduce
overlapped with the backward pass).

    python examples/gpt2_train.py --steps 10
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 examples/gpt2_train.py --steps 10
"""
from __future__ import annotations

import argparse
import json
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
from block_linear import replace_linear_with_blockwise_int8  # noqa: E402


class Block(nn.Module):
    def __init__(self, d, heads):
        super().__init__()
        self.heads = heads
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc, self.out = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)

    def forward(self, x):
        B, T, D = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.heads, D // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, D)
        x = x + self.proj(a)
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, layers=12, d=768, heads=12, vocab=50257, seq=1024):
        super().__init__()
        self.wte, self.wpe = nn.Embedding(vocab, d), nn.Embedding(seq, d)
        self.blocks = nn.ModuleList(Block(d, heads) for _ in range(layers))
        self.ln_f = nn.LayerNorm(d)
        self.lm_head = nn.Linear(d, vocab, bias=False)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)

    def forward(self, ids):
        T = ids.shape[1]
        x = self.wte(ids) + self.wpe(torch.arange(T, device=ids.device))
        for b in self.blocks:
            x = b(x)
        return self.lm_head(self.ln_f(x))


def run(a, rank, world, local, dev):
    """Trains the model described by `a` (fields as the command line options below) for a.warmup + a.steps steps on this
    rank and returns the measurements.  The process group, if any, is the caller's."""
    cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE = a.block, torch.bfloat16
    torch.manual_seed(0)
    model = GPT2(layers=a.layers, seq=a.seq).to(dev).to(torch.bfloat16)
    if not a.dense:
        model.apply(replace_linear_with_blockwise_int8)
    model.train()
    net = nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4)
    g = torch.Generator().manual_seed(5000 + rank)
    losses = []

    def step():
        ids = torch.randint(0, 50257, (a.batch, a.seq + 1), generator=g).to(dev, non_blocking=True)
        logits = net(ids[:, :-1])
        loss = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss.detach()

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        losses.append(step())
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    dt = time.perf_counter() - t0
    return {
        "model": f"gpt2-small-arch {a.layers} layers, seq {a.seq}, {'nn.Linear bf16' if a.dense else f'BlockInt8Linear block {a.block} fwd+bwd'}",
        "n_gpus": world, "batch_per_gpu": a.batch, "steps": a.steps,
        "tokens_per_s": world * a.batch * a.seq * a.steps / dt, "ms_per_step": 1e3 * dt / a.steps,
        "loss_first": float(losses[0]), "loss_last": float(losses[-1]),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--block", type=int, default=64)
    ap.add_argument("--dense", action="store_true", help="keep nn.Linear (bf16 cuBLAS) for comparison")
    ap.add_argument("--out", default=None, help="also append the JSON line to this file")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    res = run(a, rank, world, local, dev)
    if rank == 0:
        line = json.dumps(res)
        print(line)
        if a.out:
            with open(a.out, "a") as f:
                f.write(line + "\n")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
