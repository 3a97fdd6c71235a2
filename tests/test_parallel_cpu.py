"""Sharding logic on CPU ranks (gloo, world size 2): the per-rank kernels are the CPU oracle injected through the
``ops`` argument, so only the host-side partitioning, collectives and reassembly are under test."""
import os
import types

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from blockwise_int8_linear_b200 import parallel as P

BLOCK = 64


def _oracle_ops():
    import block_linear_config as cfg
    from oracle import blockwise_int8_oracle as O
    return types.SimpleNamespace(
        quantize_block_rowwise=lambda x, b=None: O.quantize(x, b or cfg.GROUP_SIZE),
        int8_matmul_block64_rowwise_dequantize=lambda a, b, sx, sw, bias=None: O.gemm(
            a, b, sx, sw, bias, cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE),
    )


def test_block_aligned_bounds():
    b = P.block_aligned_bounds(11008, 8, 64)
    assert [hi - lo for lo, hi in b] == [22 * 64] * 4 + [21 * 64] * 4
    assert b[0][0] == 0 and b[-1][1] == 11008 and all(lo % 64 == 0 for lo, _ in b)
    assert P.block_aligned_bounds(4096, 8, 64) == [(i * 512, (i + 1) * 512) for i in range(8)]
    assert P.block_aligned_bounds(150, 2, 64) == [(0, 128), (128, 150)]          # ragged tail stays on the last rank
    assert P.block_aligned_bounds(64, 4, 64) == [(0, 64), (64, 64), (64, 64), (64, 64)]
    with pytest.raises(ValueError):
        P.block_aligned_bounds(10, 0, 64)


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import block_linear_config as cfg
        from oracle import blockwise_int8_oracle as O
        cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE = BLOCK, torch.bfloat16
        ops = _oracle_ops()
        x = O.synthetic((48, 320), 1)
        w = O.synthetic((200, 320), 2, std=0.05)          # N = 200: uneven column shards (128 + 72)
        bias = O.synthetic((200,), 3, outlier_frac=0)
        full = O.linear_forward(x, w, bias, BLOCK)

        # column parallel: bit-identical to the unsharded columns
        ws, bs, (lo, hi) = P.shard_columns(w, bias, rank, world, BLOCK)
        wq, sw = O.quantize(ws, BLOCK)
        sizes = [b - a for a, b in P.block_aligned_bounds(200, world, BLOCK)]
        y = P.column_parallel_forward(x, wq, sw, bs, gather=True, sizes=sizes, ops=ops)
        assert torch.equal(y, full), "column-parallel result differs"
        y_local = P.column_parallel_forward(x, wq, sw, bs, gather=False, ops=ops)
        assert torch.equal(y_local, full[:, lo:hi])

        # row parallel: K = 320 = 5 blocks -> 3 + 2 blocks
        ws, (lo, hi) = P.shard_rows(w, rank, world, BLOCK)
        assert lo % BLOCK == 0
        wq, sw = O.quantize(ws, BLOCK)
        y = P.row_parallel_forward(x[:, lo:hi].contiguous(), wq, sw, bias, ops=ops)
        assert cfg.INPUT_OUTPUT_TORCH_TYPE == torch.bfloat16            # knob restored
        d = (y.float() - full.float()).abs().max().item()
        assert d <= 2.0 ** -7 * full.float().abs().max().item(), d      # one bf16 step at the largest magnitude
        same = (y == full).float().mean().item()
        assert same > 0.98, same

        # data parallel: gradient averaging
        torch.manual_seed(rank)
        lin = torch.nn.Linear(16, 8)
        lin(torch.randn(4, 16)).sum().backward()
        mine = [p.grad.clone() for p in lin.parameters()]
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        calls = P.allreduce_gradients(list(lin.parameters()), bucket_bytes=64)
        assert calls >= 1
        for i, p in enumerate(lin.parameters()):
            expect = sum(g[i] for g in gathered) / world
            assert torch.allclose(p.grad, expect, atol=1e-6)
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_sharded_layers_world2():
    world = 2
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    results = mgr.dict()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(results) == {0: "ok", 1: "ok"}


def _llama_worker(rank, world, port, results):
    """The Llama-architecture driver of examples/ at toy size on CPU ranks: its tensor-parallel result against its own
    one-rank result, with the CPU oracle standing in for the CUDA kernels (the driver takes an `ops` namespace)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import argparse
        import importlib.util
        import block_linear_config as cfg
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        spec = importlib.util.spec_from_file_location("llama_infer", os.path.join(root, "examples", "llama_infer.py"))
        L = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(L)
        cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE = BLOCK, torch.bfloat16
        ops = _oracle_ops()
        # FFN 704 = 11 blocks: the split over 2 ranks is uneven (6 + 5 blocks); vocab 520: 5 + 4 blocks, ragged tail
        a = argparse.Namespace(layers=2, hidden=256, heads=4, head_dim=64, ffn=704, vocab=520, batch=2, prompt=12, decode=2, block=BLOCK)
        cpu = torch.device("cpu")
        one = L.Llama(a, cpu, 0, 1, ops=ops)
        two = L.Llama(a, cpu, rank, world, ops=ops)
        ids = torch.randint(0, a.vocab, (a.batch, a.prompt), generator=torch.Generator().manual_seed(4000))
        max_len = a.prompt + a.decode
        ref = one(ids, 0, max_len)
        got = two(ids, 0, max_len)
        assert tuple(got.shape) == tuple(ref.shape) == (a.batch, 1, a.vocab)
        d = (got.float() - ref.float()).abs().max().item()
        assert d <= 2.0 ** -6 * ref.float().abs().max().item(), d
        assert (got == ref).float().mean().item() > 0.5
        # column-parallel layers: this rank's columns are bit-identical to the same columns of the unsharded layer
        x = torch.randn((3, 5, a.hidden), generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
        full = one.layers[0].gate_up(x)
        mine = two.layers[0].gate_up(x)
        lo, hi = P.block_aligned_bounds(a.ffn, world, BLOCK)[rank]
        assert torch.equal(mine, torch.cat([full[..., lo:hi], full[..., a.ffn + lo:a.ffn + hi]], dim=-1))
        # row-parallel layer: the sum of the ranks' fp32 partial results against the unsharded layer
        h = torch.randn((3, 5, a.ffn), generator=torch.Generator().manual_seed(10)).to(torch.bfloat16)
        y_full = one.layers[0].down(h)
        y_tp = two.layers[0].down(h[..., lo:hi].contiguous())
        d = (y_tp.float() - y_full.float()).abs().max().item()
        assert d <= 2.0 ** -7 * y_full.float().abs().max().item(), d
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_llama_driver_tensor_parallel_world2_equals_one_rank():
    world = 2
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    results = mgr.dict()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_llama_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(results) == {0: "ok", 1: "ok"}


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("count", [4, 1000, 1024, 4096 * 7 + 8, 300 * 4096, 4096 * 4096])
def test_prefill_sized_peer_sum_covers_every_chunk_once(world, count):
    """The index arithmetic of bi8_peer_allreduce_large, restated on the host (the kernel itself needs peer-mapped GPUs):
    chunk c of 1024 values belongs to rank c mod world; a rank's CTA b takes the rank's chunks b, b + grid, ... in groups of
    U = 8 / W per loop iteration.  Over all ranks, CTAs and iterations every chunk must come up exactly once, whatever the
    grid size the launcher picked, and no element index may pass `count`."""
    chunk = 1024
    chunks = -(-count // chunk)
    w_bound = 2 if world <= 2 else (4 if world <= 4 else 8)
    u = 8 // w_bound
    my_chunks = -(-chunks // world)
    seen = [0] * chunks
    for sms_times_occupancy in (1, 7, 148 * 3):
        seen = [0] * chunks
        want = -(-my_chunks // u)
        grid = max(1, min(want, sms_times_occupancy))
        for rank in range(world):
            for block in range(grid):
                k0 = block
                while rank + world * k0 < chunks:
                    for j in range(u):
                        c = rank + world * (k0 + j * grid)
                        if c < chunks:
                            assert c % world == rank
                            assert c * chunk < count          # the chunk's first element exists; the tail is cut per thread
                            seen[c] += 1
                    k0 += grid * u
        assert seen == [1] * chunks, (world, count, grid)
