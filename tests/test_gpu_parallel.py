"""Tensor-parallel sharding on real GPUs over NCCL (needs two): the Llama-architecture driver at toy size, two ranks
against one rank, with the CUDA kernels (the gloo tests on CPU ranks use the oracle in their place)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

BLOCK = 64


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import argparse
        import importlib.util
        import block_linear_config as cfg
        from blockwise_int8_linear_b200 import _lib
        from blockwise_int8_linear_b200 import parallel as P
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        spec = importlib.util.spec_from_file_location("llama_infer", os.path.join(root, "examples", "llama_infer.py"))
        L = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(L)
        cfg.GROUP_SIZE, cfg.INPUT_OUTPUT_TORCH_TYPE = BLOCK, torch.bfloat16
        # FFN 704 = 11 blocks: the split over 2 ranks is uneven (6 + 5 blocks); vocab 520: 5 + 4 blocks, ragged tail
        a = argparse.Namespace(layers=2, hidden=256, heads=4, head_dim=64, ffn=704, vocab=520, batch=2, prompt=12, decode=2, block=BLOCK)
        one = L.Llama(a, dev, 0, 1)
        two = L.Llama(a, dev, rank, world)
        ids = torch.randint(0, a.vocab, (a.batch, a.prompt), generator=torch.Generator().manual_seed(4000)).to(dev)
        max_len = a.prompt + a.decode
        ref = one(ids, 0, max_len)
        got = two(ids, 0, max_len)
        assert tuple(got.shape) == tuple(ref.shape) == (a.batch, 1, a.vocab)
        d = (got.float() - ref.float()).abs().max().item()
        assert d <= 2.0 ** -6 * ref.float().abs().max().item(), d
        # every rank ends with the same logits (the gather pads the uneven vocabulary shards)
        both = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(both, got.contiguous())
        assert torch.equal(both[0], both[1])
        # column-parallel layers: this rank's columns are bit-identical to the same columns of the unsharded layer
        x = torch.randn((3, 5, a.hidden), generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).to(dev)
        full = one.layers[0].gate_up(x)
        mine = two.layers[0].gate_up(x)
        lo, hi = P.block_aligned_bounds(a.ffn, world, BLOCK)[rank]
        assert torch.equal(mine, torch.cat([full[..., lo:hi], full[..., a.ffn + lo:a.ffn + hi]], dim=-1))
        # row-parallel layer: the NCCL sum of the ranks' fp32 partial results against the unsharded layer
        h = torch.randn((3, 5, a.ffn), generator=torch.Generator().manual_seed(10)).to(torch.bfloat16).to(dev)
        y_full = one.layers[0].down(h)
        y_tp = two.layers[0].down(h[..., lo:hi].contiguous())
        d = (y_tp.float() - y_full.float()).abs().max().item()
        assert d <= 2.0 ** -7 * y_full.float().abs().max().item(), d
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def _peer_worker(rank, world, port, results):
    """The library's peer-memory reduction against NCCL's all-reduce on the same partial results, eager and replayed from a
    CUDA graph; all ranks must end with bit-identical sums."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import block_linear_config as cfg
        from blockwise_int8_linear_b200 import _lib
        from blockwise_int8_linear_b200.peer import PeerAllReduce
        cfg.INPUT_OUTPUT_TORCH_TYPE = torch.bfloat16
        peer = PeerAllReduce(70 * 4096, dev)
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        bias = torch.randn(4096, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).to(torch.bfloat16)
        for m, n in ((8, 4096), (3, 1000), (1, 4)):
            for it in range(5):                                   # odd count: both buffer sets, then the first again
                part = torch.randn((m, n), device=dev, generator=g)
                ref = part.clone()
                dist.all_reduce(ref)
                got = peer(part, bias[:n] if it % 2 else None)
                want = ref.to(torch.bfloat16)
                if it % 2:
                    want = want + bias[:n]
                # NCCL may add the ranks in another order: one bf16 step at most
                assert (got.float() - want.float()).abs().max().item() <= 2.0 ** -7 * want.float().abs().max().item()
                both = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(both, got)
                assert torch.equal(both[0], both[1])
                if world == 2 and it % 2 == 0:
                    parts = [torch.empty_like(part) for _ in range(world)]
                    dist.all_gather(parts, part)
                    assert torch.equal(got, (parts[0] + parts[1]).to(torch.bfloat16))      # rank order, fp32
        # the whole row-parallel layer in one call (the GEMM's reduction kernel exchanges its sums itself) against the two
        # steps: tiles divided over CTAs (N = 4096), whole tiles (N = 15360), more than 64 rows (two-step path inside)
        from triton_functions import quantize_block_rowwise, quantize_matmul_block_rowwise_dequantize
        cfg.GROUP_SIZE = 64
        for m, k, n in ((8, 2048, 4096), (5, 1408, 15360), (33, 1024, 4096), (70, 1024, 4096)):
            w = (torch.randn((n, k), device=dev, generator=g) * 0.02).to(torch.bfloat16)
            wq, sw = quantize_block_rowwise(w)
            x = torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16)
            cfg.INPUT_OUTPUT_TORCH_TYPE = torch.float32
            part = quantize_matmul_block_rowwise_dequantize(x, wq.t(), sw)
            cfg.INPUT_OUTPUT_TORCH_TYPE = torch.bfloat16
            want = peer(part, bias[:n] if n <= 4096 else None)
            got = peer.row_parallel_linear(x, wq, sw, bias[:n] if n <= 4096 else None)
            assert torch.equal(got, want), (m, k, n, (got.float() - want.float()).abs().max().item())
        # the gated activation in front of the quantizer and the residual behind the sum, in the same call
        import torch.nn.functional as F
        for m, k, n in ((8, 2048, 4096), (70, 1024, 4096)):
            w = (torch.randn((n, k), device=dev, generator=g) * 0.02).to(torch.bfloat16)
            wq, sw = quantize_block_rowwise(w)
            gu = torch.randn((m, 2 * k), device=dev, generator=g).to(torch.bfloat16)
            res = torch.randn((m, n), device=dev, generator=torch.Generator(device=dev).manual_seed(6)).to(torch.bfloat16)
            cfg.INPUT_OUTPUT_TORCH_TYPE = torch.float32
            part = quantize_matmul_block_rowwise_dequantize(F.silu(gu[:, :k]) * gu[:, k:], wq.t(), sw)
            cfg.INPUT_OUTPUT_TORCH_TYPE = torch.bfloat16
            want = peer(part) + res
            assert torch.equal(peer(part, residual=res), want)
            got = peer.row_parallel_linear(gu[:, :k], wq, sw, op="silu_mul", x2=gu[:, k:], residual=res)
            assert torch.equal(got, want), (m, k, n, (got.float() - want.float()).abs().max().item())
        # prefill-sized sums: reduce-scatter by peer loads, all-gather by peer stores, the partial result written into the
        # exchange buffer by the GEMM itself; against the push kernel (same order of the sum: bit-identical) and NCCL
        from blockwise_int8_linear_b200.peer import PeerAllReduceLarge
        from triton_functions import pre_quantize_matmul_block_rowwise_dequantize
        large = PeerAllReduceLarge(300 * 4096, dev)
        small = PeerAllReduce(300 * 4096, dev)
        for it, (m, n) in enumerate(((300, 4096), (64, 1000), (1, 4), (257, 2052), (300, 4096))):
            part = torch.randn((m, n), device=dev, generator=g)
            large.partial(m, n).copy_(part)
            res = torch.randn((m, n), device=dev, generator=torch.Generator(device=dev).manual_seed(8)).to(torch.bfloat16)
            kind = it % 3
            got = large.reduce(m, n, bias=bias[:n] if kind == 1 else None, residual=res if kind == 2 else None).clone()
            want = small(part, bias=bias[:n] if kind == 1 else None, residual=res if kind == 2 else None)
            assert torch.equal(got, want), (m, n, kind, (got.float() - want.float()).abs().max().item())
            ref = part.clone()
            dist.all_reduce(ref)
            ref = ref.to(torch.bfloat16)
            ref = ref + bias[:n] if kind == 1 else (ref + res if kind == 2 else ref)
            assert (got.float() - ref.float()).abs().max().item() <= 2.0 ** -6 * ref.float().abs().max().item()
        # a row-parallel layer at prefill size: the GEMM's fp32 output goes straight into the exchange buffer
        m, k, n = 300, 1024, 4096
        w = (torch.randn((n, k), device=dev, generator=g) * 0.02).to(torch.bfloat16)
        wq, sw = quantize_block_rowwise(w)
        x = torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16)
        cfg.INPUT_OUTPUT_TORCH_TYPE = torch.float32
        part = quantize_matmul_block_rowwise_dequantize(x, wq.t(), sw)
        pre_quantize_matmul_block_rowwise_dequantize("none", x, wq.t(), sw, out=large.partial(m, n))
        cfg.INPUT_OUTPUT_TORCH_TYPE = torch.bfloat16
        assert torch.equal(large.reduce(m, n), small(part))
        # replayed from a graph, output fed back as the next call's residual (a residual stream living in the buffer)
        stream_view = large.reduce(m, n).clone()
        large.partial(m, n).copy_(part)
        gl = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            large.reduce(m, n)
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(gl):
            outv = large.reduce(m, n, residual=large.reduce(m, n))
        expect = small(part)
        expect = small(part, residual=expect)
        for _ in range(3):
            gl.replay()
        torch.cuda.synchronize()
        assert torch.equal(outv, expect)
        del stream_view
        # replayed from a graph: the sequence number continues on the device
        part = torch.randn((8, 4096), device=dev, generator=g)
        out = torch.empty((8, 4096), device=dev, dtype=torch.bfloat16)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            peer(part, out=out)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            peer(part, out=out)
            peer(out.float(), out=out)
        for _ in range(3):
            part.normal_(generator=g)
            graph.replay()
            ref = part.clone()
            dist.all_reduce(ref)
            ref2 = ref.to(torch.bfloat16).float()
            dist.all_reduce(ref2)
            assert (out.float() - ref2).abs().max().item() <= 2.0 ** -6 * ref2.abs().max().item()
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def _spawn(worker, world=2):
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    results = mgr.dict()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():           # a rank that never finished: end exactly that process
            p.kill()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(results) == {r: "ok" for r in range(world)}


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_allreduce_matches_nccl():
    _spawn(_peer_worker)


def test_peer_allreduce_one_rank_and_bounded_wait():
    """On one GPU: a group of one rank is a cast + bias; and with two exchange buffers of which only rank 0 ever runs, rank
    1's flags are never set, so the wait must run out after its (short) limit, the kernel must return, the status word
    must say BI8_ERR_TIMEOUT, and the next call must work."""
    import block_linear_config as cfg
    from blockwise_int8_linear_b200 import _lib
    from blockwise_int8_linear_b200.peer import PeerAllReduce
    from tests.gpu_util import DEV
    cfg.INPUT_OUTPUT_TORCH_TYPE = torch.bfloat16
    part = torch.randn((8, 4096), device=DEV)
    bias = torch.randn(4096, device=DEV).to(torch.bfloat16)
    one = PeerAllReduce(8 * 4096, DEV)
    for _ in range(3):
        assert torch.equal(one(part, bias), part.to(torch.bfloat16) + bias)
    assert _lib.device_status() == 0
    # one rank: the row-parallel layer call is the layer itself
    from triton_functions import quantize_block_rowwise, quantize_matmul_block_rowwise_dequantize
    cfg.GROUP_SIZE = 64
    big = PeerAllReduce(70 * 4096, DEV)
    for m in (8, 40, 70):
        w = (torch.randn((4096, 1024), device=DEV) * 0.02).to(torch.bfloat16)
        wq, sw = quantize_block_rowwise(w)
        x = torch.randn((m, 1024), device=DEV).to(torch.bfloat16)
        assert torch.equal(big.row_parallel_linear(x, wq, sw, bias), quantize_matmul_block_rowwise_dequantize(x, wq.t(), sw, bias))
        gu = torch.randn((m, 2048), device=DEV).to(torch.bfloat16)
        res = torch.randn((m, 4096), device=DEV).to(torch.bfloat16)
        want = res + quantize_matmul_block_rowwise_dequantize(torch.nn.functional.silu(gu[:, :1024]) * gu[:, 1024:], wq.t(), sw)
        assert torch.equal(big.row_parallel_linear(gu[:, :1024], wq, sw, op="silu_mul", x2=gu[:, 1024:], residual=res), want)
    assert _lib.device_status() == 0
    # the prefill-sized kernel with one rank, and its bounded waits with a second rank that never runs
    from blockwise_int8_linear_b200.peer import PeerAllReduceLarge
    big1 = PeerAllReduceLarge(300 * 4096, DEV)
    p300 = torch.randn((300, 4096), device=DEV)
    r300 = torch.randn((300, 4096), device=DEV).to(torch.bfloat16)
    for _ in range(3):
        big1.partial(300, 4096).copy_(p300)
        assert torch.equal(big1.reduce(300, 4096, residual=r300), p300.to(torch.bfloat16) + r300)
        assert torch.equal(big1.reduce(300, 4096, bias=bias), p300.to(torch.bfloat16) + bias)
    assert _lib.device_status() == 0
    alone = PeerAllReduceLarge(8 * 4096, DEV, _local_world=2)
    alone.partial(8, 4096).copy_(part)
    alone.reduce(8, 4096, wait_limit_us=2000)
    with pytest.raises(RuntimeError):
        _lib.device_status()                      # BI8_ERR_TIMEOUT: the other rank's `ready` flag never came
    assert _lib.device_status() == 0
    big1.partial(8, 4096).copy_(part)
    assert torch.equal(big1.reduce(8, 4096), part.to(torch.bfloat16))
    lonely = PeerAllReduce(8 * 4096, DEV, _local_world=2)
    out = torch.full((8, 4096), 7.0, device=DEV, dtype=torch.bfloat16)
    lonely(part, out=out, wait_limit_us=2000)
    with pytest.raises(RuntimeError):
        _lib.device_status()                      # BI8_ERR_TIMEOUT; reading it clears the word
    assert torch.equal(out, torch.full_like(out, 7.0))       # a chunk whose wait ran out writes nothing
    assert _lib.device_status() == 0
    assert torch.equal(one(part, bias), part.to(torch.bfloat16) + bias)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_llama_driver_tensor_parallel_nccl_equals_one_rank():
    _spawn(_worker)
