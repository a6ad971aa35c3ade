"""Two-GPU NCCL test of the multi-GPU layers with the real kernels: the column-parallel layer (block-rows
split over the ranks) must reproduce the unsharded layer's output, input gradient and its shard of the
weight gradient, also with the all-gather and the reduce-scatter fused into the kernels (NVLink peer stores and
reductions); token data parallelism must all-reduce the nnz-block gradients to the sum over ranks.
One process per GPU, rendezvous on 127.0.0.1.  Skipped with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, results):
    from pytorch_block_sparse_b200 import BlockSparseLinear, BlockSparseMatrix, native
    from pytorch_block_sparse_b200 import distributed as bsd

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        # identical full matrix on every rank
        np.random.seed(11)
        torch.manual_seed(11)
        full = BlockSparseMatrix.zeros((512, 384), n_blocks=70, device=dev)
        with torch.no_grad():
            full.data.copy_((torch.randn(full.data.shape) * 0.02).to(dev))
        bias = (torch.randn(512) * 0.02).to(dev)
        x = torch.randn(300, 384).to(dev)
        g = torch.randn(300, 512).to(dev)

        # unsharded result on this rank
        y_ref = full.reverse_matmul(x, transpose=True, bias=bias)
        dx_ref = full.reverse_matmul(g, transpose=False)
        dw_ref = full.matmul_with_output_sparse_support(g, x)

        layer = bsd.ColumnParallelBlockSparseLinear(full, bias)
        xr = x.clone().requires_grad_(True)
        y = layer(xr)
        y.backward(g)
        torch.cuda.synchronize()

        def rel(a, b):
            return float((a.double() - b.double()).norm() / b.double().norm())

        ok_fwd = rel(y, y_ref) < 2e-6
        ok_dx = rel(xr.grad, dx_ref) < 2e-6
        # the shard's gradient is the full gradient at the shard's blocks: compare through dense matrices
        per = 512 // world
        shard_dense = layer.weight.to_dense(data_replace=layer.weight.data.grad)
        full_dense = full.to_dense(data_replace=dw_ref)[rank * per:(rank + 1) * per]
        ok_dw = rel(shard_dense, full_dense) < 2e-6

        # the same layer with the all-gather fused into the forward kernel: every rank's epilogue stores its columns
        # into every rank's full-width output over NVLink peer mappings (symmetric memory), no NCCL all-gather
        fused = bsd.ColumnParallelBlockSparseLinear(full, bias, fused_gather=True)
        xf = x.clone().requires_grad_(True)
        yf = fused(xf)
        ok_fused = rel(yf, y_ref) < 2e-6 and tuple(yf.shape) == (300, 512)
        yf.backward(g)
        torch.cuda.synchronize()
        ok_fused = ok_fused and rel(xf.grad, dx_ref) < 2e-6
        ok_fused = ok_fused and rel(fused.weight.to_dense(data_replace=fused.weight.data.grad), full_dense) < 2e-6
        # rows of 64 blocks (two promotions per row: the tile leaves for the peers after its sum is complete), twice
        # in a row through the same symmetric buffer
        np.random.seed(13)
        torch.manual_seed(13)
        long_rows = BlockSparseMatrix.zeros((256, 2048), n_blocks=8 * 64, device=dev)
        with torch.no_grad():
            long_rows.data.copy_((torch.randn(long_rows.data.shape) * 0.02).to(dev))
        fused2 = bsd.ColumnParallelBlockSparseLinear(long_rows, None, fused_gather=True)
        for seed in (21, 22):
            x2 = torch.randn(150, 2048, generator=torch.Generator().manual_seed(seed)).to(dev)
            want = long_rows.reverse_matmul(x2, transpose=True)
            ok_fused = ok_fused and rel(fused2(x2), want) < 4e-6

        # the input gradient fused with a reduce-scatter over tokens (peer reductions from the dgrad epilogue) and
        # completed by an all-gather, instead of an all-reduce of the partial gradients; 512 tokens = 2 x 256
        ok_reduce = True
        x3 = torch.randn(512, 384, generator=torch.Generator().manual_seed(31)).to(dev)
        g3 = torch.randn(512, 512, generator=torch.Generator().manual_seed(32)).to(dev)
        both = bsd.ColumnParallelBlockSparseLinear(full, bias, fused_gather=True, fused_reduce=True)
        for _ in range(2):  # twice through the same symmetric shard buffer
            xb = x3.clone().requires_grad_(True)
            yb = both(xb)
            ok_reduce = ok_reduce and rel(yb, full.reverse_matmul(x3, transpose=True, bias=bias)) < 2e-6
            yb.backward(g3)
            torch.cuda.synchronize()
            ok_reduce = ok_reduce and rel(xb.grad, full.reverse_matmul(g3, transpose=False)) < 2e-6
        # columns with 64 blocks per shard: the partial sum of a row leaves tensor memory in two parts, and the
        # completed total is what travels
        np.random.seed(14)
        torch.manual_seed(14)
        tall = BlockSparseMatrix.zeros((4096, 64), n_blocks=128 * 2, device=dev)
        with torch.no_grad():
            tall.data.copy_((torch.randn(tall.data.shape) * 0.02).to(dev))
        both2 = bsd.ColumnParallelBlockSparseLinear(tall, None, fused_gather=True, fused_reduce=True)
        x4 = torch.randn(256, 64, generator=torch.Generator().manual_seed(33)).to(dev).requires_grad_(True)
        g4 = torch.randn(256, 4096, generator=torch.Generator().manual_seed(34)).to(dev)
        both2(x4).backward(g4)
        torch.cuda.synchronize()
        ok_reduce = ok_reduce and rel(x4.grad, tall.reverse_matmul(g4, transpose=False)) < 4e-6
        # a token count the shards cannot split evenly falls back to the all-reduce
        x5 = torch.randn(300, 384, generator=torch.Generator().manual_seed(35)).to(dev).requires_grad_(True)
        both(x5).backward(g)
        torch.cuda.synchronize()
        ok_reduce = ok_reduce and rel(x5.grad, dx_ref) < 2e-6

        # token data parallelism: same layer everywhere, own tokens, gradients summed over the ranks
        np.random.seed(12)
        torch.manual_seed(12)
        lin = BlockSparseLinear(384, 256, bias=True, density=0.3).to(dev)
        bsd.broadcast_sparse_state(lin, src=0)
        tok = torch.randn(200, 384, generator=torch.Generator().manual_seed(100 + rank)).to(dev)
        gy = torch.randn(200, 256, generator=torch.Generator().manual_seed(200 + rank)).to(dev)
        lin(tok).backward(gy)
        local = lin.weight.data.grad.clone()
        bsd.allreduce_sparse_grads(lin, average=False)
        gathered = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        ok_ar = rel(lin.weight.data.grad, sum(gathered)) < 1e-6
        # the same sum through this library's peer-memory all-reduce kernel (symmetric memory instead of NCCL)
        reducer = bsd.PeerAllReduce(local.numel(), dev)
        lin.weight.data.grad.copy_(local)
        bsd.allreduce_sparse_grads_peer(lin, reducer, average=False)
        torch.cuda.synchronize()
        ok_ar = ok_ar and rel(lin.weight.data.grad, sum(gathered)) < 1e-6
        bits = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(bits, lin.weight.data.grad)
        ok_ar = ok_ar and all(torch.equal(b, bits[0]) for b in bits)  # every rank holds the same bits
        results[rank] = (ok_fwd, ok_dx, ok_dw, ok_ar, ok_fused, ok_reduce, native.device_status() == 0)
    finally:
        dist.destroy_process_group()


def test_two_gpus_column_parallel_and_token_dp():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        for rank in range(world):
            assert results[rank] == (True, True, True, True, True, True, True), (rank, results[rank])
