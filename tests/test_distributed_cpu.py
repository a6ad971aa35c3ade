"""World-size-2 gloo tests (CPU) of the multi-GPU host logic: block-row sharding, the column-parallel
layer's collectives, the flat nnz-gradient all-reduce and pattern broadcast.  The dense-masked
emulator class stands in for the CUDA kernels so the plumbing runs without a GPU."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pytorch_block_sparse_b200 import BlockSparseMatrix, BlockSparseMatrixEmulator
from pytorch_block_sparse_b200 import distributed as bsd


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        np.random.seed(7)
        torch.manual_seed(7)
        full = BlockSparseMatrixEmulator.randn((128, 96), 6, block_shape=(32, 32), device="cpu")
        bias = torch.randn(128)
        dense = full.to_dense().detach().clone()

        # --- column-parallel layer: forward output and input gradient equal the unsharded layer's
        layer = bsd.ColumnParallelBlockSparseLinear(full, bias)
        x = torch.randn(5, 7, 96, requires_grad=True)
        y = layer(x)
        want = x.detach() @ dense.t() + bias
        ok_fwd = torch.allclose(y, want, atol=1e-5)
        g = torch.randn(5, 7, 128)
        y.backward(g)
        ok_dx = torch.allclose(x.grad, g @ dense, atol=1e-5)
        # local wgrad is the shard's rows of the full masked gradient
        per = 128 // world
        full_dw = (g.reshape(-1, 128).t() @ x.detach().reshape(-1, 96)) * (dense != 0)
        ok_dw = torch.allclose(layer.weight._dense.grad, full_dw[rank * per:(rank + 1) * per], atol=1e-4)

        # --- token-DP: flat all-reduce of data.grad
        np.random.seed(3)
        m = BlockSparseMatrix.randn((64, 64), 3, device="cpu")
        m.data.grad = torch.full_like(m.data, float(rank + 1))
        holder = torch.nn.ModuleList([m])
        nbytes = bsd.allreduce_sparse_grads(holder, average=False)
        ok_ar = bool((m.data.grad == sum(range(1, world + 1))).all()) and nbytes == m.data.numel() * 4

        # --- pattern broadcast: ranks start from different patterns, end with rank 0's
        np.random.seed(100 + rank)
        torch.manual_seed(100 + rank)
        p = BlockSparseMatrix.randn((128, 128), 5, device="cpu")
        holder = torch.nn.ModuleList([p])
        bsd.broadcast_sparse_state(holder, src=0)
        gathered = [torch.zeros_like(p.to_dense()) for _ in range(world)]
        dist.all_gather(gathered, p.to_dense().detach())
        ok_bc = all(torch.equal(gathered[0], t) for t in gathered)
        results[rank] = (ok_fwd, ok_dx, ok_dw, ok_ar, ok_bc)
    finally:
        dist.destroy_process_group()


def test_world_size_2_gloo():
    world = 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        for rank in range(world):
            assert results[rank] == (True, True, True, True, True), (rank, results[rank])


def test_shards_reassemble_to_the_full_matrix():
    np.random.seed(11)
    torch.manual_seed(11)
    full = BlockSparseMatrix.randn((256, 160), 17, device="cpu")
    # permute slots first so that slot order differs from position order
    free = (~full.block_mask_build(None)).nonzero()
    full.block_replace(torch.tensor([[int(free[0, 0]), int(free[0, 1]), 4], [int(free[5, 0]), int(free[5, 1]), 0]]))
    for world in (1, 2, 4, 8):
        shards = [bsd.shard_block_rows(full, r, world) for r in range(world)]
        assert sum(s.data.shape[0] for s in shards) == full.data.shape[0]
        assert torch.equal(torch.cat([s.to_dense() for s in shards], 0), full.to_dense())
