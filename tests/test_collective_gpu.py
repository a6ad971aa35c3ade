"""The kernels behind the sharded layer's fused collectives, on ONE GPU: two ranks are played one after the other
(their kernels never wait for each other, so sequential launches are a faithful stand-in), with plain local tensors
where a real run passes NVLink peer mappings.  The two-GPU run over NCCL and symmetric memory is
tests/test_distributed_gpu.py."""
import numpy as np
import pytest
import torch

from pytorch_block_sparse_b200 import BlockSparseMatrix, native
from pytorch_block_sparse_b200.distributed import shard_block_rows

from .gpu_util import assert_device_healthy

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def _matrix(shape, n_blocks, seed):
    np.random.seed(seed)
    torch.manual_seed(seed)
    w = BlockSparseMatrix.zeros(shape, n_blocks=n_blocks, device="cuda")
    with torch.no_grad():
        w.data.normal_(0, 0.02)
    return w


@pytest.mark.parametrize("rows,n_blocks,tokens", [(512, 70, 300), (2368, 12, 9000)])
@pytest.mark.parametrize("precision", ["tf32x3", "bf16x3", "tf32", "bf16"])
def test_forward_writes_its_column_slice_to_every_output(precision, rows, n_blocks, tokens):
    # bsmm_dsd_multi: each "rank" writes the columns of its block-row shard into both full-width outputs
    # (second case: a dozen blocks in 74 block-rows -- whole tiles without a block still deliver their bias tiles)
    world = 2
    full = _matrix((rows, 384), n_blocks, 3)
    bias = torch.randn(rows, device="cuda") * 0.02
    x = torch.randn(tokens, 384, device="cuda")
    prec = native.resolve_precision(precision)
    want = full.reverse_matmul(x, transpose=True, bias=bias, precision=precision)
    outs = [torch.full((tokens, rows), float("nan"), device="cuda") for _ in range(world)]
    for rank in range(world):
        shard = shard_block_rows(full, rank, world)
        n_local = shard.shape[0]
        packed = native.pack_weights(shard.data.detach(), prec)
        peers = [outs[r].data_ptr() for r in range(world) if r != rank]
        native.dsd_matmul(x, shard._plan(True), packed, n_local, True, bias=bias[rank * n_local:(rank + 1) * n_local].contiguous(),
                          out=outs[rank], out_col0=rank * n_local, peer_outs=peers)
    torch.cuda.synchronize()
    for out in outs:
        assert torch.equal(out, want)  # same kernel, same operands, same order: bit-identical to the unsharded call
    assert_device_healthy()


@pytest.mark.parametrize("shape,n_blocks,tokens", [((512, 384), 70, 512), ((4096, 64), 256, 256), ((320, 2368), 12, 9216)])
def test_input_gradient_reduce_scatter_and_sum(shape, n_blocks, tokens):
    # bsmm_dsd_scatter + bsmm_sum_row_slots: every rank's partial tiles land in its slot on the owner of the tokens;
    # adding the slots gives the unsharded input gradient.  The second shape has 64 blocks per shard and column:
    # a row's partial sum leaves tensor memory in two parts and only the total travels.
    world = 2
    full = _matrix(shape, n_blocks, 5)
    g = torch.randn(tokens, shape[0], device="cuda")
    want = full.reverse_matmul(g, transpose=False)
    k = shape[1]
    prec = native.resolve_precision("tf32x3")
    parts = [torch.full((world, tokens // world, k), float("nan"), device="cuda") for _ in range(world)]
    totals = [torch.full((tokens, k), float("nan"), device="cuda") for _ in range(world)]
    for rank in range(world):
        shard = shard_block_rows(full, rank, world)
        n_local = shard.shape[0]
        packed = native.pack_weights(shard.data.detach(), prec)
        g_local = g[:, rank * n_local:(rank + 1) * n_local].contiguous()
        native.dsd_scatter(g_local, shard._plan(False), packed, k, False, [p.data_ptr() for p in parts], rank)
    for rank in range(world):
        native.sum_row_slots(parts[rank], [t.data_ptr() for t in totals], rank * (tokens // world))
    torch.cuda.synchronize()
    for total in totals:
        assert not torch.isnan(total).any()
        assert _rel(total, want) < 4e-6
    assert torch.equal(totals[0], totals[1])
    assert_device_healthy()


def test_scatter_rejects_token_counts_it_cannot_split():
    full = _matrix((256, 128), 20, 7)
    g = torch.randn(300, 256, device="cuda")
    packed = native.pack_weights(full.data.detach(), native.resolve_precision("tf32x3"))
    parts = torch.empty(2, 150, 128, device="cuda")
    with pytest.raises(native.NativeError):
        native.dsd_scatter(g, full._plan(False), packed, 128, False, [parts.data_ptr(), parts.data_ptr()], 0)


def test_allreduce_kernel_sums_every_rank_slice():
    # bsmm_allreduce_peers: each "rank" adds its slice of all buffers and stores it into all of them
    world, elems = 3, 4 * 1000 + 8  # slices of unequal length
    bufs = [torch.randn(elems, device="cuda") for _ in range(world)]
    want = sum(b.double() for b in bufs) * 0.5
    ptrs = [b.data_ptr() for b in bufs]
    for rank in range(world):
        native.allreduce_peers(ptrs, rank, elems, 0.5, bufs[0].device)
    torch.cuda.synchronize()
    for b in bufs:
        assert torch.equal(b, bufs[0])
        assert float((b.double() - want).abs().max()) < 1e-5
    assert_device_healthy()
