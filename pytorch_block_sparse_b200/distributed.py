"""Multi-GPU use of the block-sparse Linear: one process per GPU over ``torch.distributed``.

The reference has no multi-process code (its only multi-GPU artefact is a single-process
``nn.DataParallel`` smoke test, ``pytorch_block_sparse/tests/test_data_parallel.py:11-17``).
Two schemes are provided, both plain NCCL collectives around the single-GPU kernels:

* token data parallelism -- every rank holds the same pattern and weights and its own tokens;
  after backward only the nnz-block gradient buffers ``weight.data.grad`` are summed
  (:func:`allreduce_sparse_grads`), and patterns are kept identical with
  :func:`broadcast_sparse_state`.
* column parallelism for one large layer -- the weight's block-rows are partitioned
  (:func:`shard_block_rows`); forward all-gathers the output columns, dgrad sums the partial
  input gradients, wgrad is local (:class:`ColumnParallelBlockSparseLinear`).
"""
import torch
import torch.distributed as dist
import torch.nn as nn

from .block_sparse import BlockSparseMatrix, BlockSparseMatrixBase
from .block_sparse_linear import BlockSparseLinearFunction


def sparse_matrices(model):
    return [m for m in model.modules() if isinstance(m, BlockSparseMatrixBase)]


def broadcast_sparse_state(model, src=0, group=None):
    """Make every rank's pattern and values those of ``src``: broadcasts ``data`` and the five index
    buffers of every block-sparse matrix.  Needed after construction (patterns come from each
    process's numpy RNG) and after a ``SparseOptimizer.step`` that was not seeded identically."""
    for m in sparse_matrices(model):
        with torch.no_grad():
            dist.broadcast(m.data, src, group=group)
        for name in m._INDEX_BUFFERS:
            buf = getattr(m, name)
            dist.broadcast(buf, src, group=group)
            buf.add_(0)  # bump the version counter: cached launch plans are keyed on it
        m._plan_cache = {}
        m._pack_cache = {}


def allreduce_sparse_grads(model, group=None, average=True):
    """Sum (or average) ``data.grad`` of every block-sparse matrix across ranks through one flat buffer:
    only the stored blocks travel, ``density`` times the bytes of the dense gradient."""
    grads = [m.data.grad for m in sparse_matrices(model) if m.data.grad is not None]
    if not grads:
        return 0
    flat = torch.cat([g.reshape(-1) for g in grads])
    dist.all_reduce(flat, group=group)
    if average:
        flat /= dist.get_world_size(group)
    off = 0
    for g in grads:
        g.copy_(flat[off : off + g.numel()].view_as(g))
        off += g.numel()
    return flat.numel() * flat.element_size()


def shard_block_rows(matrix, rank, world, cls=None):
    """The block-rows ``[rank*X/world, (rank+1)*X/world)`` of ``matrix`` as a matrix of its own
    (same columns).  Slots keep their relative order, so concatenating the shards' ``to_dense()``
    along dim 0 gives back ``matrix.to_dense()``."""
    X, Y = matrix.blocks_count()
    if X % world != 0:
        raise Exception("block-row count %d is not divisible by world size %d" % (X, world))
    bh, bw = matrix.block_shape
    per = X // world
    coo = matrix.build_coo_block_index().long()  # [2, nnz] in slot order
    mine = ((coo[0] >= rank * per) & (coo[0] < (rank + 1) * per)).nonzero().squeeze(-1)
    rows = coo[0, mine] - rank * per
    cols = coo[1, mine]
    mask = torch.zeros((per, Y), dtype=torch.bool, device=matrix.data.device)
    mask[rows, cols] = True
    data = matrix.data.detach().view(-1, bh, bw)[mine].reshape(-1, bw).clone()
    # slot i of the shard holds the i-th selected block; block_ptr lists slots in row-major position order
    block_ptr = torch.argsort(rows * Y + cols)  # the i-th set position (row-major) is stored in slot block_ptr[i]
    cls = cls or type(matrix)
    shard = cls((per * bh, matrix.shape[1]), mask, data, matrix.block_shape)
    shard.rebuild(mask, block_ptr)
    return shard


class _GatherColumns(torch.autograd.Function):
    """all-gather along the last dim in forward, slice of the incoming gradient in backward."""

    @staticmethod
    def forward(ctx, y_local, group):
        world = dist.get_world_size(group)
        ctx.rank = dist.get_rank(group)
        ctx.width = y_local.shape[-1]
        # gather [world, ..., n_local] then interleave to [..., world * n_local]
        parts = [torch.empty_like(y_local) for _ in range(world)]
        dist.all_gather(parts, y_local.contiguous(), group=group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, grad):
        lo = ctx.rank * ctx.width
        return grad[..., lo : lo + ctx.width].contiguous(), None


class _SumInputGrad(torch.autograd.Function):
    """identity in forward, all-reduce of the gradient in backward (partial dX of each shard)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous()
        dist.all_reduce(grad, group=ctx.group)
        return grad, None


class ColumnParallelBlockSparseLinear(nn.Module):
    """One large block-sparse Linear split by output features over the ranks of ``group``.

    Built on every rank from the same full ``weight`` (and ``bias``); keeps only its shard.
    ``forward(x)`` takes the replicated input and returns the full output on every rank."""

    def __init__(self, weight, bias=None, group=None):
        super().__init__()
        self.group = group
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.weight = shard_block_rows(weight, rank, world)
        n_local = self.weight.shape[0]
        if bias is not None:
            self.bias = nn.Parameter(bias.detach()[rank * n_local : (rank + 1) * n_local].clone())
        else:
            self.register_parameter("bias", None)
        self.fn = BlockSparseLinearFunction.apply

    def forward(self, x):
        x = _SumInputGrad.apply(x, self.group)
        if isinstance(self.weight, BlockSparseMatrix):
            y = self.fn(x, self.weight.get_differentiable_data(), self.weight, self.bias)
        else:
            y = self.fn(x, self.weight.get_differentiable_data(), self.weight)
            if self.bias is not None:
                y = y + self.bias
        return _GatherColumns.apply(y, self.group)
