"""Multi-GPU use of the block-sparse Linear: one process per GPU over ``torch.distributed``.

The reference has no multi-process code (its only multi-GPU artefact is a single-process
``nn.DataParallel`` smoke test, ``pytorch_block_sparse/tests/test_data_parallel.py:11-17``).
Two schemes are provided, as plain NCCL collectives around the single-GPU kernels and, for the sharded layer,
with the collectives fused into the kernels (peer stores / peer reductions over NVLink from the epilogue):

* token data parallelism -- every rank holds the same pattern and weights and its own tokens;
  after backward only the nnz-block gradient buffers ``weight.data.grad`` are summed
  (:func:`allreduce_sparse_grads` over NCCL, :class:`PeerAllReduce` with this library's own kernel), and
  patterns are kept identical with :func:`broadcast_sparse_state`.
* column parallelism for one large layer -- the weight's block-rows are partitioned
  (:func:`shard_block_rows`); forward all-gathers the output columns, dgrad sums the partial
  input gradients, wgrad is local (:class:`ColumnParallelBlockSparseLinear`; ``fused_gather`` /
  ``fused_reduce`` move the all-gather and the reduce-scatter half of the all-reduce into the kernels).
"""
import torch
import torch.distributed as dist
import torch.nn as nn

from . import native
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


class PeerAllReduce:
    """In-place all-reduce of one flat fp32 buffer per rank with this library's own kernel over NVLink peer mappings
    (``bsmm_allreduce_peers``) instead of NCCL: a small grid that runs beside the persistent tensor-core kernels, so
    the weight gradients of token data parallelism can travel on a side stream while the input gradient is
    computed.  ``buffer`` lives in symmetric memory; write the gradients into it (or views of it), call the object,
    read the sums from it.  Every rank obtains the same bits (sums in rank order)."""

    def __init__(self, numel, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.numel = (numel + 3) // 4 * 4
        self.buffer = symm_mem.empty(self.numel, dtype=torch.float32, device=device)
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        self._ptrs = [int(self.handle.buffer_ptrs[r]) for r in range(self.world)]
        if self.numel != numel:
            self.buffer[numel:].zero_()

    def __call__(self, average=False):
        self.handle.barrier()  # every rank's buffer is complete
        native.allreduce_peers(self._ptrs, self.rank, self.numel, 1.0 / self.world if average else 1.0, self.buffer.device)
        self.handle.barrier()  # every rank's slice has been stored everywhere
        return self.buffer


def allreduce_sparse_grads_peer(model, reducer, average=True):
    """:func:`allreduce_sparse_grads` through a :class:`PeerAllReduce` of at least the gradients' total size."""
    grads = [m.data.grad for m in sparse_matrices(model) if m.data.grad is not None]
    off = 0
    for g in grads:
        reducer.buffer[off : off + g.numel()].copy_(g.reshape(-1))
        off += g.numel()
    reducer(average=average)
    off = 0
    for g in grads:
        g.copy_(reducer.buffer[off : off + g.numel()].view_as(g))
        off += g.numel()
    return off * 4


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


class PeerOutputs:
    """Full-width output tensors in symmetric memory (one per rank, each mapped into every rank's address space
    over NVLink) for the forward product fused with its all-gather: every rank's kernel stores its column slice
    into all of them.  One tensor per (rows, width, dtype), kept for reuse."""

    def __init__(self, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self._buffers = {}

    def get(self, rows, width, dtype, device, tag="y"):
        import torch.distributed._symmetric_memory as symm_mem

        key = (rows, width, dtype, str(device), tag)
        if key not in self._buffers:
            buf = symm_mem.empty((rows, width), dtype=dtype, device=device)
            handle = symm_mem.rendezvous(buf, self.group)
            self._buffers[key] = (buf, handle)
        return self._buffers[key]


class _FusedColumnParallelFunction(torch.autograd.Function):
    """Forward of this rank's block-row shard with the all-gather fused into the kernel's epilogue (peer stores),
    backward as for the plain shard on this rank's column slice of the incoming gradient.  With ``fused_reduce``
    the input-gradient kernel stores every completed tile of its partial sum into its slot on the rank owning
    those tokens (peer stores from the epilogue: a reduce-scatter without atomics), and a second kernel adds each
    rank's slots in rank order and stores the sums into every rank's gradient tensor -- together an all-reduce of
    the partial gradients with its first half hidden under the product."""

    @staticmethod
    def forward(ctx, input, weight_data, weight, bias, outputs, group, fused_reduce=False):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        n_local = weight.shape[0]
        flat = input.reshape(-1, input.shape[-1])
        if not flat.is_contiguous():
            flat = flat.contiguous()
        packed = weight.packed_weights()
        io16 = flat.dtype == torch.bfloat16 and packed.precision == native.PREC_BF16
        full, handle = outputs.get(flat.shape[0], world * n_local, torch.bfloat16 if io16 else torch.float32, flat.device)
        peers = [int(handle.buffer_ptrs[r]) for r in range(world) if r != rank]
        handle.barrier()  # every rank is done reading the previous contents of its output
        native.dsd_matmul(flat, weight._plan(True), packed, n_local, True, bias=bias, out=full,
                          out_col0=rank * n_local, peer_outs=peers)
        handle.barrier()  # every rank's columns have arrived everywhere
        ctx.save_for_backward(input, weight_data)
        ctx.weight, ctx.packed, ctx.has_bias = weight, packed, bias is not None
        ctx.cols = (rank * n_local, (rank + 1) * n_local)
        ctx.outputs, ctx.group, ctx.fused_reduce = outputs, group, fused_reduce
        return full.view(*input.shape[:-1], world * n_local)

    @staticmethod
    def backward(ctx, grad):
        input, _ = ctx.saved_tensors
        weight = ctx.weight
        g = grad[..., ctx.cols[0]:ctx.cols[1]].contiguous()
        grad_input = grad_weight = grad_bias = None
        if ctx.needs_input_grad[1]:
            grad_weight = weight.matmul_with_output_sparse_support(g, input)
        if ctx.needs_input_grad[0]:
            world = dist.get_world_size(ctx.group)
            gf = g.reshape(-1, g.shape[-1])
            m, k = gf.shape[0], weight.shape[1]
            if ctx.fused_reduce and gf.dtype == torch.float32 and m % (128 * world) == 0 and weight.data.shape[0] > 0:
                rank = dist.get_rank(ctx.group)
                parts, hp = ctx.outputs.get(m, k, torch.float32, gf.device, tag="dx_parts")  # [world, m / world, k]
                total, ht = ctx.outputs.get(m, k, torch.float32, gf.device, tag="dx_sum")
                hp.barrier()  # every rank has summed its slots of the previous call and read its previous total
                native.dsd_scatter(gf, weight._plan(False), ctx.packed, k, False,
                                   [int(hp.buffer_ptrs[r]) for r in range(world)], rank)
                hp.barrier()  # every rank's parts have arrived
                native.sum_row_slots(parts.view(world, m // world, k), [int(ht.buffer_ptrs[r]) for r in range(world)],
                                     rank * (m // world))
                ht.barrier()  # every rank's rows of the sum have arrived
                grad_input = total.clone().view(input.shape)  # the symmetric buffer is reused by the next call
            else:
                grad_input = weight.reverse_matmul(g, transpose=False, packed=ctx.packed)
                if ctx.fused_reduce:
                    grad_input = grad_input.contiguous()
                    dist.all_reduce(grad_input, group=ctx.group)
        if ctx.has_bias and ctx.needs_input_grad[3]:
            grad_bias = g.reshape(-1, g.shape[-1]).sum(0, dtype=torch.float32)
        return grad_input, grad_weight, None, grad_bias, None, None, None


class ColumnParallelBlockSparseLinear(nn.Module):
    """One large block-sparse Linear split by output features over the ranks of ``group``.

    Built on every rank from the same full ``weight`` (and ``bias``); keeps only its shard.
    ``forward(x)`` takes the replicated input and returns the full output on every rank.
    ``fused_gather=True``: the forward kernel stores its columns straight into every rank's full-width output
    (symmetric memory, NVLink peer stores from the epilogue) instead of a separate NCCL all-gather; the returned
    tensor is then a buffer that the next forward of the same shape overwrites.
    ``fused_reduce=True`` (with ``fused_gather``): the input-gradient kernel reduce-scatters its partial sums by
    tokens over NVLink while it computes, and a sum-and-broadcast kernel replaces the all-reduce (token counts
    that are not a multiple of 128 x world size use the all-reduce)."""

    def __init__(self, weight, bias=None, group=None, fused_gather=False, fused_reduce=False):
        super().__init__()
        self.group = group
        self.fused_gather = fused_gather
        self.fused_reduce = fused_reduce and fused_gather
        self._peer_outputs = None
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.weight = shard_block_rows(weight, rank, world)
        n_local = self.weight.shape[0]
        if bias is not None:
            self.bias = nn.Parameter(bias.detach()[rank * n_local : (rank + 1) * n_local].clone())
        else:
            self.register_parameter("bias", None)
        self.fn = BlockSparseLinearFunction.apply

    def forward(self, x):
        if self.fused_gather and isinstance(self.weight, BlockSparseMatrix):
            if self._peer_outputs is None:
                self._peer_outputs = PeerOutputs(self.group)
            if not self.fused_reduce:
                x = _SumInputGrad.apply(x, self.group)
            return _FusedColumnParallelFunction.apply(
                x, self.weight.get_differentiable_data(), self.weight, self.bias, self._peer_outputs, self.group,
                self.fused_reduce,
            )
        x = _SumInputGrad.apply(x, self.group)
        if isinstance(self.weight, BlockSparseMatrix):
            y = self.fn(x, self.weight.get_differentiable_data(), self.weight, self.bias)
        else:
            y = self.fn(x, self.weight.get_differentiable_data(), self.weight)
            if self.bias is not None:
                y = y + self.bias
        return _GatherColumns.apply(y, self.group)
