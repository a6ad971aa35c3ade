"""Block-sparse weight matrix with the reference's storage contract.

Mirrors ``pytorch_block_sparse/block_sparse.py`` of huggingface/pytorch_block_sparse
(class names, method names, argument meaning, buffer names/dtypes and error
behaviour), but the two matmuls are routed to the hand-written sm_100a kernels
behind the C-ABI library (see ``native.py``) instead of the reference's
``block_sparse_native`` pybind module.

Storage contract (reference ``block_sparse.py:10-76``, ``:125-153``, ``:405-429``):

* ``data``  fp32 ``[nnz*bh, bw]``.  Slot ``s`` holds its block **transposed**:
  ``data[s*bh + c, r] == W[R*bh + r, C*bw + c]`` for the block at block-row ``R``,
  block-column ``C`` (square 32x32 blocks on the CUDA path).
* ``cols_a`` int32 ``[nnz, 2]``: ``(block-col, slot)`` in row-major block order,
  ``row_start_ends_a`` int32 ``[X+1]``: CSR offsets over block-rows.
* ``rows_b`` int32 ``[nnz, 2]``: ``(block-row, slot)`` in column-major block order,
  ``col_start_ends_b`` int32 ``[Y+1]``: CSC offsets over block-columns.
* ``blocks`` int32 ``[2*nnz]``: ``(block-col, block-row)`` pairs in **slot** order.
"""
import numpy
import torch
import torch.nn

from . import native


class BlockSparseMatrixBase(torch.nn.Module):
    """Data + index buffers of one block-sparse matrix (reference ``block_sparse.py:6-76``)."""

    _INDEX_BUFFERS = ("cols_a", "row_start_ends_a", "rows_b", "col_start_ends_b", "blocks")

    def __init__(self, shape, block_mask, data, block_shape=(32, 32)):
        super().__init__()
        self.int_type = torch.int32
        if len(shape) != 2:
            raise Exception("shape should be a tuple of 2 ints")
        self.shape = torch.Size(shape)
        if len(block_shape) != 2:
            raise Exception("block_shape should be a tuple of 2 ints")
        self.block_shape = tuple(block_shape)
        self.data = torch.nn.Parameter(data)
        self._plan_cache = {}
        self._pack_cache = {}
        self.last_grad_block_sumsq = None  # per-slot sum of squares of the most recent weight gradient
        self.rebuild(block_mask, callback=False)

    # derived, device-specific caches never travel with a pickle or a replica's state
    def __getstate__(self):
        state = dict(super().__getstate__() if hasattr(super(), "__getstate__") else self.__dict__)
        state["_plan_cache"] = {}
        state["_pack_cache"] = {}
        state.pop("_cells", None)
        return state

    # ------------------------------------------------------------------ hooks
    def updated_data(self):
        pass

    def get_differentiable_data(self):
        return self.data

    # -------------------------------------------------------------- bookkeeping
    @staticmethod
    def blocks_count_(shape, block_shape):
        return torch.Size((shape[0] // block_shape[0], shape[1] // block_shape[1]))

    def blocks_count(self):
        return self.blocks_count_(self.shape, self.block_shape)

    def build_indices(self, block_mask, block_ptr=None):
        """CSR, CSC and slot-order COO of ``block_mask`` (reference ``block_sparse.py:85-153``).

        ``block_ptr[i]`` is the data slot of the i-th set position of ``block_mask`` in
        row-major order; ``None`` means slots follow row-major order.
        Returns ``(blocks, cols_a, row_start_ends_a, rows_b, col_start_ends_b)``, all int32.
        """
        X, Y = self.blocks_count()
        device = block_mask.device
        where = torch.nonzero(block_mask, as_tuple=False)
        brow, bcol = where[:, 0], where[:, 1]
        n = where.shape[0]
        if block_ptr is None:
            slot = torch.arange(n, device=device)
        else:
            slot = block_ptr.to(device=device, dtype=torch.long)

        # slot-order list of (col, row)
        by_slot = torch.argsort(slot)
        blocks = torch.stack([bcol[by_slot], brow[by_slot]], 1).reshape(-1).to(self.int_type)

        def offsets(idx, count):
            out = torch.zeros(count + 1, dtype=torch.long, device=device)
            if n:
                out[1:] = torch.cumsum(torch.bincount(idx, minlength=count), 0)
            return out.to(self.int_type)

        # row-major order is the order nonzero() already returns
        cols_a = torch.stack([bcol, slot], 1).to(self.int_type)
        row_start_ends_a = offsets(brow, X)

        # column-major order
        by_col = torch.argsort(bcol * X + brow)
        rows_b = torch.stack([brow[by_col], slot[by_col]], 1).to(self.int_type)
        col_start_ends_b = offsets(bcol, Y)
        return blocks, cols_a, row_start_ends_a, rows_b, col_start_ends_b

    def rebuild(self, block_mask, block_ptr=None, callback=True):
        """(Re)register the five index buffers for a new pattern (reference ``block_sparse.py:33-76``)."""
        data = self.data
        bs = self.block_shape
        if block_mask.device != data.device:
            raise Exception(
                "block_mask and data should have same device, got %s and %s" % (block_mask.device, data.device)
            )
        blocks, cols_a, row_start_ends_a, rows_b, col_start_ends_b = self.build_indices(block_mask, block_ptr)

        if data.dim() != 2:
            raise Exception("data should be bidimensional, not of shape %s" % data.shape)
        if data.shape[0] != cols_a.shape[0] * bs[0]:
            raise Exception(
                "data.shape[0] (%d) should be equal to cols.shape[0]*block_shape[0] (%d)"
                % (data.shape[0], cols_a.shape[0] * bs[0])
            )
        if data.shape[1] != bs[1]:
            raise Exception("data.shape[1] (%d) should be equal to block_shape[1] (%d)" % (data.shape[1], bs[1]))
        if data.dtype != torch.float32:
            raise Exception("data should be float32, not of type %s" % data.dtype)

        new = dict(
            cols_a=cols_a,
            row_start_ends_a=row_start_ends_a,
            rows_b=rows_b,
            col_start_ends_b=col_start_ends_b,
            blocks=blocks,
        )
        for name in self._INDEX_BUFFERS:
            self.register_buffer(name, new[name])

        self.sanity_check(self.cols_a, self.row_start_ends_a, self.shape, self.block_shape)
        self.sanity_check(self.rows_b, self.col_start_ends_b, self.shape[::-1], self.block_shape[::-1])
        self.check_ = False
        self._plan_cache = {}
        self.__dict__.pop("_cells", None)
        if callback:
            self.updated_data()

    def sanity_check(self, cols, row_end, shape, block_shape):
        """Shape/dtype/range validation of one (indices, offsets) pair (reference ``block_sparse.py:431-463``)."""
        row_end = row_end[1:]
        if cols.dim() != 2:
            raise Exception("cols should be bidimensional, not of shape %s" % cols.shape)
        if cols.dtype != self.int_type:
            raise Exception("cols should be %s, not of type %s" % (self.int_type, cols.dtype))
        if row_end.dim() != 1:
            raise Exception("row_end should be unidimensional, not of shape %s" % row_end.shape)
        if row_end.shape[0] != shape[0] / block_shape[0]:
            raise Exception(
                "row_end.shape[0] (%d) should be equal to shape[0]/block_shape[0] (%d)"
                % (row_end.shape[0], shape[0] / block_shape[0])
            )
        if row_end.dtype != self.int_type:
            raise Exception("row_end should be %s, not of type %s" % (self.int_type, row_end.dtype))
        if cols.shape[0] == 0:
            return
        max_col = cols[:, 0].max()
        if max_col > shape[1] / block_shape[1]:
            raise Exception(
                "cols max element (%d) cannot be larger than shape[1]/block_shape[1] (%d)"
                % (max_col, shape[1] / block_shape[1])
            )
        if row_end.max() > cols.shape[0]:
            raise Exception(
                "row_end max element (%d) cannot be larger than cols count (%d)" % (row_end.max(), cols.shape[0])
            )
        if row_end[-1] != cols.shape[0]:
            raise Exception(
                "row_end last element (%d) should be equal to cols count (%d)" % (row_end[-1], cols.shape[0])
            )

    def build_coo_block_index(self):
        """``[2, nnz]`` int32 (block-row, block-col) of every slot, in slot order (reference ``block_sparse.py:371-403``)."""
        b = self.blocks.view(-1, 2)
        return torch.stack([b[:, 1], b[:, 0]], 0)

    def block_norm(self, p=2):
        """Per-slot norm of ``data`` (reference ``block_sparse.py:155-157``).

        The 2-norm of a 32x32-block matrix on the GPU is the square root of the per-slot sum of squares that
        a kernel of the library emits (one pass over ``data``; the same statistic rides along with every weight
        packing, see :meth:`packed_weights`, and with every weight gradient, ``last_grad_block_sumsq``).
        Other norms, other block shapes and CPU matrices use ``torch.norm``."""
        if p == 2 and self.data.is_cuda and tuple(self.block_shape) == (32, 32) and self.data.numel() > 0:
            return native.block_sumsq(self.data).sqrt_()
        d = self.data.reshape(-1, self.block_shape[0], self.block_shape[1])
        return torch.norm(d, p=p, dim=(1, 2))

    def block_mask_build(self, block_positions):
        if block_positions is None:
            block_positions = self.build_coo_block_index().long()
        mask = torch.zeros(self.blocks_count(), dtype=torch.bool, device=self.data.device)
        mask[block_positions[0], block_positions[1]] = True
        return mask

    def block_replace(self, block_replacements):
        """Move slots to new positions: rows of ``(block-row, block-col, slot)`` (reference ``block_sparse.py:167-219``).

        On a GPU the move and the re-indexing are two kernels of the library writing the existing buffers in
        place (:meth:`move_blocks_`); the checking mode (``check_``) and CPU matrices use torch ops on the host
        side, as the reference does.  Both give bit-identical buffers."""
        if self.data.is_cuda and not self.check_ and self.blocks.numel() > 0:
            repl = block_replacements.to(device=self.data.device, dtype=torch.long)
            _, Y = self.blocks_count()
            self.move_blocks_(repl[:, 2].to(torch.int32).contiguous(), (repl[:, 0] * Y + repl[:, 1]).to(torch.int32).contiguous())
            return
        pos = self.build_coo_block_index().long()
        repl = block_replacements.to(dtype=torch.long, device=pos.device)
        _, Y = self.blocks_count()

        if self.check_:
            # a target position may neither be occupied already nor be named twice
            usage = self.block_mask_build(pos).reshape(-1).long()
            usage.index_add_(0, repl[:, 0] * Y + repl[:, 1], torch.ones_like(repl[:, 0]))
            worst = usage.argmax()
            if usage[worst] > 1:
                raise Exception(f"Block position ({worst // Y},{worst % Y}) was already used")

        pos[:, repl[:, 2]] = repl[:, :2].t()
        new_mask = self.block_mask_build(pos)
        # slot of the i-th set position in row-major order
        block_ptr = torch.argsort(pos[0] * Y + pos[1])
        self.rebuild(new_mask, block_ptr)

    # ------------------------------------------------------- pattern kernels (GPU)
    def _pattern_scratch(self):
        """``(cell_slot, status)``: the slot at every block position (-1 where empty) as the pattern kernels
        keep it, and their device-side flag word; created (and filled) on first use per pattern."""
        cached = self.__dict__.get("_cells")
        X, Y = self.blocks_count()
        if cached is None or cached[0].device != self.data.device or cached[0].numel() != X * Y:
            cell_slot = torch.empty(X * Y, dtype=torch.int32, device=self.data.device)
            status = torch.zeros(1, dtype=torch.int32, device=self.data.device)
            self.__dict__["_cells"] = cached = (cell_slot, status)
            self._rebuild_indices_device()
        return cached

    def _rebuild_indices_device(self):
        cell_slot, status = self.__dict__["_cells"]
        X, Y = self.blocks_count()
        native.rebuild_indices(
            self.blocks, X, Y, cell_slot, self.row_start_ends_a, self.cols_a, self.col_start_ends_b, self.rows_b, status
        )
        self._plan_cache = {}

    def pattern_status(self):
        """Flag word of the pattern kernels since the last call (synchronizes): 0, or 1 = two slots at one
        position, 2 = position or slot out of range, 4 = empty-cell count mismatch."""
        _, status = self._pattern_scratch()
        value = int(status.item())
        status.zero_()
        return value

    def sample_free_positions(self, k, seed):
        """int32 ``[k]`` distinct empty block positions (``row * Y + col``), a pure function of the pattern and
        ``seed`` (``bsmm_sample_free_cells``)."""
        cell_slot, status = self._pattern_scratch()
        X, Y = self.blocks_count()
        return native.sample_free_cells(cell_slot, X * Y - self.blocks.shape[0] // 2, k, seed, status)

    def move_blocks_(self, slots, positions):
        """Slots ``slots[j]`` (int32) move to block positions ``positions[j]`` (int32 ``row * Y + col``); ``blocks``,
        the CSR and the CSC buffers are rewritten in place by the library's kernels, no host round trip."""
        _, status = self._pattern_scratch()
        _, Y = self.blocks_count()
        native.move_blocks(self.blocks, slots, positions, Y, status)
        self._rebuild_indices_device()
        self._pattern_changed()

    def _pattern_changed(self):
        """Derived state keyed on the index buffers is dropped (kernels wrote them behind the version counters)."""
        self._plan_cache = {}
        self.updated_data()

    # ------------------------------------------------------------------ factories
    @classmethod
    def zeros(cls, shape, n_blocks=None, blocks=None, block_shape=(32, 32), device="cuda"):
        """All-zero matrix; pattern explicit (``blocks``) or ``n_blocks`` positions drawn with
        ``numpy.random.choice`` (reference ``block_sparse.py:221-262``)."""
        for i in range(2):
            if shape[i] % block_shape[i] != 0:
                raise Exception(f"Invalid shape: shape[{i}]={shape[i]} %% block_shape[{i}]={block_shape[i]} is not 0.")
        X, Y = cls.blocks_count_(shape, block_shape)
        if n_blocks is None:
            if blocks is not None:
                for b in blocks:
                    for i in range(2):
                        if b[i] * block_shape[i] >= shape[i]:
                            raise Exception(
                                f"Invalid block definition: block[{i}] = {b[i]} : should be < {shape[i] // block_shape[i]}"
                            )
                n_blocks = len(blocks)
            else:
                n_blocks = X * Y
        else:
            assert blocks is None
        if n_blocks > X * Y:
            raise Exception("Too many blocks : %d > %d * %d = %d" % (n_blocks, X, Y, X * Y))
        if blocks is not None:
            flat = numpy.array([b[0] * Y + b[1] for b in blocks], dtype=numpy.int64)
        else:
            flat = numpy.random.choice(X * Y, size=n_blocks, replace=False)
        mask = torch.zeros(X * Y, dtype=torch.bool, device=device)
        mask[torch.as_tensor(flat, dtype=torch.int64, device=device)] = True
        data = torch.zeros((n_blocks * block_shape[0], block_shape[1]), dtype=torch.float, device=device)
        return cls(shape, mask.view(X, Y), data, block_shape)

    @classmethod
    def ones(cls, shape, n_blocks=None, blocks=None, block_shape=(32, 32), device="cuda", positive=False):
        ret = cls.zeros(shape, n_blocks, blocks, block_shape, device)
        with torch.no_grad():
            ret.data.fill_(1.0)
        ret.updated_data()
        return ret

    @classmethod
    def randn(cls, shape, n_blocks=None, blocks=None, block_shape=(32, 32), device="cuda", positive=False):
        ret = cls.zeros(shape, n_blocks, blocks, block_shape, device)
        with torch.no_grad():
            ret.data.normal_()
            if positive:
                ret.data.abs_()
        ret.updated_data()
        return ret

    @classmethod
    def from_dense(cls, dense, block_shape=(32, 32), block_count=None, blocks=None, slow=False, out=None):
        """Build from a dense matrix (reference ``block_sparse.py:299-354``).

        With an explicit pattern, a full pattern or ``out=``, every slot receives its dense
        block.  With ``block_count`` below the full count the pattern is random and ``data``
        is filled with the FIRST ``nnz*bh*bw`` values of ``dense.flatten()`` -- the reference
        keeps only the value distribution in that case, and so does this class.
        """
        bh, bw = block_shape
        full = None
        if out is None:
            if blocks is None:
                full = (dense.shape[0] * dense.shape[1]) // (bh * bw)
                if block_count is None:
                    block_count = full
            else:
                block_count = None
            ret = cls.zeros(dense.shape, n_blocks=block_count, block_shape=block_shape, blocks=blocks, device=dense.device)
        else:
            ret = out

        if out is not None or blocks is not None or block_count == full:
            coo = ret.build_coo_block_index().long()
            X, Y = dense.shape[0] // bh, dense.shape[1] // bw
            if slow:
                for s in range(coo.shape[1]):
                    r, c = int(coo[0, s]), int(coo[1, s])
                    tile = dense[r * bh : (r + 1) * bh, c * bw : (c + 1) * bw]
                    with torch.no_grad():
                        ret.data[s * bh : (s + 1) * bh] = tile.t().reshape(bh, bw)
            else:
                tiles = dense.reshape(X, bh, Y, bw).permute(0, 2, 3, 1)  # [X, Y, bw, bh]: each tile transposed
                picked = tiles[coo[0], coo[1]].reshape(-1, bh, bw)
                with torch.no_grad():
                    ret.data.copy_(picked.reshape(-1, bw))
        else:
            count = ret.data.numel()
            with torch.no_grad():
                ret.data.copy_(dense.flatten()[:count].reshape(ret.data.shape))
        ret.updated_data()
        return ret

    def __repr__(self):
        return "%s(shape=%s, cols=%s, row_start_ends_a=%s, data=%s, block_shape=%s)" % (
            self.__class__.__name__,
            self.shape,
            self.cols_a.shape,
            self.row_start_ends_a.shape,
            self.data.shape,
            self.block_shape,
        )

    def multiply_(self, factor):
        with torch.no_grad():
            self.data.multiply_(factor)
        self.updated_data()

    # ------------------------------------------------------------------ densify
    def to_sparse(self, data_replace=None):
        """Hybrid COO tensor ``[X, Y, bh, bw]`` (reference ``block_sparse.py:405-421``)."""
        coo = self.build_coo_block_index().long()
        data = self.data if data_replace is None else data_replace
        tiles = data.reshape(-1, self.block_shape[1], self.block_shape[0]).transpose(1, 2)
        X, Y = self.blocks_count()
        return torch.sparse_coo_tensor(coo, tiles, (X, Y) + tuple(self.block_shape))

    def to_dense(self, data_replace=None):
        """Dense ``[rows, cols]`` copy; ``data_replace`` densifies another tensor laid out like ``data``
        (reference ``block_sparse.py:423-429``)."""
        coo = self.build_coo_block_index().long()
        data = self.data if data_replace is None else data_replace
        bh, bw = self.block_shape
        X, Y = self.blocks_count()
        grid = torch.zeros((X, Y, bh, bw), dtype=data.dtype, device=data.device)
        grid[coo[0], coo[1]] = data.reshape(-1, bw, bh).transpose(1, 2)
        return grid.permute(0, 2, 1, 3).reshape(self.shape[0], self.shape[1])

    # ------------------------------------------------------------- interchange
    def to_bsr(self, data_replace=None):
        """The matrix as a ``torch.sparse_bsr_tensor``: blocks in CSR order, each ``[bh, bw]`` tile un-transposed.
        The reference's only sparse export is the hybrid COO tensor of :meth:`to_sparse`
        (reference ``block_sparse.py:405-421``); BSR is what ``torch.sparse`` kernels and other libraries read."""
        data = self.data.detach() if data_replace is None else data_replace
        bh, bw = self.block_shape
        slots = self.cols_a[:, 1].long()
        values = data.reshape(-1, bw, bh)[slots].transpose(1, 2).contiguous()
        return torch.sparse_bsr_tensor(
            self.row_start_ends_a.long(), self.cols_a[:, 0].long(), values, size=tuple(self.shape)
        )

    @classmethod
    def from_bsr(cls, bsr):
        """Build from a ``torch.sparse_bsr_tensor`` (2-D, block size = the block shape).  Slot ``i`` is the
        tensor's ``i``-th stored block, so ``to_bsr()`` of the result lists the same blocks (sorted by column
        inside each row, as the index buffers of this class always are)."""
        crow, col, values = bsr.crow_indices().long(), bsr.col_indices().long(), bsr.values()
        if values.dim() != 3 or crow.dim() != 1:
            raise Exception("from_bsr takes a 2-D BSR tensor without batch dimensions")
        bh, bw = int(values.shape[1]), int(values.shape[2])
        shape = tuple(bsr.shape)
        X, Y = shape[0] // bh, shape[1] // bw
        rows = torch.repeat_interleave(torch.arange(X, device=crow.device), crow[1:] - crow[:-1])
        mask = torch.zeros((X, Y), dtype=torch.bool, device=values.device)
        mask[rows, col] = True
        if int(mask.sum()) != col.shape[0]:
            raise Exception("the BSR tensor stores a block position twice")
        data = values.to(torch.float32).transpose(1, 2).reshape(-1, bw).contiguous()
        ret = cls(shape, mask, data, (bh, bw))
        ret.rebuild(mask, torch.argsort(rows * Y + col))  # i-th position in row-major order -> its slot
        return ret

    def check_with_dense(self, dense_version):
        coo = self.build_coo_block_index().long()
        bh, bw = self.block_shape
        for s in range(coo.shape[1]):
            r, c = int(coo[0, s]), int(coo[1, s])
            mine = self.data[s * bh : (s + 1) * bh, :].t()
            theirs = dense_version[r * bh : (r + 1) * bh, c * bw : (c + 1) * bw]
            if not (mine == theirs).all():
                raise Exception("non matching data")

    # ---------------------------------------------------------------- matmuls
    def tensor_prepare(self, t, message, transpose):
        """``(tensor, flag)``: which of ``t`` / ``t.t()`` is contiguous, copying only if neither
        (reference ``block_sparse.py:480-494``)."""
        ret = None
        if t.is_contiguous():
            ret = [t, True]
        if t.t().is_contiguous():
            ret = [t, False]
        if ret is not None:
            if transpose:
                ret[1] = not ret[1]
            return ret
        return t.contiguous(), False

    @staticmethod
    def _orient(t):
        """``(tensor, row_major)``: ``t`` itself if it or its transpose is contiguous, else a contiguous copy."""
        if t.is_contiguous():
            return t, True
        if t.t().is_contiguous():
            return t, False
        return t.contiguous(), True

    def flatten_first_dims(self, dense_a):
        if dense_a.dim() < 2:
            raise Exception(
                f"Invalid dimensions for dense_a {dense_a.shape} : dense_a should have at least 2 dimensions."
            )
        flat = dense_a.reshape(-1, dense_a.shape[-1]) if dense_a.dim() > 2 else dense_a
        return flat, dense_a.shape[:-1]

    def unflatten_first_dims(self, result, info):
        if len(info) > 1:
            result = result.reshape(*info, result.shape[-1])
        return result

    def _require_cuda(self):
        if not self.data.is_cuda:
            raise Exception(
                "BlockSparseMatrix matmuls run only on CUDA (sm_100a kernels, no CPU path); data is on %s"
                % self.data.device
            )

    def _plan(self, transpose):
        """Cached per-pattern launch plan for fwd (``transpose=True``, CSR) or dgrad (CSC)."""
        ptr, idx = (self.row_start_ends_a, self.cols_a) if transpose else (self.col_start_ends_b, self.rows_b)
        key = (bool(transpose), ptr.data_ptr(), ptr._version, idx.data_ptr(), idx._version)
        plan = self._plan_cache.get(key)
        if plan is None:
            plan = native.DsdPlan(ptr, idx)
            self._plan_cache = {k: v for k, v in self._plan_cache.items() if k[0] != bool(transpose)}
            self._plan_cache[key] = plan
        return plan

    def _sddmm_plan(self):
        """Cached per-pattern item table of the tensor-core wgrad kernel (built from the CSR)."""
        ptr, idx = self.row_start_ends_a, self.cols_a
        key = ("sddmm", ptr.data_ptr(), ptr._version, idx.data_ptr(), idx._version)
        plan = self._plan_cache.get(key)
        if plan is None:
            plan = native.SddmmPlan(ptr, idx)
            self._plan_cache = {k: v for k, v in self._plan_cache.items() if k[0] != "sddmm"}
            self._plan_cache[key] = plan
        return plan

    def packed_weights(self, precision=None, fresh=True):
        """Kernel-ready images of ``data`` (tf32 hi/lo or bf16, both orientations) and the fused per-slot sum
        of squares.

        ``fresh=True`` (the default) packs now: one small kernel (about 1 % of a layer step) and the only way
        to be right after writes that autograd's version counter does not see (``p.data.add_()``, fused
        optimizers, EMA copies).  ``fresh=False`` reuses the last images while ``data``'s address and version
        counter are unchanged -- for frozen weights; call :meth:`invalidate_packed` after writing ``data``
        behind autograd's back."""
        precision = native.resolve_precision(precision)
        key = (self.data.data_ptr(), self.data._version, precision)
        if fresh or self._pack_cache.get("key") != key:
            self._pack_cache = {"key": key, "pack": native.pack_weights(self.data, precision)}
        return self._pack_cache["pack"]

    def invalidate_packed(self):
        """Forget the cached weight images (see :meth:`packed_weights`)."""
        self._pack_cache = {}

    def reverse_matmul_(self, dense_a, transpose=True, bias=None, precision=None, packed=None):
        """``a @ W.T`` if ``transpose`` else ``a @ W`` (reference ``block_sparse.py:496-578``); ``a`` is 2-D.

        ``bias`` (fwd only) is added in the kernel epilogue.  ``packed`` hands in weight images made
        earlier (the autograd function packs once in forward and reuses the images in backward: the gradient
        is then taken with the weights the forward saw); by default the weights are packed now.
        Returns a contiguous ``[M, n]`` tensor (the reference returns the transposed view of an
        ``[n, M]`` buffer; values agree).
        """
        if dense_a.dim() > 2:
            dense_a = dense_a.reshape(-1, dense_a.shape[-1])
        shape_b = [self.shape[0], self.shape[1]]
        if transpose:
            shape_b.reverse()
        if dense_a.shape[1] != shape_b[0]:
            raise Exception(
                "Invalid matrices sizes (%d, %d) x (%d, %d)"
                % (dense_a.shape[0], dense_a.shape[1], shape_b[0], shape_b[1])
            )
        assert self.data.is_contiguous()
        if not dense_a.is_contiguous():
            dense_a = dense_a.contiguous()
        return native.dsd_matmul(
            dense_a,
            self._plan(transpose),
            packed if packed is not None else self.packed_weights(precision),
            n_out=shape_b[1],
            transpose=transpose,
            bias=bias,
        )

    def reverse_matmul_fused(self, dense_a, bias=None, residual=None, activation=None, precision=None, packed=None,
                             keep_pre=False):
        """``act(a @ W.T + bias + residual)`` with everything after the product done in the forward kernel's
        epilogue (tensor-core precisions).  Returns ``(out, pre)``: ``pre`` is the sum before the activation when
        ``keep_pre`` and an activation are given, else ``None``.  The reference has no counterpart: its layer adds
        the bias in a separate pass (``block_sparse_linear.py:229-233``)."""
        self._require_cuda()
        flat, lead = self.flatten_first_dims(dense_a)
        if flat.shape[1] != self.shape[1]:
            raise Exception(
                "Invalid matrices sizes (%d, %d) x (%d, %d)" % (flat.shape[0], flat.shape[1], self.shape[1], self.shape[0])
            )
        if not flat.is_contiguous():
            flat = flat.contiguous()
        fine = self._fine_matrix() if getattr(self, "_is_coarse", lambda: False)() else self
        if packed is None:
            packed = self.packed_weights(precision)
        pre = None
        if keep_pre and activation is not None:
            pre = torch.empty((flat.shape[0], self.shape[0]), dtype=torch.float32, device=flat.device)
        out = native.dsd_matmul(
            flat, fine._plan(True), packed, n_out=self.shape[0], transpose=True, bias=bias, residual=residual,
            activation=activation, pre_activation=pre,
        )
        out = self.unflatten_first_dims(out, lead)
        if pre is not None:
            pre = self.unflatten_first_dims(pre, lead)
        return out, pre

    def reverse_matmul(self, dense_a, transpose, bias=None, precision=None, packed=None):
        """Any-rank wrapper of :meth:`reverse_matmul_` (reference ``block_sparse.py:597-604``)."""
        self._require_cuda()
        flat, lead = self.flatten_first_dims(dense_a)
        ret = self.reverse_matmul_(flat, transpose=transpose, bias=bias, precision=precision, packed=packed)
        return self.unflatten_first_dims(ret, lead)

    def matmul_with_output_sparse_support_(self, dense_a, dense_b, overwrite_data=False, precision=None):
        """``(a.T @ b)`` kept only at the non-zero blocks, in ``data``'s layout
        (reference ``block_sparse.py:606-655``).  ``a``: ``[tokens, rows]``, ``b``: ``[tokens, cols]``."""
        assert dense_a.shape[0] == dense_b.shape[0]
        assert self.shape[0] == dense_a.shape[1]
        assert self.shape[1] == dense_b.shape[1]
        assert (dense_a.shape[1] % self.block_shape[1]) == 0
        assert (dense_b.shape[1] % self.block_shape[0]) == 0
        out = self.data if overwrite_data else torch.empty_like(self.data)
        a, a_rowmajor = self._orient(dense_a)
        b, b_rowmajor = self._orient(dense_b)
        # sum of squares of every gradient block, written by the kernel's epilogue (its token-range reduction)
        sumsq = torch.empty(self.data.shape[0] // 32, dtype=torch.float32, device=self.data.device)
        with torch.no_grad():
            native.sddmm(
                a, a_rowmajor, b, b_rowmajor, self.blocks, out.detach(), precision=precision,
                block_sumsq=sumsq, plan=self._sddmm_plan(),
            )
        self.last_grad_block_sumsq = sumsq
        if overwrite_data:
            self._pack_cache = {}  # the kernel wrote `data` behind autograd's version counter
        return out

    def matmul_with_output_sparse_support(self, dense_a, dense_b, overwrite_data=False, precision=None):
        """Any-rank wrapper (reference ``block_sparse.py:657-665``)."""
        self._require_cuda()
        a, lead_a = self.flatten_first_dims(dense_a)
        b, lead_b = self.flatten_first_dims(dense_b)
        assert lead_a == lead_b
        return self.matmul_with_output_sparse_support_(a, b, overwrite_data, precision=precision)


class BlockSparseMatrix(BlockSparseMatrixBase):
    """Matrix served by the CUDA kernels (reference ``block_sparse.py:668-679``).

    The kernels work on 32x32 blocks.  A matrix with larger square blocks (64x64, 128x128, any multiple of 32;
    the reference sends those to its dense-masked emulator, ``block_sparse_linear.py:202-205``) keeps the
    reference's ``data`` and index buffers in its own block units and carries a derived 32x32 matrix of the
    same non-zeros -- every block becomes ``(b/32)^2`` adjacent fine blocks -- which the kernels run on.
    ``data`` is re-tiled into the fine matrix before a product and the fine weight gradient is re-tiled back:
    two copies of weight size per step."""

    def __init__(self, shape, block_mask, data, block_shape=(32, 32)):
        if len(shape) != 2 or shape[0] % 32 != 0 or shape[1] % 32 != 0:
            raise Exception("shape should be a tuple of 2 multiples of 32")
        if len(block_shape) != 2 or block_shape[0] % 32 != 0 or block_shape[1] % 32 != 0:
            raise Exception("block_shape should be a tuple of 2 multiples of 32")
        if tuple(block_shape) != (32, 32) and block_shape[0] != block_shape[1]:
            raise Exception("blocks larger than 32x32 must be square on the CUDA path, got %s" % (block_shape,))
        object.__setattr__(self, "_fine", None)
        super().__init__(shape, block_mask, data, block_shape)

    # the fine matrix is derived state: it never travels with a pickle, a state_dict or .to()
    def __getstate__(self):
        state = super().__getstate__()
        state["_fine"] = None
        return state

    def _is_coarse(self):
        return tuple(self.block_shape) != (32, 32)

    def rebuild(self, block_mask, block_ptr=None, callback=True):
        super().rebuild(block_mask, block_ptr, callback)
        object.__setattr__(self, "_fine", None)

    def _pattern_changed(self):
        object.__setattr__(self, "_fine", None)
        super()._pattern_changed()

    def _fine_matrix(self):
        """The 32x32 matrix of the same non-zeros.  Fine slot ``(s * nb + i) * nb + j`` is the sub-block at
        row part ``i``, column part ``j`` of slot ``s``; rebuilt when the index buffers changed."""
        key = (self.blocks.data_ptr(), self.blocks._version, self.data.device)
        if self._fine is not None and self._fine[0] == key:
            return self._fine[1]
        nb = self.block_shape[0] // 32
        pairs = self.blocks.view(-1, 2).long()  # (block-col, block-row) per slot
        col, row = pairs[:, 0], pairs[:, 1]
        part = torch.arange(nb, device=col.device)
        frow = (row[:, None, None] * nb + part[None, :, None]).expand(-1, nb, nb).reshape(-1)
        fcol = (col[:, None, None] * nb + part[None, None, :]).expand(-1, nb, nb).reshape(-1)
        X, Y = self.shape[0] // 32, self.shape[1] // 32
        mask = torch.zeros((X, Y), dtype=torch.bool, device=col.device)
        mask[frow, fcol] = True
        data = torch.zeros((frow.shape[0] * 32, 32), dtype=torch.float32, device=self.data.device)
        fine = BlockSparseMatrix(tuple(self.shape), mask, data, (32, 32))
        fine.rebuild(mask, torch.argsort(frow * Y + fcol))
        fine.requires_grad_(False)
        object.__setattr__(self, "_fine", (key, fine))
        return fine

    def _to_fine(self, data):
        """``data`` layout ``[nnz * b, b]`` -> the fine matrix's ``[nnz * nb * nb * 32, 32]``."""
        nb = self.block_shape[0] // 32
        # data[s, j, c', i, r'] -> fine[s, i, j, c', r']
        return data.reshape(-1, nb, 32, nb, 32).permute(0, 3, 1, 2, 4).reshape(-1, 32)

    def _from_fine(self, fine_data):
        nb = self.block_shape[0] // 32
        return fine_data.reshape(-1, nb, nb, 32, 32).permute(0, 2, 3, 1, 4).reshape(-1, self.block_shape[1])

    def _fine_synced(self):
        fine = self._fine_matrix()
        with torch.no_grad():
            fine.data.copy_(self._to_fine(self.data.detach()))
        return fine

    def packed_weights(self, precision=None, fresh=True):
        if self._is_coarse():
            return self._fine_synced().packed_weights(precision, fresh=True)
        return super().packed_weights(precision, fresh)

    def block_norm(self, p=2):
        if self._is_coarse() and p == 2 and self.data.is_cuda and self.data.numel() > 0:
            nb2 = (self.block_shape[0] // 32) ** 2
            return native.block_sumsq(self._to_fine(self.data.detach()).contiguous()).view(-1, nb2).sum(1).sqrt_()
        return super().block_norm(p)

    def reverse_matmul_(self, dense_a, transpose=True, bias=None, precision=None, packed=None):
        if self._is_coarse():
            fine = self._fine_matrix()
            if packed is None:
                packed = self.packed_weights(precision)
            return fine.reverse_matmul_(dense_a, transpose=transpose, bias=bias, precision=precision, packed=packed)
        return super().reverse_matmul_(dense_a, transpose, bias, precision, packed)

    def matmul_with_output_sparse_support_(self, dense_a, dense_b, overwrite_data=False, precision=None):
        if self._is_coarse():
            fine = self._fine_matrix()
            grad = self._from_fine(fine.matmul_with_output_sparse_support_(dense_a, dense_b, False, precision))
            nb2 = (self.block_shape[0] // 32) ** 2
            self.last_grad_block_sumsq = fine.last_grad_block_sumsq.view(-1, nb2).sum(1)
            if overwrite_data:
                with torch.no_grad():
                    self.data.copy_(grad)
                return self.data
            return grad.contiguous()
        return super().matmul_with_output_sparse_support_(dense_a, dense_b, overwrite_data, precision)


class BlockSparseMatrixEmulator(BlockSparseMatrixBase):
    """Dense-masked stand-in for arbitrary block shapes, pure torch (reference ``block_sparse.py:682-714``)."""

    def __init__(self, shape, block_mask, data, block_shape):
        super().__init__(shape, block_mask, data, block_shape)
        self.register_parameter("_dense", None)
        self.updated_data()

    def get_differentiable_data(self):
        return self._dense

    def to_dense(self, data_replace=None):
        if data_replace is None:
            return self._dense
        return data_replace * self._mask

    def _update_data_from_dense(self):
        self.from_dense(self._dense, out=self)

    def updated_data(self):
        with torch.no_grad():
            self._dense = torch.nn.Parameter(super().to_dense())
            self._mask = super().to_dense(data_replace=torch.ones_like(self.data)) == 1

    def reverse_matmul(self, dense_a, transpose=True, bias=None, precision=None, packed=None):
        m = self._dense.t() if transpose else self._dense
        mask = self._mask.t() if transpose else self._mask
        out = dense_a.matmul(m * mask)
        return out if bias is None else out + bias

    def matmul_with_output_sparse_support(self, dense_a, dense_b, overwrite_data=False, precision=None):
        a = dense_a.reshape(-1, dense_a.shape[-1])
        b = dense_b.reshape(-1, dense_b.shape[-1])
        return a.t().mm(b) * self._mask
