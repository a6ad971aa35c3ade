"""Drop-in for the reference's pybind11 extension ``block_sparse_native``
(``pytorch_block_sparse/native/block_sparse_native.cpp:6-34``): the same two functions with the same
positional arguments, forwarding ``data_ptr()``s to ``libbsmm_b200.so``.

With ``install()`` the unmodified reference ``block_sparse.py`` (which does ``import block_sparse_native``
inside its matmul methods, ``block_sparse.py:498,608``) runs on the kernels of this library -- the
tensor-core kernels in the library's default precision, the exact-fp32 CUDA-core kernels with
``native.set_default_precision("fp32")``.

The reference hands over only raw ``data`` and index arrays.  What the tensor-core kernels need on top is
derived here:

* weight images: packed from ``data_b`` on every call (one small kernel).  ``data_b`` holds, per slot, the
  ``[k-in-block, n-in-block]`` tile for the forward product (``data`` itself) as well as for dgrad (the
  transposed copy the reference makes per call, ``block_sparse.py:538-544``), so both calls are the
  forward-orientation product of the matrix they describe;
* launch plans: built from ``ptr_b / indices_b`` and kept while those tensors live unchanged (address and
  version counter), as are the CSR arrays and item table the weight-gradient kernel wants, which are
  rebuilt from the slot-order ``sparse_blocks_c`` list.

Unlike the reference, a failing call raises instead of returning an ignored error code.
"""
import ctypes
import sys

import torch

from . import native

_MAX_CACHED = 64
_dsd_plans = {}
_sddmm_plans = {}


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _s(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _key(*tensors):
    return tuple((t.data_ptr(), t._version, tuple(t.shape), t.device.index) for t in tensors)


def _remember(cache, key, value):
    if len(cache) >= _MAX_CACHED:
        cache.pop(next(iter(cache)))
    cache[key] = value
    return value


def clear_caches():
    """Forget every cached plan (they are keyed on tensor address and version; call this after writing an
    index buffer through ``.data``)."""
    _dsd_plans.clear()
    _sddmm_plans.clear()


def _dsd_plan(ptr_b, indices_b):
    key = _key(ptr_b, indices_b)
    plan = _dsd_plans.get(key)
    if plan is None:
        plan = _remember(_dsd_plans, key, native.DsdPlan(ptr_b, indices_b))  # holds the tensors: addresses stay unique
    return plan


def _sddmm_plan(blocks, n_block_rows):
    """CSR (offsets, (block-col, slot) entries) and item table from the slot-order (block-col, block-row) list."""
    key = _key(blocks) + (n_block_rows,)
    plan = _sddmm_plans.get(key)
    if plan is None:
        pairs = blocks.view(-1, 2).long()
        cols, rows = pairs[:, 0], pairs[:, 1]
        order = torch.argsort(rows * (int(cols.max()) + 1 if cols.numel() else 1) + cols)
        idx = torch.stack([cols[order], order], 1).to(torch.int32).contiguous()
        ptr = torch.zeros(n_block_rows + 1, dtype=torch.long, device=blocks.device)
        if rows.numel():
            ptr[1:] = torch.cumsum(torch.bincount(rows, minlength=n_block_rows), 0)
        plan = native.SddmmPlan(ptr.to(torch.int32), idx)
        plan.blocks = blocks  # keeps the key's address from being reused while the entry lives
        _remember(_sddmm_plans, key, plan)
    return plan


def blocksparse_matmul_cutlass(
    dense_a, pytorch_contiguous_a, ptr_b, indices_b, data_b, m, n, k, block_size_rows_b, block_size_cols_b, dense_out
):
    """``dense_out[n, m]`` (column-major result) ``= dense_a[m, k] x B``, B given per output block-row by
    ``ptr_b / indices_b`` with ``data_b`` holding, per slot, the ``[k-in-block, n-in-block]`` tile -- the
    reference passes ``data`` for the forward product and a transposed copy of it for dgrad
    (``block_sparse.py:538-544``).  Every element of ``dense_out`` is written."""
    assert pytorch_contiguous_a
    prec = native.resolve_precision(None)
    if prec == native.PREC_FP32_SIMT or indices_b.shape[0] == 0:
        lib = native.load()
        with torch.cuda.device(dense_a.device):
            status = lib.bsmm_dsd(
                _p(dense_a), m, k, _p(ptr_b), _p(indices_b), indices_b.shape[0], _p(data_b), None, None, n,
                _p(dense_out), None, native.PREC_FP32_SIMT | native.DSD_OUT_COLMAJOR, _s(dense_a),
            )
        native.check(status, "blocksparse_matmul_cutlass")
        return status
    packed = native.pack_weights(data_b, prec)
    native.dsd_matmul(dense_a.view(m, k), _dsd_plan(ptr_b, indices_b), packed, n, True, out=dense_out, out_colmajor=True)
    return 0


def blocksparse_matmul_back_cutlass(
    dense_a, pytorch_contiguous_a, dense_b, pytorch_contiguous_b, m, n, k, block_size_rows_b, block_size_cols_b,
    sparse_c, sparse_blocks_c, sparse_blocks_length_c,
):
    """``sparse_c`` = the listed blocks of ``a x b`` with ``a`` seen as ``[m = rows, k = tokens]`` and ``b`` as
    ``[k = tokens, n = cols]``; each flag says whether that view (rather than its transpose) is the contiguous
    one (``native/block_sparse_cutlass_kernel_back.cu:113-117``).  The tensors themselves arrive as the
    reference holds them, ``[tokens, rows]`` and ``[tokens, cols]``."""
    a_token_major = not pytorch_contiguous_a  # [rows, tokens] contiguous means feature-major dY
    b_token_major = bool(pytorch_contiguous_b)
    prec = native.resolve_precision(None)
    plan = None
    if prec != native.PREC_FP32_SIMT and sparse_blocks_length_c > 0:
        plan = _sddmm_plan(sparse_blocks_c, m // 32)
    a2 = dense_a if dense_a.dim() == 2 and dense_a.shape[0] == k else dense_a.reshape(k, m)
    b2 = dense_b if dense_b.dim() == 2 and dense_b.shape[0] == k else dense_b.reshape(k, n)
    native.sddmm(a2, a_token_major, b2, b_token_major, sparse_blocks_c, sparse_c, precision=prec, plan=plan)
    return 0


def install():
    """Register this module as ``block_sparse_native`` so that ``import block_sparse_native`` finds it."""
    sys.modules["block_sparse_native"] = sys.modules[__name__]
    return sys.modules[__name__]
