"""Drop-in for the reference's pybind11 extension ``block_sparse_native``
(``pytorch_block_sparse/native/block_sparse_native.cpp:6-34``): the same two functions with the same
positional arguments, forwarding ``data_ptr()``s to ``libbsmm_b200.so``.

With ``install()`` the unmodified reference ``block_sparse.py`` (which does ``import block_sparse_native``
inside its matmul methods, ``block_sparse.py:498,608``) runs on the kernels of this library.  The reference
hands over only the raw ``data`` and index arrays, so the exact-fp32 CUDA-core kernels serve these calls;
the tensor-core kernels need the packed images and plans that ``pytorch_block_sparse_b200.BlockSparseMatrix``
caches.  Unlike the reference, a failing call raises instead of returning an ignored error code.
"""
import ctypes
import sys

import torch

from . import native


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _s(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def blocksparse_matmul_cutlass(
    dense_a, pytorch_contiguous_a, ptr_b, indices_b, data_b, m, n, k, block_size_rows_b, block_size_cols_b, dense_out
):
    """``dense_out[n, m]`` (column-major result) ``= dense_a[m, k] x B``, B given per output block-row by
    ``ptr_b / indices_b`` with ``data_b`` holding, per slot, the ``[k-in-block, n-in-block]`` tile -- the
    reference passes ``data`` for the forward product and a transposed copy of it for dgrad
    (``block_sparse.py:538-544``).  Every element of ``dense_out`` is written."""
    assert pytorch_contiguous_a
    lib = native.load()
    with torch.cuda.device(dense_a.device):
        status = lib.bsmm_dsd(
            _p(dense_a), m, k, _p(ptr_b), _p(indices_b), indices_b.shape[0], _p(data_b), None, None, n, _p(dense_out),
            None, native.PREC_FP32_SIMT | native.DSD_OUT_COLMAJOR, _s(dense_a),
        )
    native.check(status, "blocksparse_matmul_cutlass")
    return status


def blocksparse_matmul_back_cutlass(
    dense_a, pytorch_contiguous_a, dense_b, pytorch_contiguous_b, m, n, k, block_size_rows_b, block_size_cols_b,
    sparse_c, sparse_blocks_c, sparse_blocks_length_c,
):
    """``sparse_c`` = the listed blocks of ``a x b`` with ``a`` seen as ``[m = rows, k = tokens]`` and ``b`` as
    ``[k = tokens, n = cols]``; each flag says whether that view (rather than its transpose) is the contiguous
    one (``native/block_sparse_cutlass_kernel_back.cu:113-117``)."""
    lib = native.load()
    flags = native.PREC_FP32_SIMT
    if pytorch_contiguous_a:  # [rows, tokens] contiguous: feature-major dY
        flags |= native.SDDMM_A_COLMAJOR
    if not pytorch_contiguous_b:  # [cols, tokens] contiguous: feature-major X
        flags |= native.SDDMM_B_COLMAJOR
    with torch.cuda.device(dense_a.device):
        status = lib.bsmm_sddmm(
            _p(dense_a), _p(dense_b), m, n, k, _p(sparse_c), _p(sparse_blocks_c), sparse_blocks_length_c, None, None,
            None, None, flags, _s(dense_a),
        )
    native.check(status, "blocksparse_matmul_back_cutlass")
    return status


def install():
    """Register this module as ``block_sparse_native`` so that ``import block_sparse_native`` finds it."""
    sys.modules["block_sparse_native"] = sys.modules[__name__]
    return sys.modules[__name__]
