"""Loader for the REFERENCE's own CUDA extension built by oracle/build_ref.py into oracle/_ref/ --
TEST INFRASTRUCTURE (second, on-device oracle; "reference kernels on B200" comparator of bench.py).

The wrappers marshal arguments exactly as the reference's block_sparse.py does
(reverse_matmul_: block_sparse.py:496-578, matmul_with_output_sparse_support_: :606-655), using the index
buffers of a BlockSparseMatrix of this repository, which are bit-identical to the reference's.
"""
import importlib.util
import os
import sys

import torch

_SO = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "block_sparse_native.so")
_mod = None


def available():
    return os.path.exists(_SO)


def load():
    global _mod
    if _mod is None:
        saved = sys.modules.get("block_sparse_native")
        spec = importlib.util.spec_from_file_location("block_sparse_native", _SO)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        if saved is not None:
            sys.modules["block_sparse_native"] = saved
        else:
            sys.modules.pop("block_sparse_native", None)
        _mod = mod
    return _mod


def reverse_matmul(matrix, dense_a, transpose):
    """a @ W.T (transpose) or a @ W with the reference kernel K1; returns [m, n] (view of the [n, m] buffer).
    The reference launches on the legacy default stream."""
    mod = load()
    n_out = matrix.shape[0] if transpose else matrix.shape[1]
    k_in = matrix.shape[1] if transpose else matrix.shape[0]
    out = torch.zeros((n_out, dense_a.shape[0]), device=dense_a.device)
    if transpose:
        ptr_b, indices_b, data_b = matrix.row_start_ends_a, matrix.cols_a, matrix.data.detach()
    else:
        ptr_b, indices_b = matrix.col_start_ends_b, matrix.rows_b
        data_b = matrix.data.detach().view(-1, 32, 32).transpose(1, 2).reshape(-1, 32).contiguous()
    mod.blocksparse_matmul_cutlass(dense_a, True, ptr_b, indices_b, data_b, dense_a.shape[0], n_out, k_in, 32, 32, out)
    return out.t()


def sddmm(matrix, dy, x):
    """(dy.T @ x) at the stored blocks with the reference kernel K2 (contiguous token-major operands)."""
    mod = load()
    data = torch.zeros_like(matrix.data)
    mod.blocksparse_matmul_back_cutlass(dy, False, x, True, dy.shape[1], x.shape[1], dy.shape[0], 32, 32, data,
                                        matrix.blocks, matrix.blocks.shape[0] // 2)
    return data
