"""The ``block_sparse_native`` stand-in called exactly the way the reference's ``block_sparse.py`` calls the
pybind11 extension (argument order and conventions of block_sparse.py:565-577 and :640-653)."""
import numpy as np
import pytest
import torch

from oracle import block_sparse_oracle as orc
from pytorch_block_sparse_b200 import block_sparse_native as shim

from .gpu_util import check, host, make_matrix, randn

pytestmark = pytest.mark.gpu


def test_import_under_the_reference_name():
    shim.install()
    import block_sparse_native

    assert block_sparse_native.blocksparse_matmul_cutlass is shim.blocksparse_matmul_cutlass


@pytest.mark.parametrize("transpose", [True, False])
def test_reverse_matmul_call_convention(transpose):
    m = make_matrix((128, 96), n_blocks=7, seed=71)
    shape, blocks, data = host(m)
    a = randn((77, 96 if transpose else 128), seed=72)
    dense_a = a.cuda()
    shape_b = [96, 128] if transpose else [128, 96]  # the reference's shape_b after its optional reverse()
    out = torch.zeros((shape_b[1], dense_a.shape[0]), device="cuda")
    if transpose:
        ptr_b, indices_b, data_b = m.row_start_ends_a, m.cols_a, m.data.detach()
    else:
        ptr_b, indices_b = m.col_start_ends_b, m.rows_b
        data_b = m.data.detach().view(-1, 32, 32).transpose(1, 2).reshape(-1, 32).contiguous()
    shim.blocksparse_matmul_cutlass(dense_a, True, ptr_b, indices_b, data_b, dense_a.shape[0], shape_b[1], shape_b[0],
                                    32, 32, out)
    torch.cuda.synchronize()
    want = orc.forward(a.numpy(), shape, blocks, data) if transpose else orc.dgrad(a.numpy(), shape, blocks, data)
    check(out.t(), want, "fp32")


@pytest.mark.parametrize("a_feature_major,b_feature_major", [(False, False), (True, False), (False, True), (True, True)])
def test_matmul_with_output_sparse_support_call_convention(a_feature_major, b_feature_major):
    m = make_matrix((128, 96), n_blocks=6, seed=73)
    dy, x = randn((50, 128), seed=74), randn((50, 96), seed=75)
    # the reference passes the tensors as they are and flags which view is contiguous
    a = dy.t().contiguous().cuda().t() if a_feature_major else dy.cuda()
    b = x.t().contiguous().cuda().t() if b_feature_major else x.cuda()
    # tensor_prepare(a, transpose=True): contiguous a -> flag False; a.t() contiguous -> flag True
    flag_a = a_feature_major
    # tensor_prepare(b, transpose=False): contiguous b -> flag True
    flag_b = not b_feature_major
    out = torch.zeros_like(m.data)
    shim.blocksparse_matmul_back_cutlass(a, flag_a, b, flag_b, 128, 96, 50, 32, 32, out.detach(), m.blocks, 6)
    torch.cuda.synchronize()
    check(out, orc.wgrad(dy.numpy(), x.numpy(), (128, 96), m.blocks.cpu().numpy()), "fp32")
