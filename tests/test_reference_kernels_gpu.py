"""Second oracle, on the device: the reference's own CUDA kernels (built from its sources by
oracle/build_ref.py into oracle/_ref/) against this library on identical inputs.  Skipped when the
reference extension was not built."""
import pytest
import torch

from oracle import ref_cuda

from .gpu_util import make_matrix, randn

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref not built")]


def rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


@pytest.mark.parametrize("precision", ["fp32", "tf32x3"])
def test_three_contractions_match_the_reference_cuda_kernels(precision):
    m = make_matrix((512, 384), n_blocks=70, seed=81)
    # 320 tokens: the reference's wgrad kernel drops the tail of a token count that is not a multiple of 32
    # (measured: relative error sqrt(12/300) at 300 tokens), so only full steps are compared
    x = randn((320, 384), seed=82).cuda()
    dy = randn((320, 512), seed=83).cuda()
    torch.cuda.synchronize()
    ref_y = ref_cuda.reverse_matmul(m, x, True)
    ref_dx = ref_cuda.reverse_matmul(m, dy, False)
    ref_dw = ref_cuda.sddmm(m, dy, x)
    torch.cuda.synchronize()  # the reference launches on the legacy default stream
    y = m.reverse_matmul(x, transpose=True, precision=precision)
    dx = m.reverse_matmul(dy, transpose=False, precision=precision)
    dw = m.matmul_with_output_sparse_support(dy, x, precision=precision)
    torch.cuda.synchronize()
    # both sides are fp32-class computations with different summation orders
    assert rel(y, ref_y) < 5e-6 and rel(dx, ref_dx) < 5e-6 and rel(dw, ref_dw) < 5e-6
