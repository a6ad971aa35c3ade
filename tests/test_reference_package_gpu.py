"""The UNMODIFIED reference package (huggingface/pytorch_block_sparse 0.1.2, pip-installed into the git-ignored
baseline/_ref) running on this library: its ``block_sparse.py`` does ``import block_sparse_native`` inside the
two matmul methods (block_sparse.py:498,608), and ``block_sparse_native.install()`` of this repository answers
that import.  Skipped where the reference was not installed."""
import os
import sys
import time

import numpy as np
import pytest
import torch

from oracle import block_sparse_oracle as orc
from pytorch_block_sparse_b200 import block_sparse_native as shim
from pytorch_block_sparse_b200 import native

from .gpu_util import assert_device_healthy

REF_ROOT = os.environ.get(
    "BSMM_REFERENCE_SITE", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
)
pytestmark = [
    pytest.mark.gpu,
    pytest.mark.skipif(not os.path.isdir(os.path.join(REF_ROOT, "pytorch_block_sparse")), reason="reference not installed"),
]


@pytest.fixture()
def ref():
    sys.path.insert(0, REF_ROOT)
    try:
        import pytorch_block_sparse as ref_pkg
    finally:
        sys.path.remove(REF_ROOT)
    assert "b200" not in ref_pkg.__file__
    shim.install()
    yield ref_pkg
    native.set_default_precision("tf32x3")


def _step(lin, x, dy):
    lin.weight.data.grad = None
    xg = x.detach().requires_grad_(True)
    y = lin(xg)
    y.backward(dy)
    return y.detach(), xg.grad, lin.weight.data.grad


def test_reference_linear_runs_on_the_tensor_core_kernels(ref):
    """fwd + dgrad + wgrad of the reference's BlockSparseLinear (its autograd function, its matrix class, its
    argument marshalling) against the oracle, in the default precision and in 'fp32', and the default one is
    the faster: the plans and images the tensor-core kernels need are derived inside the stand-in module."""
    np.random.seed(3)
    torch.manual_seed(3)
    lin = ref.BlockSparseLinear(2048, 2048, bias=True, density=0.5)
    with torch.no_grad():
        lin.weight.data.normal_(0, 0.02)
        lin.bias.normal_(0, 0.02)
    x = torch.randn(8192, 2048, device="cuda")
    dy = torch.randn(8192, 2048, device="cuda")
    w = lin.weight
    shape, blocks, data = tuple(w.shape), w.blocks.cpu().numpy(), w.data.detach().cpu().numpy()
    rows = torch.arange(0, 8192, 86)[:96]
    want_y = orc.forward(x[rows].cpu().numpy(), shape, blocks, data, lin.bias.detach().cpu().numpy())
    want_dx = orc.dgrad(dy[rows].cpu().numpy(), shape, blocks, data)
    times = {}
    for precision in ("tf32x3", "fp32"):
        native.set_default_precision(precision)
        y, dx, dw = _step(lin, x, dy)
        torch.cuda.synchronize()
        assert orc.rel_fro(y[rows].cpu().numpy(), want_y) <= 1e-5
        assert orc.rel_fro(dx[rows].cpu().numpy(), want_dx) <= 1e-5
        coo = blocks.reshape(-1, 2)
        dwb = dw.view(-1, 32, 32)
        for s in range(0, coo.shape[0], max(1, coo.shape[0] // 6)):
            c, r = int(coo[s, 0]), int(coo[s, 1])
            want = (x[:, c * 32:(c + 1) * 32].double().t() @ dy[:, r * 32:(r + 1) * 32].double()).cpu().numpy()
            assert orc.rel_fro(dwb[s].cpu().numpy(), want) <= 1e-5
        for _ in range(2):
            _step(lin, x, dy)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(5):
            _step(lin, x, dy)
        torch.cuda.synchronize()
        times[precision] = (time.perf_counter() - t0) / 5
    assert times["tf32x3"] < times["fp32"], times
    assert_device_healthy()


def test_reference_block_replace_then_matmul(ref):
    """The reference's own block_replace (block_sparse.py:167-219) followed by its matmuls: the stand-in's cached
    plans are keyed on the index buffers, which rebuild() replaces."""
    np.random.seed(5)
    torch.manual_seed(5)
    m = ref.BlockSparseMatrix.randn((256, 128), n_blocks=9, device="cuda")
    a = torch.randn(64, 128, device="cuda")
    def want():
        return orc.forward(a.cpu().numpy(), tuple(m.shape), m.blocks.cpu().numpy(), m.data.detach().cpu().numpy())

    y0 = m.reverse_matmul(a, transpose=True)
    assert orc.rel_fro(y0.cpu().numpy(), want()) <= 1e-5
    free = (~m.block_mask_build(None)).nonzero()
    m.block_replace(torch.cat([free[:2], torch.tensor([[0], [5]], device=free.device)], -1))
    y1 = m.reverse_matmul(a, transpose=True)
    assert orc.rel_fro(y1.cpu().numpy(), want()) <= 1e-5
    assert not torch.equal(y0, y1)
    assert_device_healthy()
