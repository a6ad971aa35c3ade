"""``torch.nn.DataParallel`` over the layer (reference tests/test_data_parallel.py:11-17): one process, one thread
per GPU, replicas made by ``replicate()``.  The reference only checks that the forward runs; here the output and
the gradients are also compared with the single-GPU layer.  Skipped with fewer than two GPUs."""
import numpy as np
import pytest
import torch

from pytorch_block_sparse_b200 import BlockSparseLinear, native

pytestmark = pytest.mark.gpu


def test_data_parallel_forward_and_backward():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    np.random.seed(3)
    torch.manual_seed(3)
    linear = BlockSparseLinear(64, 128, False).to("cuda")      # the reference's case
    model = torch.nn.DataParallel(linear, device_ids=[0, 1])
    x = torch.randn(64, 64).cuda()
    out = model(x)
    assert out.shape == (64, 128)
    assert torch.allclose(out, linear(x), atol=1e-5, rtol=1e-5)

    big = BlockSparseLinear(256, 512, True, density=0.3).to("cuda")
    with torch.no_grad():
        big.weight.data.mul_(0.05)
    par = torch.nn.DataParallel(big, device_ids=[0, 1])
    xb = torch.randn(4, 75, 256, device="cuda", requires_grad=True)
    g = torch.randn(4, 75, 512, device="cuda")
    par(xb).backward(g)
    got = (xb.grad.clone(), big.weight.data.grad.clone(), big.bias.grad.clone())
    xb.grad = None
    big.zero_grad(set_to_none=True)
    big(xb).backward(g)
    want = (xb.grad, big.weight.data.grad, big.bias.grad)
    for a, b in zip(got, want):
        assert float((a.double() - b.double()).norm() / b.double().norm()) < 1e-5
    for dev in (0, 1):
        with torch.cuda.device(dev):
            assert native.device_status() == 0
