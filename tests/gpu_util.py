"""Helpers shared by the GPU parity tests: seeded cases and oracle comparison."""
import numpy as np
import torch

from oracle import block_sparse_oracle as orc
from pytorch_block_sparse_b200 import BlockSparseMatrix, native

# relative Frobenius error bounds (fp32-class modes: the bar of the reference-parity contract)
TOL = {"fp32": 1e-5, "tf32x3": 1e-5, "bf16x3": 1e-5, "tf32": 2e-3, "bf16": 1e-2}


def make_matrix(shape, n_blocks=None, blocks=None, seed=0, std=0.02, positive=False):
    """BlockSparseMatrix on cuda:0; pattern from numpy's global RNG (the reference's generator)."""
    np.random.seed(seed)
    torch.manual_seed(seed)
    m = BlockSparseMatrix.zeros(shape, n_blocks=n_blocks, blocks=blocks, device="cuda")
    data = torch.randn(m.data.shape) * std
    if positive:
        data = data.abs()
    with torch.no_grad():
        m.data.copy_(data.cuda())
    return m


def randn(shape, seed, positive=False):
    g = torch.Generator().manual_seed(seed)
    t = torch.randn(shape, generator=g)
    return t.abs() if positive else t


def host(m):
    return tuple(m.shape), m.blocks.cpu().numpy(), m.data.detach().cpu().numpy()


def check(got, want, precision, what=""):
    got = got.detach().float().cpu().numpy()
    err = orc.rel_fro(got.reshape(want.shape), want)
    assert np.isfinite(got).all(), what
    assert err <= TOL[precision], f"{what}: relative Frobenius error {err:.3e} > {TOL[precision]:.0e}"
    return err


def assert_device_healthy():
    assert native.device_status(clear=True) == 0, "a tensor-core kernel abandoned a bounded wait"
