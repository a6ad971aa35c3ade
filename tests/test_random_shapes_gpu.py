"""Seeded random shapes, densities, token counts and block sizes against a float64 dense product of
``to_dense()`` (itself pinned to the oracle's fixtures): forward with bias, input gradient, weight gradient in the
three tensor-core precisions, bf16 tensors, and the fused epilogue.  The draw includes what the hand-written cases
do not enumerate: very sparse patterns with whole groups of empty block-rows, single blocks, ragged token counts
around the 128-token tile, launches in which every CTA walks many tiles."""
import random

import numpy as np
import pytest
import torch

from pytorch_block_sparse_b200 import BlockSparseMatrix, native

from .gpu_util import assert_device_healthy

pytestmark = pytest.mark.gpu

TOL = {"tf32x3": 1e-5, "bf16x3": 1e-5, "tf32": 3e-3, "bf16": 1.5e-2}
TOKENS = [1, 2, 31, 32, 33, 64, 100, 127, 128, 129, 255, 256, 500, 1000, 1024, 2048, 4100, 9000, 20000]
DENSITIES = [0.02, 0.05, 0.1, 0.25, 0.5, 0.9, 1.0]


def _rel(got, want):
    return float((got.detach().double() - want).norm() / max(float(want.norm()), 1e-30))


@pytest.mark.parametrize("seed", [1000, 2000, 3000])
def test_random_cases(seed):
    rng = random.Random(seed)
    for case in range(40):
        bs = rng.choice([32, 32, 32, 64, 128])
        n = bs * rng.randint(1, max(1, 1536 // bs))
        k = bs * rng.randint(1, max(1, 1536 // bs))
        tokens = rng.choice(TOKENS)
        nnz = max(1, int((n // bs) * (k // bs) * rng.choice(DENSITIES)))
        np.random.seed(seed + case)
        torch.manual_seed(seed + case)
        w = BlockSparseMatrix.zeros((n, k), n_blocks=nnz, block_shape=(bs, bs), device="cuda")
        with torch.no_grad():
            w.data.normal_(0, 0.05)
        x = torch.randn(tokens, k, device="cuda")
        dy = torch.randn(tokens, n, device="cuda")
        bias = torch.randn(n, device="cuda")
        dense = w.to_dense().detach().double()
        mask = w.to_dense(data_replace=torch.ones_like(w.data)).detach().double()
        want_y, want_dx = x.double() @ dense.t() + bias.double(), dy.double() @ dense
        want_dw = (dy.double().t() @ x.double()) * mask
        what = (seed, case, tokens, n, k, nnz, bs)
        for precision in ("tf32x3", "bf16x3", "tf32", "bf16"):
            y = w.reverse_matmul(x, True, bias=bias, precision=precision)
            dx = w.reverse_matmul(dy, False, precision=precision)
            dw = w.to_dense(data_replace=w.matmul_with_output_sparse_support(dy, x, precision=precision))
            assert _rel(y, want_y) <= TOL[precision], (what, precision, "fwd")
            assert _rel(dx, want_dx) <= TOL[precision], (what, precision, "dgrad")
            assert _rel(dw, want_dw) <= TOL[precision], (what, precision, "wgrad")
        if bs == 32:
            yb = w.reverse_matmul(x.bfloat16(), True, bias=bias, precision="bf16")
            assert yb.dtype == torch.bfloat16
            assert _rel(yb.float(), x.bfloat16().double() @ dense.t() + bias.double()) <= TOL["bf16"], (what, "bf16 tensors")
            res = torch.randn(tokens, n, device="cuda")
            out, _ = w.reverse_matmul_fused(x, bias=bias, residual=res, activation="gelu")
            assert _rel(out, torch.nn.functional.gelu(want_y + res.double())) <= 2e-5, (what, "fused epilogue")
        assert native.device_status(clear=True) == 0, what
    assert_device_healthy()


def test_random_layers_forward_and_backward():
    """The layer through autograd on random configurations -- block size, density, bias, fused activation and
    residual, leading dimensions, non-contiguous inputs -- against a float64 dense computation, and the weight
    gradient for all four storage orders of its operands."""
    from pytorch_block_sparse_b200 import BlockSparseLinear

    rng = random.Random(77)
    for case in range(30):
        np.random.seed(500 + case)
        torch.manual_seed(500 + case)
        bs = rng.choice([32, 32, 64])
        fin, fout = bs * rng.randint(1, 1024 // bs), bs * rng.randint(1, 1024 // bs)
        density = rng.choice([0.05, 0.1, 0.3, 0.6, 1.0])
        if int(density * fin * fout / (bs * bs)) < 1:
            density = 1.0
        act = rng.choice([None, "gelu"])
        use_res, use_bias = rng.random() < 0.5, rng.random() < 0.7
        lead = rng.choice([(7,), (3, 50), (2, 3, 41), (129,), (1000,), (4, 600)])
        lin = BlockSparseLinear(fin, fout, bias=use_bias, density=density, block_shape=(bs, bs), activation=act)
        with torch.no_grad():
            lin.weight.data.mul_(0.05)
            if use_bias:
                lin.bias.normal_(0, 0.3)
        x = torch.randn(*lead, fin, device="cuda")
        if rng.random() < 0.3:
            x = torch.randn(*lead[:-1], fin, lead[-1], device="cuda").transpose(-1, -2)
        x = x.detach().requires_grad_(True)
        res = torch.randn(*lead, fout, device="cuda", requires_grad=True) if use_res else None
        g = torch.randn(*lead, fout, device="cuda")
        y = lin(x, residual=res)
        y.backward(g)

        dense = lin.weight.to_dense().detach().double()
        mask = lin.weight.to_dense(data_replace=torch.ones_like(lin.weight.data)).detach().double()
        xd = x.detach().double().requires_grad_(True)
        wd = dense.clone().requires_grad_(True)
        pre = xd @ wd.t()
        bd = rd = None
        if use_bias:
            bd = lin.bias.detach().double().requires_grad_(True)
            pre = pre + bd
        if use_res:
            rd = res.detach().double().requires_grad_(True)
            pre = pre + rd
        want = torch.nn.functional.gelu(pre) if act == "gelu" else pre
        want.backward(g.double())
        what = (case, lead, fin, fout, density, bs, act, use_res, use_bias)
        pairs = [(y, want.detach()), (x.grad, xd.grad),
                 (lin.weight.to_dense(data_replace=lin.weight.data.grad), wd.grad * mask)]
        if use_bias:
            pairs.append((lin.bias.grad, bd.grad))
        if use_res:
            pairs.append((res.grad, rd.grad))
        for got, ref in pairs:
            assert _rel(got, ref) <= 2e-5, what

        tokens = int(np.prod(lead))
        a, b = g.reshape(tokens, fout), x.detach().reshape(tokens, fin)
        ref_dw = lin.weight.matmul_with_output_sparse_support(a.contiguous(), b.contiguous())
        for a_fm in (False, True):
            for b_fm in (False, True):
                aa = a.t().contiguous().t() if a_fm else a.contiguous()
                bb = b.t().contiguous().t() if b_fm else b.contiguous()
                assert _rel(lin.weight.matmul_with_output_sparse_support(aa, bb), ref_dw.double()) <= 1e-5, (what, a_fm, b_fm)
        assert native.device_status(clear=True) == 0, what
    assert_device_healthy()
