"""GPU tests of the layer-level API: autograd through BlockSparseLinear against a dense masked
twin (reference tests/test_linear_nn.py), checkpoint round trips (tests/test_save.py), model
patching (tests/test_integration.py:37-64) and the sparsity optimizer (tests/test_sparse_optimizer.py)."""
import io

import numpy as np
import pytest
import torch

from pytorch_block_sparse_b200 import (
    BlockSparseLinear,
    BlockSparseMatrix,
    BlockSparseModelPatcher,
    PseudoBlockSparseLinear,
    SparseOptimizer,
    native,
)

from .gpu_util import assert_device_healthy

pytestmark = pytest.mark.gpu


class DenseTwin(torch.nn.Module):
    """nn.Linear whose weight is masked to the sparse layer's pattern every forward."""

    def __init__(self, sparse):
        super().__init__()
        w = sparse.weight
        self.weight = torch.nn.Parameter(w.to_dense().detach().clone())
        self.register_buffer("mask", w.to_dense(data_replace=torch.ones_like(w.data)).detach())
        self.bias = None if sparse.bias is None else torch.nn.Parameter(sparse.bias.detach().clone())

    def forward(self, x):
        return torch.nn.functional.linear(x, self.weight * self.mask, self.bias)


@pytest.mark.parametrize("precision,atol", [("fp32", 1e-5), ("tf32x3", 1e-5), ("bf16x3", 3e-5)])
@pytest.mark.parametrize("bias", [True, False])
def test_training_steps_match_dense_masked_twin(precision, atol, bias):
    # reference tests/test_linear_nn.py:58-134: output, dX and dW agree step after step under Adam, 40 steps
    native.set_default_precision(precision)
    try:
        np.random.seed(0)
        torch.manual_seed(0)
        torch.backends.cuda.matmul.allow_tf32 = False
        lin = BlockSparseLinear(256, 128, bias=bias, density=0.4)
        with torch.no_grad():
            lin.weight.data.mul_(0.05)
            if bias:
                lin.bias.normal_(0, 0.02)
        twin = DenseTwin(lin).cuda()
        opt_a = torch.optim.Adam(lin.parameters(), lr=1e-3)
        opt_b = torch.optim.Adam(twin.parameters(), lr=1e-3)
        for step in range(40):
            x = torch.randn(8, 50, 256, device="cuda", requires_grad=True)
            x2 = x.detach().clone().requires_grad_(True)
            y, y2 = lin(x), twin(x2)
            assert torch.allclose(y, y2, atol=atol, rtol=1e-4), (step, (y - y2).abs().max())
            g = torch.randn_like(y)
            opt_a.zero_grad()
            opt_b.zero_grad()
            y.backward(g)
            y2.backward(g)
            assert torch.allclose(x.grad, x2.grad, atol=atol, rtol=1e-4), step
            dw = lin.weight.to_dense(data_replace=lin.weight.data.grad)
            dw2 = twin.weight.grad * twin.mask
            # (entries of a gradient block are sums of 400 products of N(0,1) values: 1e-5 of their scale is 2e-4)
            assert torch.allclose(dw, dw2, atol=20 * atol, rtol=1e-4), (step, (dw - dw2).abs().max())
            if bias:
                assert torch.allclose(lin.bias.grad, twin.bias.grad, atol=1e-4, rtol=1e-4)
            opt_a.step()
            opt_b.step()
        assert_device_healthy()
    finally:
        native.set_default_precision("tf32x3")


def test_from_torch_linear_and_pseudo_layer():
    np.random.seed(1)
    torch.manual_seed(1)
    dense = torch.nn.Linear(128, 64).cuda()
    full = BlockSparseLinear(0, 0, False, torch_nn_linear=dense, density=1.0)
    x = torch.randn(33, 128, device="cuda")
    assert torch.allclose(full(x), dense(x), atol=1e-5)
    half = BlockSparseLinear(0, 0, False, torch_nn_linear=dense, density=0.5)
    assert half.block_count == 4 and half.weight.data.shape == (4 * 32, 32)
    # density < 1 keeps the first nnz*1024 dense values, rescaled (reference block_sparse.py:345-350)
    want = dense.weight.detach().flatten()[: 4 * 1024].reshape(128, 32) / np.sqrt(0.5)
    assert torch.allclose(half.weight.data, want)
    pseudo = PseudoBlockSparseLinear(half)
    assert torch.allclose(pseudo(x), half(x), atol=1e-5)


def test_save_and_load():
    # reference tests/test_save.py:11-51
    np.random.seed(2)
    lin = BlockSparseLinear(64, 128, True, density=0.5)
    x = torch.randn(10, 64, device="cuda")
    y = lin(x)
    keys = list(lin.state_dict().keys())
    assert keys == ["bias", "weight.data", "weight.cols_a", "weight.row_start_ends_a", "weight.rows_b",
                    "weight.col_start_ends_b", "weight.blocks"]
    buf = io.BytesIO()
    torch.save(lin.state_dict(), buf)
    buf.seek(0)
    np.random.seed(3)
    other = BlockSparseLinear(64, 128, True, density=0.5)
    assert not torch.allclose(other(x), y)
    other.load_state_dict(torch.load(buf))
    assert torch.equal(other(x), y)  # plans and packed weights were rebuilt from the loaded buffers
    buf = io.BytesIO()
    torch.save(lin, buf)
    buf.seek(0)
    assert torch.equal(torch.load(buf, weights_only=False)(x), y)


def test_patcher_parameter_counts():
    model = torch.nn.Sequential(torch.nn.Linear(128, 256), torch.nn.ReLU(), torch.nn.Linear(256, 64)).cuda()
    before = sum(p.numel() for p in model.parameters())
    mp = BlockSparseModelPatcher()
    mp.add_pattern("0", {"density": 0.5})
    mp.add_pattern("2", {"density": 0.25})
    mp.patch_model(model)
    after = sum(p.numel() for p in model.parameters())
    assert isinstance(model[0], BlockSparseLinear) and isinstance(model[2], BlockSparseLinear)
    assert before - after == 128 * 256 // 2 + 256 * 64 * 3 // 4
    y = model(torch.randn(5, 128, device="cuda"))
    y.sum().backward()
    assert model[0].weight.data.grad.shape == model[0].weight.data.shape


def test_sparse_optimizer_with_adam_on_gpu():
    # reference tests/test_sparse_optimizer.py:57-90
    np.random.seed(4)
    torch.manual_seed(4)
    lin = BlockSparseLinear(256, 256, True, density=0.5)
    adam = torch.optim.Adam(lin.parameters(), lr=1e-3)
    so = SparseOptimizer(SparseOptimizer.sparse_objects(lin), lr=0.25)
    so.attach_optimizer(adam)
    x = torch.randn(64, 256, device="cuda")
    lin(x).square().mean().backward()
    adam.step()
    before = lin.weight.block_mask_build(None).clone()
    so.step()
    after = lin.weight.block_mask_build(None)
    assert int((before != after).sum()) == 2 * int(0.25 * lin.block_count)
    y = lin(x)  # the new pattern is picked up by fresh plans
    dense = lin.weight.to_dense()
    assert torch.allclose(y, x @ dense.t() + lin.bias, atol=1e-4)
    assert_device_healthy()


def test_data_parallel_forward():
    # reference tests/test_data_parallel.py:11-17
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    lin = BlockSparseLinear(64, 128, False)
    model = torch.nn.DataParallel(lin)
    out = model(torch.randn(16, 64, device="cuda"))
    assert out.shape == (16, 128)


def test_nonsquare_block_shape_uses_emulator():
    lin = BlockSparseLinear(64, 32, True, density=0.5, block_shape=(4, 8))
    x = torch.randn(6, 64, device="cuda", requires_grad=True)
    y = lin(x)
    y.sum().backward()
    assert torch.allclose(y, x @ lin.weight.to_dense().t() + lin.bias, atol=1e-5)


def test_backward_thread_without_a_cuda_context():
    """The tensor maps are encoded by a driver entry point that needs a current context.  Autograd runs
    backward in a thread of its own; when the caching allocator serves all of that thread's allocations
    from memory freed earlier, the kernels' launcher is the first thing in the thread that needs the
    context.  Needs a fresh process: the backward thread lives as long as the process."""
    import subprocess
    import sys

    script = r'''
import numpy as np, torch
from pytorch_block_sparse_b200 import BlockSparseLinear
np.random.seed(0); torch.manual_seed(0)
lin = BlockSparseLinear(1024, 256, bias=True, density=0.5)
x = torch.randn(256, 1024, device="cuda"); dy = torch.randn(256, 256, device="cuda")
# the same computations in the main thread first: afterwards the allocator's cache holds every size that
# backward will ask for, and the backward thread makes no runtime call of its own before the launcher
w, b = lin.weight, lin.bias.detach()
for _ in range(3):
    y = w.reverse_matmul(x, transpose=True, bias=b)
    dx = w.reverse_matmul(dy, transpose=False)
    dw = w.matmul_with_output_sparse_support(dy, x)
    db = dy.sum(0)
    del y, dx, dw, db
torch.cuda.synchronize()
xd = x.detach().requires_grad_(True)
out = lin(xd)
out.backward(dy)
torch.cuda.synchronize()
assert torch.isfinite(xd.grad).all() and torch.isfinite(lin.weight.data.grad).all()
print("backward ok")
'''
    import os

    env = dict(os.environ)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    res = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env, timeout=300)
    assert res.returncode == 0 and "backward ok" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


def test_kernels_run_on_the_callers_stream():
    """Forward and backward issued under a side stream are ordered with that stream's work (the reference
    launches on the legacy default stream whatever the caller's stream is)."""
    import numpy as np

    from pytorch_block_sparse_b200 import BlockSparseLinear

    np.random.seed(3)
    torch.manual_seed(3)
    lin = BlockSparseLinear(384, 256, bias=True, density=0.4)
    x = torch.randn(700, 384, device="cuda")
    dy = torch.randn(700, 256, device="cuda")
    xr = x.clone().requires_grad_(True)
    lin(xr).backward(dy)
    want = (xr.grad.clone(), lin.weight.data.grad.clone())
    lin.weight.data.grad = None
    torch.cuda.synchronize()

    side = torch.cuda.Stream()
    big = torch.empty(64 << 20, device="cuda")
    with torch.cuda.stream(side):
        # a long fill first: the input written after it is only complete when the stream reaches our kernels
        for _ in range(4):
            big.normal_()
        xs = torch.zeros_like(x)
        xs.copy_(x)
        xs.requires_grad_(True)
        y = lin(xs)
        y.backward(dy)
    side.synchronize()
    assert torch.equal(xs.grad, want[0])
    assert torch.allclose(lin.weight.data.grad, want[1], rtol=1e-5, atol=1e-6)


def test_writes_through_dot_data_are_seen_by_the_next_forward():
    """``p.data.mul_()`` does not bump autograd's version counter (fused optimizers, EMA copies and
    ``weight.data.data[...] = ...`` write this way).  The layer packs its weight images on every forward, so the
    tensor-core paths cannot run on stale images; the opt-in cache (``fresh=False``) is dropped by
    ``invalidate_packed()``."""
    np.random.seed(21)
    torch.manual_seed(21)
    lin = BlockSparseLinear(128, 96, bias=False, density=0.5)
    x = torch.randn(40, 128, device="cuda")
    y0 = lin(x).detach().clone()
    version = lin.weight.data._version
    lin.weight.data.data.mul_(2.0)
    assert lin.weight.data._version == version  # the write is invisible to the version counter
    y1 = lin(x).detach()
    assert torch.allclose(y1, 2.0 * y0, rtol=1e-6, atol=0)
    # dgrad uses the images of its own forward
    xg = x.clone().requires_grad_(True)
    lin(xg).sum().backward()
    want = torch.ones(40, 96, device="cuda") @ lin.weight.to_dense()
    assert torch.allclose(xg.grad, want, rtol=1e-4, atol=1e-5)
    # the opt-in cache, and its invalidation
    w = lin.weight
    cached = w.packed_weights(fresh=False)
    assert w.packed_weights(fresh=False) is cached
    w.data.data.mul_(0.5)
    assert w.packed_weights(fresh=False) is cached  # stale by design until told
    w.invalidate_packed()
    assert w.packed_weights(fresh=False) is not cached
    y2 = w.reverse_matmul(x, transpose=True, packed=w.packed_weights(fresh=False))
    assert torch.allclose(y2, y0, rtol=1e-6, atol=0)


def test_block_norm_comes_from_the_statistic_kernel():
    np.random.seed(22)
    torch.manual_seed(22)
    lin = BlockSparseLinear(256, 128, bias=False, density=0.5)
    w = lin.weight
    want = torch.norm(w.data.detach().reshape(-1, 32, 32), p=2, dim=(1, 2))
    assert torch.allclose(w.block_norm(), want, rtol=1e-5)
    assert torch.allclose(w.block_norm(p=1), torch.norm(w.data.detach().reshape(-1, 32, 32), p=1, dim=(1, 2)), rtol=1e-5)
    # the weight gradient's statistic is kept beside the matrix
    x = torch.randn(64, 256, device="cuda", requires_grad=True)
    lin(x).sum().backward()
    g = w.data.grad.reshape(-1, 32, 32)
    assert torch.allclose(w.last_grad_block_sumsq, (g * g).sum((1, 2)), rtol=1e-4)


def test_checkpoint_written_by_the_reference_runs_on_the_kernels(golden):
    g = golden("checkpoint")
    np.random.seed(23)
    lin = BlockSparseLinear(192, 128, bias=True, density=9 / 24)
    assert lin.weight.data.shape == g["sd/weight.data"].shape
    lin(torch.randn(4, 192, device="cuda"))  # plans of the constructor's own pattern are cached now
    lin.load_state_dict({k: torch.from_numpy(g["sd/" + k]) for k in g["keys"]}, strict=True)
    y = lin(torch.from_numpy(g["x"]).cuda())
    err = float((y.detach().cpu().double() - torch.from_numpy(g["y"]).double()).norm() / np.linalg.norm(g["y"]))
    assert err <= 1e-5, err
    assert_device_healthy()


@pytest.mark.parametrize("block", [64, 128])
def test_larger_square_blocks_on_the_tensor_core_kernels(block):
    """A layer with 64x64 / 128x128 blocks (the reference serves them with its dense-masked emulator,
    block_sparse_linear.py:202-205): forward, input gradient and weight gradient against the dense masked layer."""
    np.random.seed(block)
    torch.manual_seed(block)
    lin = BlockSparseLinear(512, 384, bias=True, density=0.5, block_shape=(block, block))
    assert isinstance(lin.weight, BlockSparseMatrix) and lin.weight.block_shape == (block, block)
    with torch.no_grad():
        lin.weight.data.normal_(0, 0.05)
        lin.bias.normal_(0, 0.05)
    dense = lin.weight.to_dense().detach().double()
    mask = lin.weight.to_dense(data_replace=torch.ones_like(lin.weight.data)).double()
    x = torch.randn(3, 70, 512, device="cuda", requires_grad=True)
    dy = torch.randn(3, 70, 384, device="cuda")
    y = lin(x)
    y.backward(dy)
    xd, dyd = x.detach().double().reshape(-1, 512), dy.double().reshape(-1, 384)

    def rel(got, want):
        return float((got.double() - want).norm() / want.norm())

    assert rel(y.detach().reshape(-1, 384), xd @ dense.t() + lin.bias.detach().double()) <= 1e-5
    assert rel(x.grad.reshape(-1, 512), dyd @ dense) <= 1e-5
    want_dw = (dyd.t() @ xd) * mask
    got_dw = lin.weight.to_dense(data_replace=lin.weight.data.grad).double()
    assert rel(got_dw, want_dw) <= 1e-5
    assert rel(lin.bias.grad, dyd.sum(0)) <= 1e-5
    norms = lin.weight.block_norm()
    want_norms = torch.norm(lin.weight.data.detach().reshape(-1, block, block), dim=(1, 2))
    assert torch.allclose(norms, want_norms, rtol=1e-5)
    assert_device_healthy()


@pytest.mark.parametrize("activation,with_residual", [("gelu", False), (None, True), ("gelu", True)])
@pytest.mark.parametrize("density", [0.3, 1.0])
def test_fused_epilogue_matches_the_unfused_layer(activation, with_residual, density):
    """bias + residual + GELU applied inside the forward kernel against the same layer followed by torch ops,
    forward and all gradients.  Density 1.0 on 2048 input features gives rows of 64 blocks: two promotions per
    row, i.e. the path where the activation waits for the completed sum."""
    np.random.seed(31)
    torch.manual_seed(31)
    fused = BlockSparseLinear(2048, 128, bias=True, density=density, activation=activation)
    with torch.no_grad():
        fused.weight.data.normal_(0, 0.03)
        fused.bias.normal_(0, 0.5)
    plain = BlockSparseLinear(2048, 128, bias=True, density=density)
    plain.load_state_dict(fused.state_dict())
    x = torch.randn(3, 67, 2048, device="cuda")
    res = torch.randn(3, 67, 128, device="cuda") if with_residual else None
    dy = torch.randn(3, 67, 128, device="cuda")

    def run(layer, use_fused):
        xg = x.clone().requires_grad_(True)
        rg = res.clone().requires_grad_(True) if res is not None else None
        layer.weight.data.grad = None
        layer.bias.grad = None
        if use_fused:
            y = layer(xg, residual=rg)
        else:
            y = layer(xg)
            if rg is not None:
                y = y + rg
            if activation == "gelu":
                y = torch.nn.functional.gelu(y)
        y.backward(dy)
        return y.detach(), xg.grad, layer.weight.data.grad.clone(), layer.bias.grad.clone(), None if rg is None else rg.grad

    got, want = run(fused, True), run(plain, False)
    for g, w, what in zip(got, want, ("y", "dx", "dw", "dbias", "dres")):
        if w is None:
            continue
        err = float((g.double() - w.double()).norm() / w.double().norm())
        assert err <= 1e-5, (what, err)
    # inference path (no pre-activation kept)
    with torch.no_grad():
        y_eval = fused(x, residual=res)
    assert float((y_eval.double() - want[0].double()).norm() / want[0].double().norm()) <= 1e-5
    assert_device_healthy()


@pytest.mark.parametrize("precision,tol", [("tf32", 2e-3), ("bf16", 1e-2)])
def test_fused_epilogue_in_the_other_tensor_core_precisions(precision, tol):
    np.random.seed(33)
    torch.manual_seed(33)
    native.set_default_precision(precision)
    try:
        lin = BlockSparseLinear(1024, 256, bias=True, density=0.5, activation="gelu")
        with torch.no_grad():
            lin.weight.data.normal_(0, 0.03)
            lin.bias.normal_(0, 0.5)
        x = torch.randn(300, 1024, device="cuda")
        res = torch.randn(300, 256, device="cuda")
        want = torch.nn.functional.gelu(x.double() @ lin.weight.to_dense().detach().double().t() + lin.bias.detach().double() + res.double())
        got = lin(x, residual=res)
        assert float((got.double() - want).norm() / want.norm()) <= tol
        if precision == "bf16":  # bf16 tensors in memory: bias + GELU in the epilogue, bf16 result
            lin_b = BlockSparseLinear(1024, 256, bias=True, density=0.5, activation="gelu")
            lin_b.load_state_dict(lin.state_dict())
            with torch.no_grad():  # (with gradients the layer keeps an fp32 pre-activation and works on fp32 tensors)
                got_b = lin_b(x.bfloat16())
            want_b = torch.nn.functional.gelu(x.bfloat16().double() @ lin.weight.to_dense().detach().double().t() + lin.bias.detach().double())
            assert got_b.dtype == torch.bfloat16
            assert float((got_b.double() - want_b).norm() / want_b.norm()) <= tol
    finally:
        native.set_default_precision("tf32x3")
    assert_device_healthy()


def test_layer_step_replays_as_a_cuda_graph():
    # the library allocates nothing and synchronises nowhere, and its launches go to the caller's stream: one
    # forward + backward of the layer is capturable, and a replay on new inputs reproduces the eager result
    np.random.seed(5)
    torch.manual_seed(5)
    lin = BlockSparseLinear(256, 128, bias=True, density=0.4)
    x = torch.randn(96, 256, device="cuda", requires_grad=True)
    g = torch.randn(96, 128, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture: plans, symbol addresses, kernel attributes
        for _ in range(3):
            lin(x).backward(g)
    torch.cuda.current_stream().wait_stream(side)
    lin.zero_grad(set_to_none=True)
    x.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = lin(x)
        y.backward(g)
    for seed in (1, 2):
        gen = torch.Generator(device="cuda").manual_seed(seed)
        with torch.no_grad():
            x.copy_(torch.randn(96, 256, device="cuda", generator=gen))
            g.copy_(torch.randn(96, 128, device="cuda", generator=gen))
        graph.replay()
        torch.cuda.synchronize()
        got = (y.detach().clone(), x.grad.clone(), lin.weight.data.grad.clone(), lin.bias.grad.clone())
        x2 = x.detach().clone().requires_grad_(True)
        lin2_grads = torch.autograd.grad(lin(x2), (x2, lin.weight.data, lin.bias), g)
        assert torch.equal(got[0], lin(x2).detach())
        for a, b in zip(got[1:], lin2_grads):
            assert torch.equal(a, b)
    assert_device_healthy()
