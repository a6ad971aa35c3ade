"""Host-side logic of the package on CPU: index buffers, block_replace, densification, state-dict
contract, error behaviour -- bit-exact against the reference fixtures and the oracle."""
import io

import numpy as np
import pytest
import torch

from oracle import block_sparse_oracle as orc
from pytorch_block_sparse_b200 import BlockSparseMatrix, BlockSparseMatrixEmulator, SparseOptimizer
from pytorch_block_sparse_b200.util import BlockSparseModelPatcher

INDEX_KEYS = ("blocks", "cols_a", "row_start_ends_a", "rows_b", "col_start_ends_b")


def test_reference_test_basic_vectors():
    m = BlockSparseMatrix.randn((128, 64), None, blocks=[(0, 0), (1, 0), (2, 0), (0, 1)], device="cpu")
    assert m.row_start_ends_a.tolist() == [0, 2, 3, 4, 4]
    assert m.cols_a.tolist() == [[0, 0], [1, 1], [0, 2], [0, 3]]
    assert m.col_start_ends_b.tolist() == [0, 3, 4]
    assert m.rows_b.tolist() == [[0, 0], [1, 2], [2, 3], [0, 1]]
    for k in INDEX_KEYS:
        assert getattr(m, k).dtype == torch.int32
    hash(m)


def test_indices_match_reference_fixtures(golden):
    g = golden("indices")
    for name in g["names"]:
        shape = tuple(int(v) for v in g[f"{name}/shape"])
        seed = int(g[f"{name}/seed"])
        if seed >= 0:
            np.random.seed(seed)
            m = BlockSparseMatrix.zeros(shape, n_blocks=int(g[f"{name}/n"]), device="cpu")
        else:
            m = BlockSparseMatrix.zeros(shape, blocks=[(0, 0), (1, 0), (2, 0), (0, 1)], device="cpu")
        for k in INDEX_KEYS:
            assert np.array_equal(getattr(m, k).numpy(), g[f"{name}/{k}"]), (name, k)
        assert np.array_equal(m.block_mask_build(None).numpy(), g[f"{name}/mask"])


def test_block_replace_matches_reference_fixtures(golden):
    g = golden("replace")
    for name in g["names"]:
        shape = tuple(int(v) for v in g[f"{name}/shape"])
        mask = torch.zeros(shape[0] // 32, shape[1] // 32, dtype=torch.bool)
        coo = orc.coo_from_indices(g[f"{name}/before/row_start_ends_a"], g[f"{name}/before/cols_a"])
        mask[coo[0], coo[1]] = True
        n = coo.shape[1]
        m = BlockSparseMatrix(shape, mask, torch.arange(n * 1024, dtype=torch.float32).reshape(n * 32, 32))
        dense_before = m.to_dense()
        m.check_ = True
        repl = torch.tensor(g[f"{name}/replacements"])
        m.block_replace(repl)
        for k in INDEX_KEYS:
            assert np.array_equal(getattr(m, k).numpy(), g[f"{name}/after/{k}"]), (name, k)
        # data moves with its slot (reference tests/test_replace.py:104-129)
        dense_after = m.to_dense()
        for r, c, s in repl.tolist():
            r0, c0 = int(coo[0, s]), int(coo[1, s])
            assert torch.equal(dense_after[r * 32:(r + 1) * 32, c * 32:(c + 1) * 32],
                               dense_before[r0 * 32:(r0 + 1) * 32, c0 * 32:(c0 + 1) * 32])


def test_block_replace_rejects_used_position():
    m = BlockSparseMatrix.zeros((128, 64), blocks=[(0, 0), (1, 0), (2, 0), (0, 1)], device="cpu")
    m.check_ = True
    with pytest.raises(Exception, match=r"Block position \(0,1\) was already used"):
        m.block_replace(torch.tensor([(0, 1, 0)]))


def test_dense_round_trips(golden):
    g = golden("dense")
    shape = tuple(int(v) for v in g["shape"])
    coo = g["blocks"].reshape(-1, 2)
    m = BlockSparseMatrix.zeros(shape, blocks=[(int(r), int(c)) for c, r in coo], device="cpu")
    assert np.array_equal(m.blocks.numpy(), g["blocks"])
    with torch.no_grad():
        m.data.copy_(torch.from_numpy(g["data"]))
    dense = m.to_dense()
    assert np.array_equal(dense.detach().numpy(), g["dense"])
    m.check_with_dense(dense)
    assert np.allclose(m.block_norm().detach().numpy(), g["block_norm"], rtol=1e-6)
    assert np.array_equal(m.to_sparse().to_dense().permute(0, 2, 1, 3).reshape(shape).detach().numpy(), g["dense"])

    fd = BlockSparseMatrix.from_dense(torch.from_numpy(g["fd_dense"]), blocks=[(0, 0), (1, 2), (0, 1)])
    assert np.array_equal(fd.blocks.numpy(), g["fd_blocks"])
    assert np.array_equal(fd.data.detach().numpy(), g["fd_data"])
    slow = BlockSparseMatrix.from_dense(torch.from_numpy(g["fd_dense"]), blocks=[(0, 0), (1, 2), (0, 1)], slow=True)
    assert torch.equal(slow.data, fd.data)
    np.random.seed(22)
    tr = BlockSparseMatrix.from_dense(torch.from_numpy(g["fd_dense"]), block_count=3)
    assert np.array_equal(tr.blocks.numpy(), g["fd_trunc_blocks"])
    assert np.array_equal(tr.data.detach().numpy(), g["fd_trunc_data"])


def test_full_round_trip_sizes():
    # reference tests/test_basic.py:48-67
    for size in [(32, 32), (64, 32), (32, 64), (64, 64), (256, 64)]:
        n = size[0] * size[1] // 1024
        m = BlockSparseMatrix.randn(size, n, device="cpu")
        a = m.to_dense()
        m2 = BlockSparseMatrix.from_dense(a, (32, 32), block_count=None)
        m2.check_with_dense(a)
        assert torch.equal(a, m2.to_dense())


def test_constructor_errors():
    with pytest.raises(Exception, match="multiples of 32"):
        BlockSparseMatrix((48, 32), torch.ones(1, 1, dtype=torch.bool), torch.zeros(32, 32))
    with pytest.raises(Exception, match="Invalid shape"):
        BlockSparseMatrix.zeros((48, 32), 1, device="cpu")
    with pytest.raises(Exception, match="Too many blocks"):
        BlockSparseMatrix.zeros((32, 32), 2, device="cpu")
    with pytest.raises(Exception, match="float32"):
        BlockSparseMatrix((32, 32), torch.ones(1, 1, dtype=torch.bool), torch.zeros(32, 32, dtype=torch.float64))
    m = BlockSparseMatrix.zeros((32, 64), 1, device="cpu")
    with pytest.raises(Exception, match="no CPU path|only on CUDA"):
        m.reverse_matmul(torch.zeros(4, 64), transpose=True)
    with pytest.raises(Exception, match="at least 2 dimensions"):
        m.flatten_first_dims(torch.zeros(4))


def test_state_dict_contract():
    # reference tests/test_save.py: whole-module pickle and state_dict round trip
    np.random.seed(5)
    m = BlockSparseMatrix.randn((128, 96), 5, device="cpu")
    sd = m.state_dict()
    assert list(sd.keys()) == ["data", "cols_a", "row_start_ends_a", "rows_b", "col_start_ends_b", "blocks"]
    np.random.seed(6)
    m2 = BlockSparseMatrix.zeros((128, 96), 5, device="cpu")
    m2.load_state_dict(sd)
    assert torch.equal(m2.to_dense(), m.to_dense())
    buf = io.BytesIO()
    torch.save(m, buf)
    buf.seek(0)
    m3 = torch.load(buf, weights_only=False)
    assert torch.equal(m3.to_dense(), m.to_dense())


def test_emulator_cpu():
    # reference tests/test_emulate.py
    for bs in [(32, 32), (4, 8), (4, 1)]:
        shape = (bs[0] * 4, bs[1] * 6)
        m = BlockSparseMatrixEmulator.randn(shape, 7, block_shape=bs, device="cpu")
        dense = m.to_dense()
        a = BlockSparseMatrixEmulator.from_dense(dense, bs, blocks=[tuple(int(v) for v in p) for p in m.build_coo_block_index().t()])
        b = BlockSparseMatrixEmulator.from_dense(dense, bs, blocks=[tuple(int(v) for v in p) for p in m.build_coo_block_index().t()], slow=True)
        assert torch.equal(a.data, b.data) and torch.equal(a.data, m.data)
        x = torch.randn(5, shape[1])
        assert torch.allclose(m.reverse_matmul(x, transpose=True), x @ dense.t(), atol=1e-5)
        dy = torch.randn(5, shape[0])
        assert torch.allclose(m.reverse_matmul(dy, transpose=False), dy @ dense, atol=1e-5)
        mask = m._mask.float()
        assert torch.allclose(m.matmul_with_output_sparse_support(dy, x), (dy.t() @ x) * mask, atol=1e-5)


def test_sparse_optimizer_step_counts_cpu():
    # reference tests/test_sparse_optimizer.py:18-55: one step moves int(ratio*n) blocks
    np.random.seed(0)
    torch.manual_seed(0)
    m = BlockSparseMatrix.randn((256, 256), 32, device="cpu")
    before = m.block_mask_build(None).clone()
    ratio = 0.25
    opt = SparseOptimizer([m], lr=ratio)
    opt.step()
    after = m.block_mask_build(None)
    assert int((before != after).sum()) == 2 * int(ratio * 32)
    assert int(after.sum()) == 32


def test_sparse_optimizer_masks_adam_state_cpu():
    np.random.seed(1)
    torch.manual_seed(1)
    m = BlockSparseMatrix.randn((128, 128), 8, device="cpu")
    adam = torch.optim.Adam([m.data], lr=1e-3)
    m.data.grad = torch.ones_like(m.data)
    adam.step()
    opt = SparseOptimizer([m], lr=0.5)
    opt.attach_optimizer(adam)
    norms = m.block_norm()
    recycled = norms.sort()[1][:4]
    opt.step()
    st = adam.state[m.data]
    for s in range(8):
        blk = st["exp_avg"][s * 32:(s + 1) * 32]
        assert bool((blk == 0).all()) == (s in recycled.tolist())


def test_patcher_names_cpu():
    model = torch.nn.Sequential(torch.nn.Linear(64, 64), torch.nn.ReLU(), torch.nn.Linear(64, 32))
    mp = BlockSparseModelPatcher()
    names = [d["regexp"] for d in mp.get_patchable_layers(model)]
    assert names == ["0", "2"]
    mp.add_pattern("1", {"density": 0.5})
    with pytest.raises(Exception, match="not a Linear layer"):
        mp.patch_model(model)


def _layer_shaped(weight, bias):
    class LayerShaped(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = weight
            self.bias = torch.nn.Parameter(bias)

    return LayerShaped()


def test_checkpoint_written_by_the_reference_loads(golden):
    """tests/golden/checkpoint.npz is the state_dict the REFERENCE produces for one layer (keys of
    reference block_sparse.py:23,58-65) after a block_replace, i.e. with slot order != row-major order.
    Loading it into a matrix of this package built with another pattern must reproduce the reference's dense
    weight exactly: the index buffers travel with the checkpoint."""
    g = golden("checkpoint")
    sd = {k: torch.from_numpy(g["sd/" + k]) for k in g["keys"]}
    np.random.seed(7)
    m = BlockSparseMatrix.zeros((128, 192), n_blocks=9, device="cpu")
    layer = _layer_shaped(m, torch.zeros(128))
    assert sorted(layer.state_dict().keys()) == sorted(sd.keys())
    assert not np.array_equal(m.blocks.numpy(), g["sd/weight.blocks"])
    layer.load_state_dict(sd, strict=True)
    assert np.array_equal(m.to_dense().detach().numpy(), g["dense"])
    y = torch.from_numpy(g["x"]) @ m.to_dense().t() + layer.bias
    assert np.allclose(y.detach().numpy(), g["y"], rtol=1e-6, atol=1e-6)
    # and back out: what this package saves is what the reference saved
    for k, v in layer.state_dict().items():
        assert np.array_equal(v.numpy(), g["sd/" + k]), k


@pytest.mark.parametrize("block_shape", [(32, 32), (64, 64)])
def test_bsr_round_trip(block_shape):
    np.random.seed(8)
    torch.manual_seed(8)
    m = BlockSparseMatrix.randn((256, 384), n_blocks=7, block_shape=block_shape, device="cpu")
    free = (~m.block_mask_build(None)).nonzero()
    m.block_replace(torch.cat([free[:1], torch.tensor([[3]])], -1))  # slot order != row-major order
    bsr = m.to_bsr()
    assert bsr.layout == torch.sparse_bsr
    assert torch.equal(bsr.to_dense(), m.to_dense())
    back = BlockSparseMatrix.from_bsr(bsr)
    assert torch.equal(back.to_dense(), m.to_dense())
    assert torch.equal(back.row_start_ends_a, m.row_start_ends_a)
    assert torch.equal(back.cols_a[:, 0], m.cols_a[:, 0])
    assert torch.equal(back.col_start_ends_b, m.col_start_ends_b)
    assert torch.equal(back.rows_b[:, 0], m.rows_b[:, 0])
    # a BSR tensor whose columns are not sorted inside a row
    crow = torch.tensor([0, 2, 2]); col = torch.tensor([1, 0]); vals = torch.randn(2, 32, 32)
    odd = torch.sparse_bsr_tensor(crow, col, vals, size=(64, 64))
    got = BlockSparseMatrix.from_bsr(odd)
    want = torch.zeros(64, 64); want[:32, 32:] = vals[0]; want[:32, :32] = vals[1]
    assert torch.equal(got.to_dense(), want)


def test_larger_square_blocks_expand_to_the_same_non_zeros():
    """64x64 and 128x128 matrices run on the 32x32 kernels through a derived fine matrix: same dense matrix,
    and the two re-tilings are inverse to each other."""
    for b in (64, 128):
        np.random.seed(b)
        torch.manual_seed(b)
        m = BlockSparseMatrix.randn((256, 512), n_blocks=3, block_shape=(b, b), device="cpu")
        fine = m._fine_matrix()
        assert fine.block_shape == (32, 32) and fine.data.shape[0] == m.data.shape[0] * (b // 32)
        with torch.no_grad():
            fine.data.copy_(m._to_fine(m.data.detach()))
        assert torch.equal(fine.to_dense(), m.to_dense())
        assert torch.equal(m._from_fine(fine.data), m.data.detach())
        assert "_fine" not in "".join(m.state_dict().keys())
