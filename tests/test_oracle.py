"""Pins the CPU oracle: every function of oracle/block_sparse_oracle.py against vectors produced by
the reference itself (tests/golden/*.npz) and the literal vectors in the reference's tests."""
import numpy as np

from oracle import block_sparse_oracle as orc

INDEX_KEYS = ("blocks", "cols_a", "row_start_ends_a", "rows_b", "col_start_ends_b")


def test_literal_vectors_of_reference_test_basic():
    # pytorch_block_sparse/tests/test_basic.py:11-46
    mask = orc.mask_from_blocks((128, 64), [(0, 0), (1, 0), (2, 0), (0, 1)])
    idx = orc.build_indices(mask)
    assert idx["row_start_ends_a"].tolist() == [0, 2, 3, 4, 4]
    assert idx["cols_a"].tolist() == [[0, 0], [1, 1], [0, 2], [0, 3]]
    assert idx["col_start_ends_b"].tolist() == [0, 3, 4]
    assert idx["rows_b"].tolist() == [[0, 0], [1, 2], [2, 3], [0, 1]]
    assert idx["blocks"].tolist() == [0, 0, 1, 0, 0, 1, 0, 2]


def test_literal_vectors_of_reference_test_replace():
    # pytorch_block_sparse/tests/test_replace.py:23-43
    mask = orc.mask_from_blocks((128, 64), [(0, 0), (1, 0), (2, 0), (0, 1)])
    idx = orc.build_indices(mask)
    coo = orc.coo_from_indices(idx["row_start_ends_a"], idx["cols_a"])
    assert coo.T.tolist() == [[0, 0], [0, 1], [1, 0], [2, 0]]
    new_mask, ptr = orc.block_replace((128, 64), idx["row_start_ends_a"], idx["cols_a"], [(3, 1, 0), (2, 1, 2), (1, 1, 1)])
    after = orc.build_indices(new_mask, ptr)
    assert after["row_start_ends_a"].tolist() == [0, 0, 1, 3, 4]
    assert after["cols_a"].tolist() == [[1, 1], [0, 3], [1, 2], [1, 0]]
    assert new_mask.astype(int).tolist() == [[0, 0], [0, 1], [1, 1], [0, 1]]
    assert after["col_start_ends_b"].tolist() == [0, 1, 4]
    assert after["rows_b"].tolist() == [[2, 3], [1, 1], [2, 2], [3, 0]]
    assert after["blocks"].tolist() == [1, 3, 1, 1, 1, 2, 0, 2]


def test_indices_against_reference_fixtures(golden):
    g = golden("indices")
    for name in g["names"]:
        shape = tuple(g[f"{name}/shape"])
        seed = int(g[f"{name}/seed"])
        if seed >= 0:  # the oracle draws the pattern exactly like the reference: global numpy RNG
            np.random.seed(seed)
            mask = orc.random_mask(shape, int(g[f"{name}/n"]))
            assert (mask == g[f"{name}/mask"]).all(), name
        else:
            mask = g[f"{name}/mask"]
        idx = orc.build_indices(mask)
        for k in INDEX_KEYS:
            assert idx[k].dtype == np.int32
            assert np.array_equal(idx[k], g[f"{name}/{k}"]), (name, k)
        coo = orc.coo_from_indices(idx["row_start_ends_a"], idx["cols_a"])
        assert np.array_equal(coo.T.reshape(-1, 2)[:, ::-1].reshape(-1), idx["blocks"])


def test_block_replace_against_reference_fixtures(golden):
    g = golden("replace")
    for name in g["names"]:
        shape = tuple(g[f"{name}/shape"])
        mask, ptr = orc.block_replace(
            shape, g[f"{name}/before/row_start_ends_a"], g[f"{name}/before/cols_a"], g[f"{name}/replacements"]
        )
        assert np.array_equal(mask, g[f"{name}/after/mask"])
        after = orc.build_indices(mask, ptr)
        for k in INDEX_KEYS:
            assert np.array_equal(after[k], g[f"{name}/after/{k}"]), (name, k)


def test_dense_conversions_against_reference_fixtures(golden):
    g = golden("dense")
    shape = tuple(g["shape"])
    dense = orc.to_dense(shape, g["blocks"], g["data"])
    assert np.array_equal(dense, g["dense"])
    assert np.array_equal(orc.from_dense(dense, g["blocks"]), g["data"])
    assert np.array_equal(orc.from_dense(g["fd_dense"], g["fd_blocks"]), g["fd_data"])
    assert np.array_equal(orc.from_dense_truncating(g["fd_dense"], 3), g["fd_trunc_data"])
    assert np.allclose(orc.block_norm(g["data"]), g["block_norm"], rtol=1e-6)


def test_contractions_against_reference_fixtures(golden):
    g = golden("linear")
    shape = tuple(g["small/shape"])
    blocks, data = g["small/blocks"], g["small/data"]
    x, dy, bias = g["small/x"], g["small/dy"], g["small/bias"]
    y = orc.forward(x, shape, blocks, data, bias)
    dx = orc.dgrad(dy, shape, blocks, data)
    dw = orc.wgrad(dy, x, shape, blocks)
    # the fixture is the reference's fp32 torch.matmul result; the oracle computes in float64
    assert orc.rel_fro(y.reshape(-1, shape[0]), g["small/y"]) < 2e-6
    assert orc.rel_fro(dx.reshape(-1, shape[1]), g["small/dx"]) < 2e-6
    assert orc.rel_fro(dw, g["small/dw"]) < 2e-6
