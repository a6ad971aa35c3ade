"""GPU tests of the pattern kernels (csrc/bsmm_pattern.cu) through the C-ABI and of the sparsity optimizer
built on them: index buffers bit-exact against the reference-generated fixtures (reference
tests/test_replace.py:23-43, tests/test_basic.py:11-46) and against the host derivation, exact k-smallest
selection, uniform and reproducible sampling of empty positions, and the optimizer step
(reference tests/test_sparse_optimizer.py:18-55)."""
import numpy as np
import pytest
import torch

from pytorch_block_sparse_b200 import BlockSparseLinear, BlockSparseMatrix, SparseOptimizer, native
from pytorch_block_sparse_b200.sparse_optimizer import MagnitudeSparseOptimizerStrategy

from .gpu_util import assert_device_healthy

pytestmark = pytest.mark.gpu
INDEX_KEYS = ("blocks", "cols_a", "row_start_ends_a", "rows_b", "col_start_ends_b")


def _from_slot_order(shape, blocks_flat):
    """A CUDA matrix whose slot s sits at (blocks[2s+1], blocks[2s]) -- the fixture's (col, row) pairs."""
    pairs = np.asarray(blocks_flat).reshape(-1, 2)
    return BlockSparseMatrix.zeros(tuple(int(v) for v in shape), blocks=[(int(r), int(c)) for c, r in pairs], device="cuda")


@pytest.mark.parametrize("case", ["explicit", "random"])
def test_block_replace_on_the_device_matches_the_reference(case, golden):
    g = golden("replace")
    m = _from_slot_order(g[case + "/shape"], g[case + "/before/blocks"])
    for key in INDEX_KEYS:  # the fixture's "before" state has slots in row-major order
        assert np.array_equal(getattr(m, key).cpu().numpy(), g[f"{case}/before/{key}"]), key
    before_ptrs = {key: getattr(m, key).data_ptr() for key in INDEX_KEYS}
    m.block_replace(torch.from_numpy(g[case + "/replacements"]))
    for key in INDEX_KEYS:
        assert np.array_equal(getattr(m, key).cpu().numpy(), g[f"{case}/after/{key}"]), key
        assert getattr(m, key).data_ptr() == before_ptrs[key]  # rewritten in place by the kernels
    assert np.array_equal(m.block_mask_build(None).cpu().numpy(), g[case + "/after/mask"])
    assert m.pattern_status() == 0
    # the checking mode takes the host path and refuses an occupied target, with the reference's message
    m.check_ = True
    occupied = m.build_coo_block_index()[:, 0].tolist()
    with pytest.raises(Exception, match="was already used"):
        m.block_replace(torch.tensor([[occupied[0], occupied[1], 1]]))


@pytest.mark.parametrize("shape,n_blocks", [((4096, 4096), 4096), ((32768, 8192), 26214), ((96, 160), 15), ((32, 32), 1)])
def test_rebuild_indices_kernel_equals_host_derivation(shape, n_blocks):
    np.random.seed(n_blocks)
    m = BlockSparseMatrix.zeros(shape, n_blocks=n_blocks, device="cuda")
    X, Y = m.blocks_count()
    # shuffle the slots so that slot order differs from row-major order
    perm = torch.randperm(n_blocks, generator=torch.Generator().manual_seed(1)).cuda()
    pos = m.build_coo_block_index().long()[:, perm]
    mask = m.block_mask_build(pos)
    m.rebuild(mask, torch.argsort(pos[0] * Y + pos[1]))
    want = {key: getattr(m, key).clone() for key in INDEX_KEYS}
    for key in INDEX_KEYS[1:]:
        getattr(m, key).fill_(-7)
    m._pattern_scratch()  # first use derives the buffers from `blocks` on the device
    for key in INDEX_KEYS:
        assert torch.equal(getattr(m, key), want[key]), key
    cell_slot, _ = m._pattern_scratch()
    assert int((cell_slot >= 0).sum()) == n_blocks
    assert m.pattern_status() == 0
    # a duplicated position is flagged
    if n_blocks > 1:
        m.blocks[2:4] = m.blocks[0:2]
        m._rebuild_indices_device()
        assert m.pattern_status() & 1


@pytest.mark.parametrize("n,k", [(4096, 1024), (26214, 2621), (1000, 1), (1000, 1000), (77, 13)])
def test_select_lowest_is_the_exact_k_smallest(n, k):
    g = torch.Generator().manual_seed(n + k)
    stat = torch.rand(n, generator=g).cuda()
    stat[::7] = stat[3]  # many ties, some of them at the threshold for one of the cases
    got = native.select_lowest(stat, k).long()
    assert got.unique().numel() == k
    want_values = torch.sort(stat)[0][:k]
    assert torch.equal(torch.sort(stat[got])[0], want_values)
    # ties at the threshold are taken in index order
    thr = want_values[-1]
    ties_taken = got[stat[got] == thr]
    all_ties = (stat == thr).nonzero().flatten()
    assert torch.equal(torch.sort(ties_taken)[0], all_ties[: ties_taken.numel()])
    # negative values and zeros order correctly
    signed = torch.tensor([0.5, -1.0, 0.0, -0.25, 3.0, -7.5], device="cuda")
    assert sorted(native.select_lowest(signed, 3).tolist()) == [1, 3, 5]


def test_sample_free_positions_distinct_free_reproducible_and_uniform():
    np.random.seed(3)
    m = BlockSparseMatrix.zeros((1024, 2048), n_blocks=512, device="cuda")  # 32 x 64 cells, 1536 empty
    occupied = m.block_mask_build(None).reshape(-1)
    a = m.sample_free_positions(300, seed=11).long()
    assert a.unique().numel() == 300 and not occupied[a].any()
    assert torch.equal(a, m.sample_free_positions(300, seed=11).long())
    assert not torch.equal(a, m.sample_free_positions(300, seed=12).long())
    everything = m.sample_free_positions(1536, seed=5).long()  # k = all empty cells: a permutation of them
    assert torch.equal(torch.sort(everything)[0], (~occupied).nonzero().flatten())
    # every empty cell is drawn about equally often over many seeds (k / free = 1/4 each time)
    counts = torch.zeros(32 * 64, device="cuda")
    for seed in range(400):
        counts[m.sample_free_positions(384, seed=1000 + seed).long()] += 1
    free_counts = counts[~occupied]
    assert counts[occupied].sum() == 0
    assert abs(float(free_counts.mean()) - 100.0) < 1e-3
    assert float(free_counts.std()) < 12.0  # binomial(400, 1/4): sigma = 8.7
    assert m.pattern_status() == 0


@pytest.mark.parametrize("distribution", ["uniform", "gaussian"])
def test_sparse_optimizer_step_on_the_device(distribution):
    np.random.seed(5)
    torch.manual_seed(5)
    lin = BlockSparseLinear(512, 256, bias=True, density=0.25)
    w = lin.weight
    nnz = w.blocks.shape[0] // 2
    adam = torch.optim.Adam(lin.parameters(), lr=1e-3)
    so = SparseOptimizer(SparseOptimizer.sparse_objects(lin), lr=0.25, new_coefficients_distribution=distribution, seed=9)
    so.attach_optimizer(adam)
    x = torch.randn(64, 512, device="cuda")
    lin(x).square().mean().backward()
    adam.step()
    norms = w.block_norm().clone()
    data_before = w.data.detach().clone()
    mask_before = w.block_mask_build(None).clone()
    k = int(0.25 * nnz)
    lowest = set(torch.sort(norms)[1][:k].tolist())
    so.step()
    assert w.pattern_status() == 0
    mask_after = w.block_mask_build(None)
    assert int(mask_after.sum()) == nnz  # block count is preserved (reference test_sparse_optimizer.py:41-55)
    assert int((mask_before != mask_after).sum()) == 2 * k
    changed = (w.data.detach().view(nnz, -1) != data_before.view(nnz, -1)).any(1).nonzero().flatten().tolist()
    assert set(changed) == lowest  # exactly the k weakest slots were recycled
    moved = torch.tensor(sorted(lowest), device="cuda")
    for key in ("exp_avg", "exp_avg_sq"):
        state = adam.state[w.data][key].view(nnz, -1)
        assert float(state[moved].abs().sum()) == 0.0
        kept = torch.ones(nnz, dtype=torch.bool, device="cuda")
        kept[moved] = False
        assert float(state[kept].abs().sum()) > 0.0
    # host-side re-derivation of the buffers from the moved `blocks` agrees bit for bit
    want = w.build_indices(mask_after, torch.argsort(w.build_coo_block_index().long()[0] * w.blocks_count()[1]
                                                     + w.build_coo_block_index().long()[1]))
    for got, ref in zip((w.blocks, w.cols_a, w.row_start_ends_a, w.rows_b, w.col_start_ends_b), want):
        assert torch.equal(got, ref)
    y = lin(x)  # fresh plans and images of the new pattern
    assert torch.allclose(y, x @ w.to_dense().t() + lin.bias, atol=1e-4)
    assert_device_healthy()


def test_same_seed_gives_the_same_pattern_on_every_replica():
    """What data-parallel ranks rely on: two replicas with identical state and seed stay identical, step after
    step, without exchanging anything."""
    replicas = []
    for _ in range(2):
        np.random.seed(6)
        torch.manual_seed(6)
        m = BlockSparseMatrix.randn((512, 768), n_blocks=96, device="cuda")
        replicas.append((m, SparseOptimizer([m], lr=0.2, new_coefficients_distribution="gaussian", seed=31)))
    for _ in range(3):
        for m, so in replicas:
            so.step()
        a, b = replicas[0][0], replicas[1][0]
        for key in INDEX_KEYS:
            assert torch.equal(getattr(a, key), getattr(b, key)), key
        assert torch.equal(a.data, b.data)
    other = SparseOptimizer([replicas[0][0]], lr=0.2, seed=32)
    other.step()
    assert not torch.equal(replicas[0][0].blocks, replicas[1][0].blocks)


def test_strategy_on_larger_blocks():
    np.random.seed(7)
    torch.manual_seed(7)
    m = BlockSparseMatrix.randn((512, 512), n_blocks=20, block_shape=(64, 64), device="cuda")
    recycled = MagnitudeSparseOptimizerStrategy(0.3, "gaussian", 0.1, seed=2).run(m)
    assert recycled.slots.numel() == 6 and int(m.block_mask_build(None).sum()) == 20
    a = torch.randn(40, 512, device="cuda")
    assert torch.allclose(m.reverse_matmul(a, transpose=True), a @ m.to_dense().t(), atol=1e-3)
    assert m.pattern_status() == 0
