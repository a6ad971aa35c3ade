"""GPU parity of the three contractions, called through the C-ABI (native.* -> ctypes ->
libbsmm_b200.so), against the CPU oracle on identical seeded inputs.

Tolerances: relative Frobenius error <= 1e-5 for the fp32-class modes ("fp32" CUDA-core FMA, "tf32x3"
tensor-core 3-pass and "bf16x3", which splits into bf16 pairs in forward and dgrad), bookkeeping bit-exact.  Shapes follow the reference's own tests
(pytorch_block_sparse/tests/test_matmul.py:141-244, test_matmul_back.py:205-238, test_replace.py:140-161).
"""
import numpy as np
import pytest
import torch

from oracle import block_sparse_oracle as orc
from pytorch_block_sparse_b200 import native

from oracle import ref_cuda

from .gpu_util import TOL, assert_device_healthy, check, host, make_matrix, randn

pytestmark = pytest.mark.gpu

PRECISIONS = ["fp32", "tf32x3", "bf16x3"]

# (leading dims of a, sizes[1], sizes[2], blocks) -- reference tests/test_matmul.py:141-227
REFERENCE_CASES = [
    ((32,), 32, 32, [(0, 0)]),
    ((32,), 64, 32, [(0, 0)]),
    ((64,), 32, 32, [(0, 0)]),
    ((128,), 32, 32, [(0, 0)]),
    ((128,), 64, 32, [(0, 0)]),
    ((128,), 64, 32, [(0, 1)]),
    ((128,), 64, 32, [(0, 0), (0, 1)]),
    ((32,), 32, 64, [(0, 0)]),
    ((32,), 32, 64, [(1, 0)]),
    ((32,), 32, 64, [(0, 0), (1, 0)]),
    ((64, 32), 32, 64, [(0, 0), (1, 0)]),
    ((64, 128, 32), 128, 256, [(0, 0)]),
    ((64, 128, 32), 128, 256, [(0, 0), (1, 0)]),
    ((32,), 64, 64, [(0, 0), (1, 0), (0, 1)]),
    ((32,), 64, 128, [(0, 0), (1, 0), (0, 1), (2, 0)]),
    ((1,), 32, 32, [(0, 0)]),
]


def run_dsd(m, a, transpose, precision, bias=None):
    out = m.reverse_matmul(a.cuda(), transpose=transpose, bias=None if bias is None else bias.cuda(), precision=precision)
    torch.cuda.synchronize()
    return out


def oracle_dsd(m, a, transpose, bias=None):
    shape, blocks, data = host(m)
    if transpose:
        return orc.forward(a.numpy(), shape, blocks, data, None if bias is None else bias.numpy())
    return orc.dgrad(a.numpy(), shape, blocks, data)


@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("transpose", [True, False])
def test_dsd_reference_shapes(precision, transpose):
    for i, (lead, s1, s2, blocks) in enumerate(REFERENCE_CASES):
        # the reference builds the matrix as (sizes[2], sizes[1]) and multiplies a[.., s1] by its
        # transpose, or a[.., s2] by the matrix itself (tests/test_matmul.py:29-46)
        m = make_matrix((s2, s1), blocks=blocks, seed=i, std=1.0, positive=True)
        k, n = (s1, s2) if transpose else (s2, s1)
        a = randn(lead + (k,), seed=100 + i, positive=True)
        got = run_dsd(m, a, transpose, precision)
        assert got.shape == lead + (n,)
        check(got, oracle_dsd(m, a, transpose), precision, f"case {i} transpose={transpose}")
    assert_device_healthy()


@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("tokens", [1, 31, 33, 127, 129, 200, 517])
def test_dsd_ragged_token_counts(precision, tokens):
    m = make_matrix((96, 160), n_blocks=9, seed=tokens)
    x = randn((tokens, 160), seed=1)
    dy = randn((tokens, 96), seed=2)
    check(run_dsd(m, x, True, precision), oracle_dsd(m, x, True), precision, "fwd")
    check(run_dsd(m, dy, False, precision), oracle_dsd(m, dy, False), precision, "dgrad")
    assert_device_healthy()


@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("density", [0.05, 0.25, 0.5, 1.0])
def test_dsd_random_patterns_with_bias_and_empty_rows(precision, density):
    shape = (512, 384)  # 16 x 12 blocks: two row-groups of 8; low density leaves empty block-rows
    n_blocks = max(1, int(density * 16 * 12))
    m = make_matrix(shape, n_blocks=n_blocks, seed=int(density * 100))
    x = randn((300, 384), seed=3)
    bias = randn((512,), seed=4) * 0.02
    got = run_dsd(m, x, True, precision, bias)
    want = oracle_dsd(m, x, True, bias)
    check(got, want, precision, "fwd+bias")
    # block-rows without any block are exactly the bias
    counts = np.diff(m.row_start_ends_a.cpu().numpy())
    for r in np.nonzero(counts == 0)[0]:
        sl = got[:, r * 32:(r + 1) * 32].cpu()
        assert torch.equal(sl, bias[r * 32:(r + 1) * 32].expand_as(sl))
    dy = randn((300, 512), seed=5)
    check(run_dsd(m, dy, False, precision), oracle_dsd(m, dy, False), precision, "dgrad")
    assert_device_healthy()


@pytest.mark.parametrize("precision", PRECISIONS)
def test_dsd_reference_output_layout(precision):
    """The [n, m] column-major buffer the reference's native entry point fills (block_sparse.py:516,578)."""
    m = make_matrix((128, 96), n_blocks=7, seed=7)
    x = randn((77, 96), seed=8).cuda()
    packed = m.packed_weights(precision)
    out = native.dsd_matmul(x, m._plan(True), packed, n_out=128, transpose=True, out_colmajor=True)
    torch.cuda.synchronize()
    assert out.shape == (128, 77)
    check(out.t(), oracle_dsd(m, x.cpu(), True), precision)
    assert_device_healthy()


@pytest.mark.parametrize("precision", PRECISIONS)
def test_golden_small_case_of_the_reference(precision, golden):
    g = golden("linear")
    shape = tuple(int(v) for v in g["small/shape"])
    coo = g["small/blocks"].reshape(-1, 2)
    m = make_matrix(shape, blocks=[(int(r), int(c)) for c, r in coo], seed=0)
    assert np.array_equal(m.blocks.cpu().numpy(), g["small/blocks"])
    with torch.no_grad():
        m.data.copy_(torch.from_numpy(g["small/data"]))
    x, dy, bias = (torch.from_numpy(g[f"small/{k}"]) for k in ("x", "dy", "bias"))
    y = run_dsd(m, x, True, precision, bias)
    dx = run_dsd(m, dy, False, precision)
    dw = m.matmul_with_output_sparse_support(dy.cuda(), x.cuda(), precision=precision)
    torch.cuda.synchronize()
    # fixtures hold the reference's own fp32 CPU results: allow its rounding on top of ours
    for got, key in ((y, "y"), (dx, "dx"), (dw, "dw")):
        want = g[f"small/{key}"]
        assert orc.rel_fro(got.float().cpu().numpy().reshape(want.shape), want) < 1e-5, key
    assert_device_healthy()


def test_config1_sampled_golden(golden):
    """Benchmark configuration 1 (X [256,1024], W 256x1024 density 0.5): inputs re-derived from the seed,
    outputs compared with the strided sample recorded from the reference."""
    import hashlib

    g = golden("linear")
    np.random.seed(1)
    torch.manual_seed(1)
    from pytorch_block_sparse_b200 import BlockSparseMatrix

    m = BlockSparseMatrix.zeros((256, 1024), n_blocks=128, device="cpu")
    with torch.no_grad():
        m.data.normal_(0, 0.02)
    x = torch.randn(256, 1024)
    dy = torch.randn(256, 256)
    bias = torch.randn(256) * 0.02
    h = hashlib.sha256()
    for a in (m.blocks.numpy(), m.data.detach().numpy(), x.numpy(), dy.numpy(), bias.numpy()):
        h.update(np.ascontiguousarray(a).tobytes())
    if h.hexdigest() != str(g["c1/input_sha256"]):
        pytest.skip("torch CPU RNG stream differs from the one the fixture was recorded with")
    m = m.cuda()
    stride = int(g["c1/stride"])
    for precision in PRECISIONS:
        y = m.reverse_matmul(x.cuda(), transpose=True, bias=bias.cuda(), precision=precision)
        dx = m.reverse_matmul(dy.cuda(), transpose=False, precision=precision)
        dw = m.matmul_with_output_sparse_support(dy.cuda(), x.cuda(), precision=precision)
        for got, key in ((y, "y"), (dx, "dx"), (dw, "dw")):
            want = g[f"c1/{key}"]
            assert orc.rel_fro(got.float().cpu().numpy().reshape(-1)[::stride], want) < 1e-5, (precision, key)
    assert_device_healthy()


@pytest.mark.parametrize("precision", PRECISIONS)
@pytest.mark.parametrize("a_rowmajor,b_rowmajor", [(True, True), (True, False), (False, True), (False, False)])
def test_sddmm_orientations(precision, a_rowmajor, b_rowmajor):
    # reference tests/test_matmul_back.py:226-237: either orientation of both operands, no copies
    m = make_matrix((128, 96), n_blocks=6, seed=3)
    for tokens in (1, 40, 256):
        dy = randn((tokens, 128), seed=9)
        x = randn((tokens, 96), seed=10)
        a = dy.cuda() if a_rowmajor else dy.t().contiguous().cuda().t()
        b = x.cuda() if b_rowmajor else x.t().contiguous().cuda().t()
        got = m.matmul_with_output_sparse_support(a, b, precision=precision)
        torch.cuda.synchronize()
        want = orc.wgrad(dy.numpy(), x.numpy(), tuple(m.shape), m.blocks.cpu().numpy())
        check(got, want, precision, f"tokens={tokens}")
    assert_device_healthy()


@pytest.mark.parametrize("precision", PRECISIONS)
def test_sddmm_split_tokens_and_leading_dims(precision):
    m = make_matrix((64, 64), n_blocks=2, seed=4)  # few blocks, many tokens: the token axis is split
    dy = randn((4, 1000, 64), seed=11)
    x = randn((4, 1000, 64), seed=12)
    got = m.matmul_with_output_sparse_support(dy.cuda(), x.cuda(), precision=precision)
    torch.cuda.synchronize()
    want = orc.wgrad(dy.numpy(), x.numpy(), (64, 64), m.blocks.cpu().numpy())
    check(got, want, precision)
    assert_device_healthy()


@pytest.mark.parametrize("precision", PRECISIONS)
def test_kernels_follow_slots_after_block_replace(precision):
    # reference tests/test_replace.py:140-161
    m = make_matrix((128, 64), blocks=[(0, 0), (1, 0), (2, 0), (0, 1)], seed=5, std=1.0, positive=True)
    m.block_replace(torch.tensor([(3, 1, 0), (2, 1, 2), (1, 1, 1)]))
    assert m.cols_a.cpu().tolist() == [[1, 1], [0, 3], [1, 2], [1, 0]]
    a = randn((1, 64), seed=13, positive=True)
    check(run_dsd(m, a, True, precision), oracle_dsd(m, a, True), precision, "fwd")
    b = randn((1, 128), seed=14, positive=True)
    check(run_dsd(m, b, False, precision), oracle_dsd(m, b, False), precision, "dgrad")
    got = m.matmul_with_output_sparse_support(b.cuda(), a.cuda(), precision=precision)
    want = orc.wgrad(b.numpy(), a.numpy(), (128, 64), m.blocks.cpu().numpy())
    check(got, want, precision, "wgrad")
    assert_device_healthy()


def test_pack_statistic_matches_block_norm():
    m = make_matrix((256, 256), n_blocks=20, seed=6, std=1.0)
    want = orc.block_norm(m.data.detach().cpu().numpy()) ** 2
    for precision in PRECISIONS:
        got = m.packed_weights(precision).block_sumsq.cpu().numpy()
        assert np.allclose(got, want, rtol=1e-5)


@pytest.mark.parametrize("group", [4, 5, 6, 8])
def test_plan_is_the_group_merge_of_the_csr(group):
    m = make_matrix((512, 2048), n_blocks=880, seed=8)  # rows of ~55 of 64 blocks: promotions inside a row
    plan = m._plan(True)
    raw = plan.buffer(group)
    torch.cuda.synchronize()
    raw = raw.cpu().numpy()
    groups = (16 + group - 1) // group
    off = raw[: (groups + 1) * 4].view(np.int32)
    slabs = raw[(groups + 1) * 4: (2 * groups + 1) * 4].view(np.int32)
    ent_off = ((2 * groups + 1) * 4 + 15) // 16 * 16
    ent = raw[ent_off: ent_off + plan.nnz * 16].view(np.int32).reshape(-1, 4)
    ptr = m.row_start_ends_a.cpu().numpy()
    idx = m.cols_a.cpu().numpy()
    assert (np.diff(ptr) > 48).any()
    for g in range(groups):
        rows = range(g * group, min(16, g * group + group))
        want = sorted((int(idx[e, 0]), r - g * group, int(idx[e, 1])) for r in rows for e in range(ptr[r], ptr[r + 1]))
        assert off[g] == ptr[g * group]
        got = ent[off[g]: off[g + 1]]
        assert [(int(c), int(r), int(s)) for c, s, r, _ in got] == want
        assert slabs[g] == len({c for c, _, _ in want})
        seen = {}
        for i, (c, s, r, flags) in enumerate(got):
            first = i == 0 or got[i - 1][0] != c
            last = i == len(got) - 1 or got[i + 1][0] != c
            seen[r] = seen.get(r, 0) + 1
            row_len = ptr[g * group + r + 1] - ptr[g * group + r]
            drain = seen[r] % 48 == 0 or seen[r] == row_len  # promotion every 48 blocks of a row and at its end
            row_end = seen[r] == row_len                       # bit 6: the promotion after it completes the row
            # MMA warp of a row: row mod 4.  Bit 3: last block of its slab for its warp; on the slab's last
            # block, bits 4-5: warps without a block in the slab
            slab = [int(q[2]) for q in got if q[0] == c]
            warp_last = not any(q > r and q % 4 == r % 4 for q in slab)
            idle = 4 - len({q % 4 for q in slab})
            assert flags == ((1 if first else 0) | (2 if last else 0) | (4 if drain else 0) | (8 if warp_last else 0)
                             | ((idle << 4) if last else 0) | (64 if row_end else 0))


@pytest.mark.parametrize("group", ["4", "6", "8"])
def test_bf16_mode(group, monkeypatch):
    """Opt-in 'bf16' precision: operands rounded to bf16 inside the kernels (tensors stay fp32), fp32
    accumulation; bound 1e-2 relative Frobenius on all three contractions."""
    monkeypatch.setenv("BSMM_PLAN_GROUP", group)
    m = make_matrix((416, 352), n_blocks=70, seed=41)
    x, dy, bias = randn((2100, 352), seed=42), randn((2100, 416), seed=43), randn((416,), seed=44)
    check(run_dsd(m, x, True, "bf16", bias), oracle_dsd(m, x, True, bias), "bf16", "fwd")
    check(run_dsd(m, dy, False, "bf16"), oracle_dsd(m, dy, False), "bf16", "dgrad")
    got = m.matmul_with_output_sparse_support(dy.cuda(), x.cuda(), precision="bf16")
    torch.cuda.synchronize()
    want = orc.wgrad(dy.numpy(), x.numpy(), tuple(m.shape), m.blocks.cpu().numpy())
    check(got, want, "bf16", "wgrad")
    assert orc.rel_fro(got.float().cpu().numpy().reshape(want.shape), want) > 1e-4  # really bf16 operands
    assert_device_healthy()


def test_single_pass_tf32_wgrad():
    """Opt-in 'tf32' precision of the weight gradient: bound 2e-3 relative Frobenius; 2100 tokens cross two
    promotion points and leave a ragged last step."""
    m = make_matrix((256, 384), n_blocks=40, seed=31)
    dy, x = randn((2100, 256), seed=32), randn((2100, 384), seed=33)
    got = m.matmul_with_output_sparse_support(dy.cuda(), x.cuda(), precision="tf32")
    torch.cuda.synchronize()
    want = orc.wgrad(dy.numpy(), x.numpy(), tuple(m.shape), m.blocks.cpu().numpy())
    check(got, want, "tf32", "wgrad")
    assert orc.rel_fro(got.float().cpu().numpy().reshape(want.shape), want) > 1e-6  # really the single pass
    assert_device_healthy()


@pytest.mark.parametrize("group", ["4", "5", "6", "8"])
def test_dsd_every_tile_width(group, monkeypatch):
    monkeypatch.setenv("BSMM_PLAN_GROUP", group)
    m = make_matrix((416, 352), n_blocks=70, seed=21)  # 13 x 11 blocks: ragged last group for every width
    x = randn((333, 352), seed=22)
    dy = randn((333, 416), seed=23)
    bias = randn((416,), seed=24)
    check(run_dsd(m, x, True, "tf32x3", bias), oracle_dsd(m, x, True, bias), "tf32x3", "fwd")
    check(run_dsd(m, dy, False, "tf32x3"), oracle_dsd(m, dy, False), "tf32x3", "dgrad")
    assert_device_healthy()


@pytest.mark.parametrize("precision", PRECISIONS)
def test_dsd_long_rows_stay_within_the_error_bound(precision):
    """96 blocks per output row (K = 4096 at density 0.75): the tensor-core accumulator alone would drift
    past 1e-5 here; the periodic promotion to an fp32 master tile keeps the error at the CUDA-core level."""
    m = make_matrix((256, 4096), n_blocks=int(0.75 * 8 * 128), seed=31)
    x = randn((256, 4096), seed=32)
    bound = 6e-6 if precision == "bf16x3" else 4e-6  # (the bf16 pair splitting alone leaves 4.6e-6)
    err = check(run_dsd(m, x, True, precision), oracle_dsd(m, x, True), precision, "fwd")
    assert err < bound, err
    m2 = make_matrix((4096, 256), n_blocks=int(0.75 * 8 * 128), seed=33)
    dy = randn((256, 4096), seed=34)
    err = check(run_dsd(m2, dy, False, precision), oracle_dsd(m2, dy, False), precision, "dgrad")
    assert err < bound, err
    assert_device_healthy()


@pytest.mark.parametrize("transpose", [True, False])
def test_single_pass_tf32_mode(transpose):
    """Opt-in 'tf32' precision: one tensor-core pass on operands rounded to tf32 (the accuracy class of
    cuBLAS with allow_tf32); bound 2e-3 relative Frobenius."""
    m = make_matrix((512, 384), n_blocks=60, seed=41)
    a = randn((300, 384 if transpose else 512), seed=42)
    got = run_dsd(m, a, transpose, "tf32")
    err = orc.rel_fro(got.float().cpu().numpy(), oracle_dsd(m, a, transpose))
    assert 1e-6 < err < 2e-3, err
    assert_device_healthy()


@pytest.mark.parametrize("precision", PRECISIONS)
def test_sddmm_long_token_axis_and_statistic(precision):
    """Many tokens (several promotion segments and token ranges) with rows of more than 16 blocks
    (several items per row); also the fused per-slot sum of squares."""
    m = make_matrix((128, 1024), n_blocks=90, seed=51)
    dy = randn((5000, 128), seed=52)
    x = randn((5000, 1024), seed=53)
    out = torch.empty_like(m.data)
    sumsq = torch.empty(90, device="cuda")
    native.sddmm(dy.cuda(), True, x.cuda(), True, m.blocks, out.detach(), precision=precision, block_sumsq=sumsq,
                 plan=m._sddmm_plan())
    torch.cuda.synchronize()
    want = orc.wgrad(dy.numpy(), x.numpy(), (128, 1024), m.blocks.cpu().numpy())
    err = check(out, want, precision)
    assert err < (6e-6 if precision == "bf16x3" else 4e-6), err  # (the bf16 pair splitting alone leaves 4.6e-6)
    assert np.allclose(sumsq.cpu().numpy(), orc.block_norm(want) ** 2, rtol=1e-4)
    assert_device_healthy()


@pytest.mark.parametrize("precision", ["tf32x3", "bf16x3", "tf32", "bf16"])
@pytest.mark.parametrize("a_rowmajor,b_rowmajor", [(False, True), (True, False), (False, False)])
def test_sddmm_feature_major_operands_stay_on_the_tensor_cores(precision, a_rowmajor, b_rowmajor):
    """The reference serves all four contiguity combinations of (dY, X) with one kernel
    (native/block_sparse_cutlass_kernel_back.cu:145-157).  Here the tensor-core kernel reads a feature-major
    operand through a [features, tokens] tensor map; the test checks values against the oracle, that the library
    asks for the tensor-core kernel's workspace (i.e. does not drop to the CUDA-core kernel), and -- on a shape
    large enough to tell -- that it is as fast as the token-major case."""
    m = make_matrix((128, 1024), n_blocks=90, seed=61)
    tokens = 3000
    dy = randn((tokens, 128), seed=62)
    x = randn((tokens, 1024), seed=63)
    a = dy.cuda() if a_rowmajor else dy.t().contiguous().cuda().t()
    b = x.cuda() if b_rowmajor else x.t().contiguous().cuda().t()
    flags = native.PRECISIONS[precision] | (0 if a_rowmajor else native.SDDMM_A_COLMAJOR) | (0 if b_rowmajor else native.SDDMM_B_COLMAJOR)
    assert native.load().bsmm_sddmm_workspace_bytes(128, 1024, tokens, 90, flags) > 0
    got = m.matmul_with_output_sparse_support(a, b, precision=precision)
    torch.cuda.synchronize()
    want = orc.wgrad(dy.numpy(), x.numpy(), (128, 1024), m.blocks.cpu().numpy())
    check(got, want, precision)
    # a token count that is not a multiple of 4 cannot be described by a feature-major tensor map: CUDA-core kernel
    got = m.matmul_with_output_sparse_support(a[:2999], b[:2999], precision=precision)
    check(got, orc.wgrad(dy.numpy()[:2999], x.numpy()[:2999], (128, 1024), m.blocks.cpu().numpy()), precision)
    assert_device_healthy()


def test_sddmm_feature_major_speed_class():
    big = make_matrix((2048, 2048), n_blocks=1024, seed=64)
    g = torch.Generator().manual_seed(65)
    dy_t = torch.randn(2048, 8192, generator=g).cuda()   # feature-major storage
    x_t = torch.randn(2048, 8192, generator=g).cuda()
    dy_c, x_c = dy_t.t().contiguous(), x_t.t().contiguous()

    def timed(a, b):
        for _ in range(2):
            out = big.matmul_with_output_sparse_support(a, b)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            out = big.matmul_with_output_sparse_support(a, b)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 5, out

    t_tm, ref = timed(dy_c, x_c)
    t_fm, got = timed(dy_t.t(), x_t.t())
    assert float((got.double() - ref.double()).norm() / ref.double().norm()) < 1e-5
    assert t_fm < 1.5 * t_tm, (t_fm, t_tm)   # the CUDA-core kernel is about four times slower
    assert_device_healthy()


def test_missing_cuda_tensor_is_rejected():
    m = make_matrix((64, 64), n_blocks=2, seed=9)
    with pytest.raises(native.NativeError):
        m.reverse_matmul(torch.zeros(4, 64), transpose=True)


def _rel_fro_gpu(got, want):
    return float((got.double() - want.double()).norm() / want.double().norm())


def _full_size_case(shape, n_blocks, tokens, precision, seed, check_reference_kernels=False, golden_pattern=None):
    """One benchmark configuration at its full size, checked three ways.  The numpy oracle is too slow for the
    whole problem, so the tensor-core kernels are compared (a) with the exact-fp32 CUDA-core kernels on the
    device, which the small cases pin to the oracle, (b) with the oracle on a sample of 96 token rows / 8
    blocks, (c) through properties that do not depend on the size: scaling an input by 4 scales the result by
    exactly 4, and permuting the token rows permutes forward rows / leaves the weight gradient within rounding,
    and optionally (d) with the reference's own CUDA kernels where they were built."""
    tol = TOL[precision]
    n_out, n_in = shape
    m = make_matrix(shape, n_blocks=n_blocks, seed=seed)
    if golden_pattern is not None:  # the pattern is the one the reference draws from this seed
        for key in ("blocks", "cols_a", "row_start_ends_a", "rows_b", "col_start_ends_b"):
            assert np.array_equal(getattr(m, key).cpu().numpy(), golden_pattern[key]), key
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(tokens, n_in, generator=g).cuda()
    dy = torch.randn(tokens, n_out, generator=g).cuda()
    bias = (torch.randn(n_out, generator=g) * 0.02).cuda()

    y = m.reverse_matmul(x, transpose=True, bias=bias, precision=precision)
    dx = m.reverse_matmul(dy, transpose=False, precision=precision)
    dw = m.matmul_with_output_sparse_support(dy, x, precision=precision)
    y_ref = m.reverse_matmul(x, transpose=True, bias=bias, precision="fp32")
    dx_ref = m.reverse_matmul(dy, transpose=False, precision="fp32")
    dw_ref = m.matmul_with_output_sparse_support(dy, x, precision="fp32")
    torch.cuda.synchronize()
    for got, want, what in ((y, y_ref, "fwd"), (dx, dx_ref, "dgrad"), (dw, dw_ref, "wgrad")):
        assert torch.isfinite(got).all(), what
        err = _rel_fro_gpu(got, want)
        assert err <= tol, f"{what}: {err:.3e}"
    del y_ref, dx_ref

    # (b) oracle on a sample: 96 token rows spread over the range; 8 blocks of the weight gradient
    shp, blocks, data = host(m)
    rows = torch.arange(0, tokens, max(1, tokens // 96))[:96]
    want = orc.forward(x[rows].cpu().numpy(), shp, blocks, data, bias.cpu().numpy())
    assert orc.rel_fro(y[rows].cpu().numpy(), want) <= tol
    want = orc.dgrad(dy[rows].cpu().numpy(), shp, blocks, data)
    assert orc.rel_fro(dx[rows].cpu().numpy(), want) <= tol
    dw_blocks = dw.view(-1, 32, 32)
    coo = blocks.reshape(-1, 2)
    for s in range(0, n_blocks, max(1, n_blocks // 8)):
        c, r = int(coo[s, 0]), int(coo[s, 1])
        want = (x[:, c * 32:(c + 1) * 32].double().t() @ dy[:, r * 32:(r + 1) * 32].double()).cpu().numpy()
        assert orc.rel_fro(dw_blocks[s].cpu().numpy(), want) <= tol, s

    # (d) the reference's own CUDA kernels (int indexing: tokens x features below 2^31)
    if check_reference_kernels and ref_cuda.available() and tokens * max(n_out, n_in) < 2 ** 31 and tokens % 32 == 0:
        torch.cuda.synchronize()
        ref_y = ref_cuda.reverse_matmul(m, x, True) + bias
        ref_dx = ref_cuda.reverse_matmul(m, dy, False)
        ref_dw = ref_cuda.sddmm(m, dy, x)
        torch.cuda.synchronize()  # the reference launches on the legacy default stream
        assert _rel_fro_gpu(y, ref_y) <= tol and _rel_fro_gpu(dx, ref_dx) <= tol and _rel_fro_gpu(dw, ref_dw) <= tol
        del ref_y, ref_dx, ref_dw
    del dx, dw_ref

    # (c) size-independent properties
    y0 = m.reverse_matmul(x, transpose=True, precision=precision)
    y4 = m.reverse_matmul(x * 4.0, transpose=True, precision=precision)
    assert torch.equal(y4, y0 * 4.0)  # powers of two commute with every rounding step
    del y4
    perm = torch.randperm(tokens, generator=g).cuda()
    yp = m.reverse_matmul(x[perm].contiguous(), transpose=True, precision=precision)
    assert torch.equal(yp, y0[perm])  # a token's result does not depend on its position
    del yp, y0
    dwp = m.matmul_with_output_sparse_support(dy[perm].contiguous(), x[perm].contiguous(), precision=precision)
    assert _rel_fro_gpu(dwp, dw) <= tol  # a sum over tokens in another order
    assert_device_healthy()


def test_sddmm_repeated_launches_agree_bit_for_bit():
    """Regression: the X split warps used to release a slab right after issuing their loads; now and then the TMA
    refill overtook loads still queued, and a few rows of one block came from the next unit (a few per cent off,
    in about one launch in 25 with feature-major X, whose 16-byte loads leave the warps earliest).  Every storage
    order and tensor-core precision, many launches: all results of one configuration are identical."""
    m = make_matrix((832, 992), n_blocks=26 * 31, seed=517)  # rows of 31 blocks: items of 8, 8, 8 and 7
    dy = randn((2400, 832), seed=518).cuda()
    x = randn((2400, 992), seed=519).cuda()
    dy_fm, x_fm = dy.t().contiguous().t(), x.t().contiguous().t()
    for precision in ("tf32x3", "bf16x3", "tf32", "bf16"):
        want = m.matmul_with_output_sparse_support(dy, x, precision=precision).clone()
        for a, b in ((dy, x_fm), (dy_fm, x_fm), (dy_fm, x), (dy, x)):
            first = m.matmul_with_output_sparse_support(a, b, precision=precision).clone()
            assert _rel_fro_gpu(first, want) <= TOL[precision], precision
            for _ in range(60):
                assert torch.equal(m.matmul_with_output_sparse_support(a, b, precision=precision), first), precision
    assert_device_healthy()


@pytest.mark.parametrize("precision", ["tf32x3", "bf16x3", "tf32", "bf16"])
def test_full_size_config3(precision):
    """Benchmark configuration 3 at density 0.25 in full (4096 x 4096, 4096 blocks, 16384 tokens): every
    persistent CTA walks ~28 tiles."""
    _full_size_case((4096, 4096), 4096, 16384, precision, seed=51, check_reference_kernels=precision == "tf32x3")


@pytest.mark.parametrize("density", [0.1, 0.5, 0.75])
def test_full_size_config3_density_sweep(density):
    """The other densities of benchmark configuration 3 in the default precision: rows of 13 (d = 0.1) to 96
    (d = 0.75) blocks, i.e. no promotion at all up to three promotions per row and tile."""
    _full_size_case((4096, 4096), int(density * 4096 * 4096 / 1024), 16384, "tf32x3", seed=61 + int(density * 100),
                    check_reference_kernels=True)


@pytest.mark.parametrize("shape", [(3072, 768), (768, 3072)])
def test_full_size_config2(shape, golden):
    """Benchmark configuration 2: the two RoBERTa-base FFN layers (768 -> 3072 and 3072 -> 768, density 0.5) on
    4096 tokens.  The 768 x 3072 pattern is the one the reference itself draws from numpy seed 2 (committed
    fixture), so the whole chain pattern -> indices -> plans -> kernels is pinned to the reference here."""
    pattern = None
    if shape == (768, 3072):
        idx = golden("indices")
        name = "random_s2_768x3072_n1152"
        pattern = {k: idx[name + "/" + k] for k in ("blocks", "cols_a", "row_start_ends_a", "rows_b", "col_start_ends_b")}
    _full_size_case(shape, 1152, 4096, "tf32x3", seed=2, check_reference_kernels=True, golden_pattern=pattern)


def test_full_size_config5_shard():
    """One GPU's block-row shard of benchmark configuration 5 (32768 x 8192 at density 0.1 over 8 GPUs:
    4096 x 8192 per GPU) on its 65536 tokens: 512 token tiles, 8 token ranges in the weight gradient."""
    _full_size_case((4096, 8192), int(0.1 * 4096 * 8192 / 1024), 65536, "tf32x3", seed=71)


def test_bf16_tensors_in_memory():
    """'bf16' precision with bf16 activations and outputs in HBM (benchmark configuration 5 says "X bf16"): the kernels
    read bf16 boxes and write bf16 tiles, the weight gradient stays fp32.  Checked against the fp32 oracle on the
    bf16-rounded inputs (<= 1e-2), and against the same precision on fp32 copies of those inputs (same operand
    values, so only the output rounding differs)."""
    m = make_matrix((512, 1024), n_blocks=200, seed=91)
    x = randn((777, 1024), seed=92).bfloat16()
    dy = randn((777, 512), seed=93).bfloat16()
    bias = (randn((512,), seed=94) * 0.02)
    shape, blocks, data = host(m)
    y = m.reverse_matmul(x.cuda(), transpose=True, bias=bias.cuda(), precision="bf16")
    dx = m.reverse_matmul(dy.cuda(), transpose=False, precision="bf16")
    dw = m.matmul_with_output_sparse_support(dy.cuda(), x.cuda(), precision="bf16")
    torch.cuda.synchronize()
    assert y.dtype == torch.bfloat16 and dx.dtype == torch.bfloat16 and dw.dtype == torch.float32
    xf, dyf = x.float(), dy.float()
    check(y.float(), orc.forward(xf.numpy(), shape, blocks, data, bias.numpy()), "bf16", "fwd")
    check(dx.float(), orc.dgrad(dyf.numpy(), shape, blocks, data), "bf16", "dgrad")
    check(dw, orc.wgrad(dyf.numpy(), xf.numpy(), shape, blocks), "bf16", "wgrad")
    y32 = m.reverse_matmul(xf.cuda(), transpose=True, bias=bias.cuda(), precision="bf16")
    dw32 = m.matmul_with_output_sparse_support(dyf.cuda(), xf.cuda(), precision="bf16")
    assert float((y.float() - y32).norm() / y32.norm()) < 4e-3      # one bf16 rounding of the output
    assert float((dw - dw32).norm() / dw32.norm()) < 1e-5           # same operands, fp32 result
    # through the layer: bf16 in, bf16 out, fp32 weight gradient
    from pytorch_block_sparse_b200 import BlockSparseLinear
    native.set_default_precision("bf16")
    try:
        np.random.seed(95)
        lin = BlockSparseLinear(1024, 512, bias=True, density=0.4)
        xb = x.cuda().requires_grad_(True)
        out = lin(xb)
        out.backward(dy.cuda())
        assert out.dtype == torch.bfloat16 and xb.grad.dtype == torch.bfloat16
        assert lin.weight.data.grad.dtype == torch.float32 and lin.bias.grad.dtype == torch.float32
        dense = lin.weight.to_dense().detach()
        want = xf.cuda() @ dense.t() + lin.bias.detach()
        assert float((out.float() - want).norm() / want.norm()) < 1e-2
    finally:
        native.set_default_precision("tf32x3")
    assert_device_healthy()


def _shifted(t, elems=1):
    """A copy of ``t`` whose storage starts ``elems`` elements into a larger allocation: a misaligned view, as the
    parameters and buffers of an nn.DataParallel replica are (slices of one flat broadcast buffer)."""
    flat = torch.empty(t.numel() + elems, dtype=t.dtype, device=t.device)
    view = flat[elems:].view(t.shape)
    view.copy_(t)
    return view


@pytest.mark.parametrize("precision", PRECISIONS)
def test_misaligned_tensors_are_taken(precision):
    # index buffers, data, bias and operands on 4-byte boundaries give the results of the aligned call
    m = make_matrix((256, 192), n_blocks=17, seed=21)
    a, g = randn((70, 192), 5).cuda(), randn((70, 256), 6).cuda()
    bias = randn((256,), 7).cuda()
    want_y = m.reverse_matmul(a, transpose=True, bias=bias, precision=precision)
    want_dx = m.reverse_matmul(g, transpose=False, precision=precision)
    want_dw = m.matmul_with_output_sparse_support(g, a, precision=precision)

    prec = native.resolve_precision(precision)
    packed = native.pack_weights(_shifted(m.data.detach()), prec)
    plan_f = native.DsdPlan(_shifted(m.row_start_ends_a), _shifted(m.cols_a))
    plan_d = native.DsdPlan(_shifted(m.col_start_ends_b), _shifted(m.rows_b))
    y = native.dsd_matmul(_shifted(a), plan_f, packed, 256, True, bias=_shifted(bias))
    dx = native.dsd_matmul(_shifted(g), plan_d, packed, 192, False)
    plan_w = native.SddmmPlan(_shifted(m.row_start_ends_a), _shifted(m.cols_a))
    dw = torch.empty_like(m.data)
    native.sddmm(_shifted(g), True, _shifted(a), True, _shifted(m.blocks), dw, precision=prec, plan=plan_w)
    torch.cuda.synchronize()
    assert torch.equal(y, want_y) and torch.equal(dx, want_dx) and torch.equal(dw, want_dw)
    assert_device_healthy()


@pytest.mark.parametrize("group", ["4", "5", "6", "8"])
def test_dsd_groups_of_empty_rows_between_tiles(group, monkeypatch):
    # Whole groups of output block-rows without a block, in a launch where every CTA walks several tiles: a tile
    # without entries has no chunk of the plan to read, and the tile after it must still be decoded from its own.
    monkeypatch.setenv("BSMM_PLAN_GROUP", group)
    rows = [2, 11, 12, 12, 13, 15, 15, 17, 17, 19, 21, 21, 22, 25, 27, 30]
    cols = [2, 5, 1, 4, 5, 0, 8, 1, 7, 1, 3, 7, 1, 3, 2, 5]
    m = make_matrix((37 * 32, 9 * 32), blocks=list(zip(rows, cols)), seed=51)
    x = randn((9000, 9 * 32), seed=52)
    bias = randn((37 * 32,), seed=53)
    for precision in ("tf32x3", "tf32"):
        if (precision == "tf32x3" and group == "8") or (precision == "tf32" and group == "5"):
            continue  # 8-row tiles leave 3xTF32 no tensor memory, 5-row tiles exist for 3xTF32 only
        got = run_dsd(m, x, True, precision, bias)
        check(got, oracle_dsd(m, x, True, bias), precision, "fwd")
        empty = got[:, 4 * 32:8 * 32]  # block-rows 4..7 hold no block: bias exactly
        assert torch.equal(empty, bias[4 * 32:8 * 32].cuda().expand_as(empty))
    # the same pattern seen from the other side: dgrad of the transposed layout has the empty groups on its output
    mt = make_matrix((9 * 32, 37 * 32), blocks=list(zip(cols, rows)), seed=54)
    dy = randn((9000, 9 * 32), seed=55)
    check(run_dsd(mt, dy, False, "tf32x3" if group != "8" else "tf32"), oracle_dsd(mt, dy, False),
          "tf32x3" if group != "8" else "tf32", "dgrad")
    assert_device_healthy()
