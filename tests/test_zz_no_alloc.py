"""The allocation-free weight-gradient entry point, bsmm_sddmm_static.

Who needs it: a host that may not call cudaMalloc where wgrad runs -- a stream being captured into a CUDA
graph, a runtime that hands out all device memory up front, an allocator callback.  bsmm_sddmm wants a
caller-allocated workspace for the partial sums of its token ranges; the static variant keeps them in an
array inside the library image (64 MiB, shared by every call on the device).

Checked here, through the C-ABI: same result as bsmm_sddmm on the same inputs (the kernels and the
token split are identical, so bit-exact; the tolerance of the other wgrad tests is also applied), on two
calls in a row with different inputs (the array keeps the previous call's bytes), and a clean refusal of
a problem beyond the limit.  The file sorts last so that a run stopping at the first failure has already
run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import block_sparse_oracle as orc
from pytorch_block_sparse_b200 import native

from .gpu_util import TOL, assert_device_healthy, make_matrix, randn

pytestmark = pytest.mark.gpu


def test_static_scratch_variant_matches_workspace_variant_twice():
    m = make_matrix((128, 1024), n_blocks=90, seed=61)
    plan = m._sddmm_plan()
    lib = native.load()
    for call, tokens in enumerate((6000, 4500)):  # both split the token axis: the scratch array is used
        dy = randn((tokens, 128), seed=62 + call).cuda()
        x = randn((tokens, 1024), seed=64 + call).cuda()
        need = lib.bsmm_sddmm_workspace_bytes(128, 1024, tokens, 90, native.PREC_TF32X3)
        assert 0 < need <= native.SDDMM_STATIC_MAX_BYTES
        ref = torch.empty_like(m.data)
        native.sddmm(dy, True, x, True, m.blocks, ref.detach(), precision="tf32x3", plan=plan)
        got = torch.full_like(m.data, float("nan"))
        stat = torch.empty(90, device="cuda")
        allocated = torch.cuda.memory_allocated()
        native.sddmm_static(dy, x, m.blocks, got.detach(), plan, block_sumsq=stat)
        assert torch.cuda.memory_allocated() == allocated  # the wrapper went through no torch allocation either
        torch.cuda.synchronize()
        assert torch.equal(got, ref), f"call {call}"
        want = orc.wgrad(dy.cpu().numpy(), x.cpu().numpy(), (128, 1024), m.blocks.cpu().numpy())
        assert orc.rel_fro(got.detach().cpu().numpy(), want) <= TOL["tf32x3"]
        assert np.allclose(stat.cpu().numpy(), orc.block_norm(want) ** 2, rtol=1e-4)
    assert_device_healthy()


def test_static_scratch_variant_refuses_oversized_problems():
    lib = native.load()
    fake = ctypes.c_void_p(0x1000)
    # 9000 blocks x 4 KiB x two token ranges is beyond 64 MiB; refused before anything is launched
    assert lib.bsmm_sddmm_workspace_bytes(4096, 4096, 65536, 9000, native.PREC_TF32X3) > native.SDDMM_STATIC_MAX_BYTES
    status = lib.bsmm_sddmm_static(fake, fake, 4096, 4096, 65536, fake, fake, 9000, fake, fake, None,
                                   native.PREC_TF32X3, None)
    assert status == 4  # BSMM_ERR_TOO_LARGE
    assert b"limit" in lib.bsmm_status_string(status)
