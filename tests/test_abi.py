"""The C-ABI library: builds for sm_100a, loads, exports exactly what include/bsmm_b200.h declares,
and validates arguments before touching the device (no kernel runs here)."""
import ctypes
import os
import re

from pytorch_block_sparse_b200 import build as bsmm_build
from pytorch_block_sparse_b200 import native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "bsmm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bsmm_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = bsmm_build.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    names = declared_functions()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(native.EXPORTS) == names


def test_abi_version_and_status_strings():
    lib = native.load()
    assert lib.bsmm_abi_version() == native.ABI_VERSION
    assert lib.bsmm_status_string(0) == b"ok"
    assert b"invalid" in lib.bsmm_status_string(1)


def test_size_queries():
    lib = native.load()
    assert lib.bsmm_packed_bytes(10, native.PREC_TF32X3) == 2 * 10 * 8192
    assert lib.bsmm_packed_bytes(10, native.PREC_BF16) == 2 * 10 * 2048
    assert lib.bsmm_packed_bytes(10, native.PREC_FP32_SIMT) == 0
    assert lib.bsmm_packed_bytes(-1, native.PREC_TF32X3) == -1
    assert lib.bsmm_plan_bytes(16, 100, 8) == 32 + 100 * 16
    assert lib.bsmm_plan_bytes(16, 100, 4) == 48 + 100 * 16
    assert lib.bsmm_plan_bytes(16, 100, 7) == -1
    assert lib.bsmm_plan_group(16384, 128, 4096, native.PREC_TF32) == 8
    assert lib.bsmm_plan_group(16384, 128, 4096, native.PREC_TF32X3) == 4  # many waves: four activation stages
    assert lib.bsmm_plan_group(4096, 96, 2304, native.PREC_TF32X3) == 6
    assert lib.bsmm_plan_group(128, 24, 288, native.PREC_TF32X3) == 4
    assert lib.bsmm_packed_bytes(10, native.PREC_TF32) == 2 * 10 * 8192
    assert lib.bsmm_packed_bytes(10, native.PREC_BF16X3) == 2 * 10 * 4096  # bf16 hi | lo images
    assert lib.bsmm_plan_group(16384, 128, 4096, native.PREC_BF16X3) == 4  # rows with correction columns: as 3xTF32
    assert lib.bsmm_sddmm_workspace_bytes(4096, 4096, 16384, 4096, native.PREC_BF16X3) == \
        lib.bsmm_sddmm_workspace_bytes(4096, 4096, 16384, 4096, native.PREC_TF32X3) > 0  # wgrad computes as 3xTF32
    assert lib.bsmm_sddmm_plan_bytes(8, 100) == 16 + 16 * (100 // 8 + 8)  # items of at most 8 blocks
    assert lib.bsmm_sddmm_workspace_bytes(64, 64, 100, 2, native.PREC_FP32_SIMT) == 0


def test_argument_validation_without_device():
    lib = native.load()
    null = ctypes.c_void_p(None)
    fake = ctypes.c_void_p(0x1000)
    # n not a multiple of 32
    assert lib.bsmm_dsd(fake, 4, 32, fake, fake, 1, fake, null, null, 33, fake, null, 0, null) == 1
    # null output
    assert lib.bsmm_dsd(fake, 4, 32, fake, fake, 1, fake, null, null, 32, null, null, 0, null) == 1
    # tensor-core precision without packed images / plan, or without the plan's group size in the flags
    assert lib.bsmm_dsd(fake, 4, 32, fake, fake, 1, fake, null, null, 32, fake, null, native.PREC_TF32X3 | (6 << 8), null) == 1
    assert lib.bsmm_dsd(fake, 4, 32, fake, fake, 1, fake, fake, fake, 32, fake, null, native.PREC_TF32X3, null) == 1
    # bias with dgrad
    assert lib.bsmm_dsd(fake, 4, 32, fake, fake, 1, fake, null, null, 32, fake, fake, native.DSD_DGRAD, null) == 2
    # empty problem is a no-op
    assert lib.bsmm_dsd(null, 0, 32, fake, null, 0, null, null, null, 32, fake, null, 0, null) == 0
    # misaligned pointer
    assert lib.bsmm_sddmm(ctypes.c_void_p(0x1004), fake, 32, 32, 8, fake, fake, 1, null, null, null, null, 0, null) == 1
    assert lib.bsmm_sddmm(fake, fake, 48, 32, 8, fake, fake, 1, null, null, null, null, 0, null) == 1
    assert lib.bsmm_sddmm(fake, fake, 32, 32, 8, fake, fake, 1, null, null, null, null, 7, null) == 2  # no such arithmetic
    assert lib.bsmm_build_sddmm_plan(null, 4, 4, fake, null) == 1
    assert lib.bsmm_pack_weights(null, 3, native.PREC_TF32X3, fake, null, null) == 1
    assert lib.bsmm_build_plan(null, fake, 4, 4, 6, fake, null) == 1
    assert lib.bsmm_build_plan(fake, fake, 4, 4, 7, fake, null) == 1
