"""Builds the REFERENCE's own CUDA extension (block_sparse_native) for sm_100a from its sources where they
lie, into oracle/_ref/ -- TEST INFRASTRUCTURE: a second, on-device oracle and the "reference kernels on
B200" comparator of bench.py.  Nothing of the reference is copied into this repository; the product
never loads this library.

    python oracle/build_ref.py /path/to/reference/checkout

The three sources (native/block_sparse_native.cpp, block_sparse_cutlass_kernel.cu,
block_sparse_cutlass_kernel_back.cu) need torch's extension headers, so the recipe goes through
torch.utils.cpp_extension (nvcc + ninja), not through the reference's setup.py.
"""
import os
import sys


def build(reference_root, verbose=True):
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", "3")
    from torch.utils import cpp_extension

    pkg = os.path.join(reference_root, "pytorch_block_sparse")
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    os.makedirs(out, exist_ok=True)
    srcs = [os.path.join(pkg, "native", f) for f in
            ("block_sparse_native.cpp", "block_sparse_cutlass_kernel.cu", "block_sparse_cutlass_kernel_back.cu")]
    return cpp_extension.load(
        name="block_sparse_native", sources=srcs, extra_include_paths=[pkg], build_directory=out,
        extra_cuda_cflags=["-O3", "-gencode", "arch=compute_100a,code=sm_100a"], verbose=verbose,
    )


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BSMM_REFERENCE_ROOT")
    if not root:
        sys.exit("usage: python oracle/build_ref.py /path/to/reference/checkout   (or set BSMM_REFERENCE_ROOT)")
    build(root)
    print("built into oracle/_ref")
