"""Builds libbsmm_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: ``python -m pytorch_block_sparse_b200.build [--force] [--verbose]``.

``python -m pytorch_block_sparse_b200.build --microbench [--run]`` compiles (and runs, on a B200) the
single-CTA micro-benchmarks under ``csrc/microbench/``: cycles per ``tcgen05.mma`` by shape and operand source,
the kernels' exact MMA sequences, mbarrier wait and ring hand-off costs, tensor-memory store/load costs and
the L2 -> shared-memory bulk-copy bandwidth.  The kernels' cost model rests on these figures.
"""
import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_PATH = os.path.join(PKG_DIR, "libbsmm_b200.so")
SOURCES = ["bsmm_api.cu", "bsmm_simt.cu", "bsmm_pack.cu", "bsmm_plan.cu", "bsmm_pattern.cu", "bsmm_collective.cu", "bsmm_umma.cu", "bsmm_sddmm_umma.cu"]
HEADERS = ["bsmm_common.cuh", "bsmm_umma.cuh", "bsmm_ptx.cuh"]


def nvcc_path():
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.join(INCLUDE, "bsmm_b200.h")]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    """Compile every .cu for sm_100a and link the shared library; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    srcs = [os.path.join(CSRC, f) for f in SOURCES if os.path.exists(os.path.join(CSRC, f))]
    cmd = [
        nvcc_path(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-lineinfo", "-std=c++17",
        "--shared", "-Xcompiler", "-fPIC",
        "-I", INCLUDE, "-I", CSRC,
        "-o", LIB_PATH,
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += srcs
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n%s\n%s" % (" ".join(cmd), res.stdout))
    if verbose:
        print(res.stdout)
    return LIB_PATH


MICROBENCH_DIR = os.path.join(CSRC, "microbench")
MICROBENCH_BIN = os.path.join(PKG_DIR, "microbench_bin")


def build_microbench(run=False):
    """Compile every csrc/microbench/*.cu into microbench_bin/<name>; with run=True execute them in turn."""
    os.makedirs(MICROBENCH_BIN, exist_ok=True)
    built = []
    for src in sorted(f for f in os.listdir(MICROBENCH_DIR) if f.endswith(".cu")):
        exe = os.path.join(MICROBENCH_BIN, src[:-3])
        cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
               "-I", CSRC, "-I", INCLUDE, "-o", exe, os.path.join(MICROBENCH_DIR, src)]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n%s\n%s" % (" ".join(cmd), res.stdout))
        built.append(exe)
    if run:
        for exe in built:
            print("==", os.path.basename(exe), flush=True)
            subprocess.run([exe], check=False)
    return built


if __name__ == "__main__":
    if "--microbench" in sys.argv:
        for path in build_microbench(run="--run" in sys.argv):
            print(path)
    else:
        build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
        print(LIB_PATH)
