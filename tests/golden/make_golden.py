"""Generates tests/golden/*.npz by running the REFERENCE implementation on CPU.

Run where the reference checkout is importable:

    PYTHONPATH=<reference checkout> python tests/golden/make_golden.py

It imports ``pytorch_block_sparse`` (the reference), builds matrices with its own factories
(``BlockSparseMatrix.zeros/randn/from_dense`` on ``device="cpu"``), and records

* index buffers for explicit and seeded random patterns           -> indices.npz
* ``block_replace`` results                                       -> replace.npz
* ``to_dense`` / ``from_dense`` values                             -> dense.npz
* fwd / dgrad / wgrad of the reference's ``to_dense`` + ``torch.matmul`` path
  (a small case in full, benchmark configuration 1 as a strided sample)   -> linear.npz
* the ``state_dict`` of a layer-shaped reference module (the keys a reference checkpoint holds for one
  ``BlockSparseLinear``), its dense weight and one forward result        -> checkpoint.npz

The committed .npz files are what the tests read; the reference is not needed to run them.
"""
import hashlib
import os
import sys

import numpy as np
import torch

import pytorch_block_sparse as ref  # the reference, not this repository's package

assert "b200" not in ref.__file__, "PYTHONPATH must point at the reference checkout"
OUT = os.path.dirname(os.path.abspath(__file__))
BSM = ref.BlockSparseMatrix


def indices_of(m):
    return {k: getattr(m, k).numpy().copy() for k in ("blocks", "cols_a", "row_start_ends_a", "rows_b", "col_start_ends_b")}


def gen_indices():
    out = {}
    cases = []
    # the explicit pattern of the reference's tests/test_basic.py:11-46
    cases.append(("explicit_128x64", (128, 64), [(0, 0), (1, 0), (2, 0), (0, 1)], None, None))
    for seed, shape, n in [(0, (256, 1024), 128), (1, (64, 64), 1), (2, (768, 3072), 1152), (3, (96, 160), 15), (4, (32, 32), 1), (5, (512, 512), 256)]:
        cases.append((f"random_s{seed}_{shape[0]}x{shape[1]}_n{n}", shape, None, n, seed))
    names = []
    for name, shape, blocks, n, seed in cases:
        if seed is not None:
            np.random.seed(seed)
        m = BSM.zeros(shape, n_blocks=n, blocks=blocks, device="cpu")
        names.append(name)
        out[name + "/shape"] = np.array(shape)
        out[name + "/seed"] = np.array(-1 if seed is None else seed)
        out[name + "/n"] = np.array(len(blocks) if blocks is not None else n)
        out[name + "/mask"] = m.block_mask_build(None).numpy()
        for k, v in indices_of(m).items():
            out[name + "/" + k] = v
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(OUT, "indices.npz"), **out)


def gen_replace():
    out = {}
    names = []
    # the case of the reference's tests/test_replace.py:23-43
    m = BSM.zeros((128, 64), blocks=[(0, 0), (1, 0), (2, 0), (0, 1)], device="cpu")
    cases = [("explicit", m, np.array([(3, 1, 0), (2, 1, 2), (1, 1, 1)]))]
    np.random.seed(11)
    torch.manual_seed(11)
    m2 = BSM.zeros((256, 512), n_blocks=40, device="cpu")
    free = (~m2.block_mask_build(None)).nonzero()
    pick = torch.randperm(free.shape[0])[:9]
    slots = torch.randperm(40)[:9]
    cases.append(("random", m2, torch.cat([free[pick], slots.unsqueeze(-1)], -1).numpy()))
    for name, mat, repl in cases:
        names.append(name)
        out[name + "/shape"] = np.array(mat.shape)
        for k, v in indices_of(mat).items():
            out[name + "/before/" + k] = v
        out[name + "/replacements"] = repl
        mat.block_replace(torch.tensor(repl))
        for k, v in indices_of(mat).items():
            out[name + "/after/" + k] = v
        out[name + "/after/mask"] = mat.block_mask_build(None).numpy()
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(OUT, "replace.npz"), **out)


def gen_dense():
    out = {}
    np.random.seed(21)
    torch.manual_seed(21)
    m = BSM.randn((96, 128), n_blocks=5, device="cpu")
    out["shape"] = np.array(m.shape)
    out["blocks"] = m.blocks.numpy()
    out["data"] = m.data.detach().numpy()
    out["dense"] = m.to_dense().detach().numpy()
    # from_dense with an explicit pattern (gather path) and with a truncated block count
    dense = torch.randn(64, 96)
    g = BSM.from_dense(dense, blocks=[(0, 0), (1, 2), (0, 1)])
    out["fd_dense"] = dense.numpy()
    out["fd_blocks"] = g.blocks.numpy()
    out["fd_data"] = g.data.detach().numpy()
    np.random.seed(22)
    t = BSM.from_dense(dense, block_count=3)
    out["fd_trunc_blocks"] = t.blocks.numpy()
    out["fd_trunc_data"] = t.data.detach().numpy()
    out["block_norm"] = m.block_norm().detach().numpy()
    np.savez_compressed(os.path.join(OUT, "dense.npz"), **out)


def ref_linear(m, x, dy, bias):
    """fwd / dgrad / wgrad exactly as the reference's dense path computes them on CPU."""
    wd = m.to_dense()
    y = x.reshape(-1, x.shape[-1]) @ wd.t() + bias
    dx = dy.reshape(-1, dy.shape[-1]) @ wd
    mask = m.to_dense(data_replace=torch.ones_like(m.data))
    dw_dense = (dy.reshape(-1, dy.shape[-1]).t() @ x.reshape(-1, x.shape[-1])) * mask
    dw = BSM.from_dense(dw_dense, blocks=[(int(r), int(c)) for r, c in m.build_coo_block_index().t()]).data
    return y, dx, dw.detach()


def sha(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def gen_linear():
    out = {}
    # small case, stored in full
    np.random.seed(31)
    torch.manual_seed(31)
    m = BSM.zeros((128, 256), n_blocks=16, device="cpu")
    with torch.no_grad():
        m.data.normal_(0, 0.02)
    x = torch.randn(3, 20, 256)
    dy = torch.randn(3, 20, 128)
    bias = torch.randn(128) * 0.02
    y, dx, dw = ref_linear(m, x, dy, bias)
    out["small/shape"] = np.array(m.shape)
    for k, v in indices_of(m).items():
        out["small/" + k] = v
    out["small/data"] = m.data.detach().numpy()
    out["small/x"] = x.numpy()
    out["small/dy"] = dy.numpy()
    out["small/bias"] = bias.numpy()
    out["small/y"] = y.detach().numpy()
    out["small/dx"] = dx.detach().numpy()
    out["small/dw"] = dw.numpy()

    # benchmark configuration 1: inputs re-derived from the seed by the test (hash recorded), outputs sampled
    np.random.seed(1)
    torch.manual_seed(1)
    m = BSM.zeros((256, 1024), n_blocks=128, device="cpu")
    with torch.no_grad():
        m.data.normal_(0, 0.02)
    x = torch.randn(256, 1024)
    dy = torch.randn(256, 256)
    bias = torch.randn(256) * 0.02
    y, dx, dw = ref_linear(m, x, dy, bias)
    out["c1/input_sha256"] = np.array(sha(m.blocks.numpy(), m.data.detach().numpy(), x.numpy(), dy.numpy(), bias.numpy()))
    out["c1/blocks"] = m.blocks.numpy()
    out["c1/stride"] = np.array(61)
    out["c1/y"] = y.detach().numpy().reshape(-1)[::61]
    out["c1/dx"] = dx.detach().numpy().reshape(-1)[::61]
    out["c1/dw"] = dw.numpy().reshape(-1)[::61]
    np.savez_compressed(os.path.join(OUT, "linear.npz"), **out)


def gen_checkpoint():
    """What a checkpoint written by the reference holds for one BlockSparseLinear: ``weight.data``, the five
    index buffers under ``weight.*`` and ``bias`` (BlockSparseLinear itself is CUDA-only in the reference,
    block_sparse_linear.py:217, so a module of the same attribute layout is assembled on the CPU)."""

    class LayerShaped(torch.nn.Module):
        def __init__(self, weight, bias):
            super().__init__()
            self.weight = weight
            self.bias = torch.nn.Parameter(bias)

    np.random.seed(41)
    torch.manual_seed(41)
    m = BSM.randn((128, 192), n_blocks=9, device="cpu")
    # a pattern history: two slots moved, so slot order differs from row-major order
    free = (~m.block_mask_build(None)).nonzero()
    m.block_replace(torch.cat([free[[1, 4]], torch.tensor([[6], [2]])], -1))
    layer = LayerShaped(m, torch.randn(128) * 0.02)
    out = {"sd/" + k: v.detach().numpy() for k, v in layer.state_dict().items()}
    out["keys"] = np.array(list(layer.state_dict().keys()))
    out["dense"] = m.to_dense().detach().numpy()
    x = torch.randn(10, 192)
    out["x"] = x.numpy()
    out["y"] = (x @ m.to_dense().t() + layer.bias).detach().numpy()
    np.savez_compressed(os.path.join(OUT, "checkpoint.npz"), **out)


if __name__ == "__main__":
    gen_checkpoint()
    gen_indices()
    gen_replace()
    gen_dense()
    gen_linear()
    print("wrote", sorted(f for f in os.listdir(OUT) if f.endswith(".npz")))
