"""B200-native block-sparse Linear engine with the pytorch_block_sparse API."""
from .block_sparse import BlockSparseMatrix, BlockSparseMatrixBase, BlockSparseMatrixEmulator
from .block_sparse_linear import BlockSparseLinear, BlockSparseLinearFunction, PseudoBlockSparseLinear
from .sparse_optimizer import SparseOptimizer
from .util import BlockSparseModelPatcher
from .native import set_default_precision

__all__ = [
    "BlockSparseMatrix",
    "BlockSparseMatrixBase",
    "BlockSparseMatrixEmulator",
    "BlockSparseLinear",
    "BlockSparseLinearFunction",
    "PseudoBlockSparseLinear",
    "BlockSparseModelPatcher",
    "SparseOptimizer",
    "set_default_precision",
]
