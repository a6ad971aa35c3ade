"""Sparsity-pattern optimizer: magnitude pruning of blocks + random regrowth, on the device.

Public surface of ``pytorch_block_sparse/sparse_optimizer.py`` of the reference (same class names, same
param-group keys: ``lr`` = fraction of blocks recycled per step, ``method``, ``new_coefficients_scale``,
``new_coefficients_distribution``; same exception texts), same step (reference ``sparse_optimizer.py:38-87``,
``:127-155``, ``:292-304``): rank the slots by block norm, move the lowest ``lr`` fraction to random empty
positions, re-initialise the moved slots and zero their Adam moments.

The step itself is rebuilt around the library's pattern kernels (``csrc/bsmm_pattern.cu``) and runs without a
host round trip when the matrix lives on a GPU:

* ranking     the per-slot sum of squares comes from the statistic kernel; the recycled slots are the exact
              ``k`` smallest (``bsmm_select_lowest``, a radix select) -- no full sort;
* regrowth    ``k`` distinct empty positions from a keyed permutation of the empty cells
              (``bsmm_sample_free_cells``): a pure function of (pattern, seed), so every rank of a data-parallel
              job that constructs its ``SparseOptimizer`` with the same ``seed`` moves the same blocks to the
              same places, where the reference draws ``torch.randperm`` on the host per process;
* re-indexing ``bsmm_move_blocks`` + ``bsmm_rebuild_indices`` rewrite ``blocks``, the CSR and the CSC buffers
              in place (bit-identical to what ``block_replace`` derives on the host);
* state       the moved slots are re-initialised and their Adam moments zeroed by slot index
              (``index_copy_`` / ``index_fill_`` on ``[nnz, block]`` views): no ``data``-sized mask.

CPU matrices take the host path (``block_replace`` with torch ops), as in the reference.
"""
import torch
import torch.optim as optim

from . import native
from .block_sparse import BlockSparseMatrix


class RecycledSlots:
    """Which slots a cleaning step moved: ``slots`` (int64 ``[k]``) out of ``nnz`` slots of ``block`` values each.
    Stands where the reference passes a ``data``-shaped 0/1 mask (``sparse_optimizer.py:78-87``)."""

    def __init__(self, slots, nnz, block_shape):
        self.slots = slots
        self.nnz = nnz
        self.block_shape = tuple(block_shape)

    def zero_(self, tensor):
        """Zero the moved slots of a tensor laid out like ``data``."""
        if self.slots.numel():
            tensor.view(self.nnz, -1).index_fill_(0, self.slots, 0)
        return tensor

    def as_mask(self, like):
        """The reference's ``state_keep_mask``: 1 where the slot stayed, 0 where it moved."""
        return self.zero_(torch.ones_like(like))


class SparseOptimizerStrategy:
    def run(self, block_sparse_matrix):
        raise NotImplementedError()


class MagnitudeSparseOptimizerStrategy(SparseOptimizerStrategy):
    def __init__(self, cleanup_ratio, new_coefficients_distribution="uniform", new_coefficients_scale=0.1, seed=0):
        self.cleanup_ratio = cleanup_ratio
        self.new_coefficients_distribution = new_coefficients_distribution
        self.new_coefficients_scale = new_coefficients_scale
        self.seed = int(seed)

    def fresh_values(self, data, count, block_elems, generator=None):
        """``[count, block]`` values for re-initialised slots, from the distribution the reference uses
        (``sparse_optimizer.py:23-36``).  Its "uniform" draws with ``random_(0, 1)``, which yields only zeros, so
        that mode is the constant ``-std * scale``; kept as is.  ``mean`` / ``std`` stay tensors: no host sync."""
        mean, std = data.mean(), data.std()
        scale = self.new_coefficients_scale
        if self.new_coefficients_distribution == "gaussian":
            noise = torch.randn((count, block_elems), generator=generator, device=data.device, dtype=data.dtype)
            return noise * (std * scale) + mean * scale
        if self.new_coefficients_distribution == "uniform":
            return (torch.zeros((count, block_elems), device=data.device, dtype=data.dtype) - 0.5) * (2 * std * scale)
        raise Exception("Unknown new coefficients method %s" % self.new_coefficients_distribution)

    def run(self, block_sparse_matrix):
        bsm = block_sparse_matrix
        X, Y = bsm.blocks_count()
        nnz = bsm.blocks.shape[0] // 2
        k = int(nnz * self.cleanup_ratio)
        k = min(k, X * Y - nnz)  # there must be an empty position for every moved block
        device = bsm.data.device
        if k <= 0:
            return RecycledSlots(torch.empty(0, dtype=torch.long, device=device), nnz, bsm.block_shape)
        norms = bsm.block_norm()
        if bsm.data.is_cuda:
            recycled32 = native.select_lowest(norms, k)
            cells = bsm.sample_free_positions(k, self.seed)
            bsm.move_blocks_(recycled32, cells)
            recycled = recycled32.long()
            generator = torch.Generator(device=device)
            generator.manual_seed(self.seed)
        else:
            recycled = norms.sort()[1][:k]
            free = (~bsm.block_mask_build(None)).nonzero()
            g = torch.Generator().manual_seed(self.seed)
            pick = torch.randperm(free.shape[0], generator=g)[:k]
            bsm.block_replace(torch.cat([free[pick], recycled.unsqueeze(-1)], -1))
            generator = g
        with torch.no_grad():
            data = bsm.data.detach()
            data.view(nnz, -1).index_copy_(0, recycled, self.fresh_values(data, k, data.numel() // nnz, generator))
        bsm.updated_data()
        bsm.invalidate_packed()
        return RecycledSlots(recycled, nnz, bsm.block_shape)


class _RequiredParameter(object):
    def __repr__(self):
        return "<required parameter>"


required = _RequiredParameter()


class OptimizerStateUpdater:
    def __init__(self, optimizer, sparse_object):
        self.optimizer = optimizer
        if not isinstance(sparse_object, BlockSparseMatrix):
            raise Exception(f"Unknown sparse_object type {sparse_object}")
        self.sparse_object = sparse_object

    def update_state_data(self, param, recycled):
        raise NotImplementedError()

    def update_state(self, recycled):
        """Apply to the optimizer state of the matrix's ``data`` parameter; False if no group holds it."""
        target = self.sparse_object.data
        params = [p for group in self.optimizer.param_groups for p in group["params"] if p is target]
        for param in params:
            self.update_state_data(param, recycled)
        return bool(params)


class AdamOptimizerStateUpdater(OptimizerStateUpdater):
    MOMENTS = ("exp_avg", "exp_avg_sq", "max_exp_avg_sq")

    @staticmethod
    def is_compatible(optimizer):
        if isinstance(optimizer, (optim.Adam, optim.AdamW)):
            return True
        try:
            import transformers.optimization as transformers_optim

            adamw = getattr(transformers_optim, "AdamW", None)
            return adamw is not None and isinstance(optimizer, adamw)
        except Exception:
            return False

    def update_state_data(self, param, recycled):
        for key, value in self.optimizer.state[param].items():
            if key in self.MOMENTS:
                if isinstance(recycled, RecycledSlots):
                    recycled.zero_(value)
                else:  # a data-shaped keep mask, the reference's convention
                    value *= recycled
            elif key != "step":  # shared step count: bias correction of the fresh blocks is slightly off, as in the reference
                raise Exception(f"Unknown key in Adam parameter state {key}")


class SparseOptimizer(torch.optim.Optimizer):
    """``SparseOptimizer([BlockSparseMatrix, ...], lr=0.1, method="magnitude", ...)``; call ``step()``
    once per training step (reference ``sparse_optimizer.py:158-304``).  ``seed`` (not in the reference) makes the
    regrowth positions and the fresh values a function of (seed, step number, matrix number): give every rank of
    a data-parallel job the same value and the patterns stay identical without any broadcast."""

    METHODS = ["magnitude"]
    COEFFICIENTS_DISTRIBUTION = ["uniform", "gaussian"]
    allowed_keys = {"lr", "method", "new_coefficients_scale", "new_coefficients_distribution"}

    def __init__(
        self,
        sparse_objects,
        lr=1e-1,
        method="magnitude",
        new_coefficients_scale=0.1,
        new_coefficients_distribution="uniform",
        seed=0,
    ):
        if not 0.0 < lr:
            raise ValueError("Invalid learning rate: {}".format(lr))
        defaults = dict(
            lr=lr,
            method=method,
            new_coefficients_scale=new_coefficients_scale,
            new_coefficients_distribution=new_coefficients_distribution,
        )
        self.seed = int(seed)
        self.steps_done = 0
        super().__init__([{"sparse_objects": sparse_objects}], defaults)
        self.attached_optimizers = []

    @staticmethod
    def sparse_objects(model):
        return [m for _, m in model.named_modules() if isinstance(m, BlockSparseMatrix)]

    def attach_optimizer(self, optimizer):
        if optimizer not in self.attached_optimizers:
            self.attached_optimizers.append(optimizer)

    def add_param_group(self, sparse_objects_group):
        assert isinstance(sparse_objects_group, dict), "param group must be a dict"
        unknown = [k for k in sparse_objects_group if k != "sparse_objects" and k not in self.allowed_keys]
        if unknown:
            raise Exception("Unknown cleaning parameter %s" % unknown[0])
        objs = sparse_objects_group["sparse_objects"]
        objs = [objs] if isinstance(objs, BlockSparseMatrix) else list(objs)
        for p in objs:
            if not isinstance(p, BlockSparseMatrix):
                raise Exception("I don't know how to clean this type of object: %s" % p)
        sparse_objects_group["sparse_objects"] = objs
        for name, default in self.defaults.items():
            if default is required and name not in sparse_objects_group:
                raise ValueError("parameter group didn't specify a value of required optimization parameter " + name)
            sparse_objects_group.setdefault(name, default)
        if sparse_objects_group["method"] not in self.METHODS:
            raise Exception(f"Invalid Method {sparse_objects_group['method']}")
        if sparse_objects_group["new_coefficients_distribution"] not in self.COEFFICIENTS_DISTRIBUTION:
            raise Exception(
                f"Invalid new coefficients distribution {sparse_objects_group['new_coefficients_distribution']}"
            )
        already = {id(p) for group in self.param_groups for p in group["sparse_objects"]}
        if any(id(p) in already for p in objs):
            raise ValueError("some parameters appear in more than one parameter group")
        self.param_groups.append(sparse_objects_group)

    def clean(self, p, method, clean_ratio, new_coefficients_scale, new_coefficients_distribution, seed=None):
        if not isinstance(p, BlockSparseMatrix):
            raise Exception("I don't know how to clean this : %s" % p)
        if method != "magnitude":
            raise Exception(f"Unknowncleaning method {method}")
        strategy = MagnitudeSparseOptimizerStrategy(
            clean_ratio,
            new_coefficients_distribution=new_coefficients_distribution,
            new_coefficients_scale=new_coefficients_scale,
            seed=self.seed if seed is None else seed,
        )
        recycled = strategy.run(p)
        if not self.attached_optimizers:
            return
        found = False
        for optimizer in self.attached_optimizers:
            if not AdamOptimizerStateUpdater.is_compatible(optimizer):
                raise Exception(f"unsupported optimizer {optimizer.__class__}")
            found = AdamOptimizerStateUpdater(optimizer, p).update_state(recycled) or found
        if not found:
            raise Exception(f"Could not find sparse object {p} in optimizers {self.attached_optimizers}")

    def step(self):
        ordinal = 0
        for group in self.param_groups:
            ratio = group["lr"]
            for p in group["sparse_objects"]:
                ordinal += 1
                if ratio == 0.0:
                    continue
                self.clean(
                    p,
                    clean_ratio=ratio,
                    method=group["method"],
                    new_coefficients_scale=group["new_coefficients_scale"],
                    new_coefficients_distribution=group["new_coefficients_distribution"],
                    seed=(self.seed * 1000003 + self.steps_done) * 1009 + ordinal,
                )
        self.steps_done += 1
