"""Sparsity-pattern optimizer: magnitude pruning of blocks + random regrowth.

Mirrors ``pytorch_block_sparse/sparse_optimizer.py`` of the reference: the same classes, the
same param-group keys (``lr`` = fraction of blocks recycled per step, ``method``,
``new_coefficients_scale``, ``new_coefficients_distribution``) and the same step:
rank slots by block norm, move the lowest ``lr`` fraction to random free positions
(``block_replace``), re-initialise the moved slots and zero their Adam moments
(reference ``sparse_optimizer.py:38-87``, ``:127-155``, ``:292-304``).

The block norms come from the per-slot sum of squares that the weight-packing kernel already
produces for the matmuls, so ranking costs no extra pass over ``data``.
"""
import torch
import torch.optim as optim

from .block_sparse import BlockSparseMatrix


class SparseOptimizerStrategy:
    def run(self, block_sparse_matrix):
        raise NotImplementedError()


class MagnitudeSparseOptimizerStrategy(SparseOptimizerStrategy):
    def __init__(self, cleanup_ratio, new_coefficients_distribution="uniform", new_coefficients_scale=0.1):
        self.cleanup_ratio = cleanup_ratio
        self.new_coefficients_distribution = new_coefficients_distribution
        self.new_coefficients_scale = new_coefficients_scale

    def initialize_new_blocks(self, old_data, new_data):
        """Fill ``new_data`` with the distribution the reference uses (``sparse_optimizer.py:23-36``),
        including its ``random_(0, 1)`` draw for "uniform" (which yields zeros before the shift)."""
        mean, std = old_data.mean(), old_data.std()
        scale = self.new_coefficients_scale
        if self.new_coefficients_distribution == "gaussian":
            new_data.normal_(mean=float(mean * scale), std=float(std * scale))
        elif self.new_coefficients_distribution == "uniform":
            new_data.random_(0, 1)
            new_data -= 0.5
            new_data *= 2 * std * scale
        else:
            raise Exception("Unknown new coefficients method %s" % self.new_coefficients_distribution)

    def block_norms(self, bsm):
        return bsm.block_norm()

    def run(self, block_sparse_matrix):
        bsm = block_sparse_matrix
        bh, bw = bsm.block_shape
        order = self.block_norms(bsm).sort()[1]
        recycled = order[: int(order.shape[0] * self.cleanup_ratio)]

        free = (~bsm.block_mask_build(None)).nonzero()
        pick = torch.randperm(free.shape[0])[: recycled.shape[0]].to(free.device)
        bsm.block_replace(torch.cat([free[pick], recycled.unsqueeze(-1)], -1))

        moved = torch.zeros(bsm.data.shape[0] // bh, dtype=torch.bool, device=bsm.data.device)
        moved[recycled] = True
        moved = moved.repeat_interleave(bh).unsqueeze(-1).expand(-1, bw).float()

        fresh = torch.zeros_like(bsm.data)
        self.initialize_new_blocks(bsm.data, fresh)
        keep = 1.0 - moved
        with torch.no_grad():
            bsm.data.mul_(keep).add_(fresh * moved)
        return keep


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

    def update_state_data(self, param, state_keep_mask):
        raise NotImplementedError()

    def update_state(self, state_keep_mask):
        target = self.sparse_object.data
        found = False
        for group in self.optimizer.param_groups:
            for param in group["params"]:
                if param is target:
                    found = True
                    self.update_state_data(param, state_keep_mask)
        return found


class AdamOptimizerStateUpdater(OptimizerStateUpdater):
    @staticmethod
    def is_compatible(optimizer):
        if isinstance(optimizer, (optim.Adam, optim.AdamW)):
            return True
        try:
            import transformers.optimization as transformers_optim

            adamw = getattr(transformers_optim, "AdamW", None)
            if adamw is not None and isinstance(optimizer, adamw):
                return True
        except Exception:
            pass
        return False

    def update_state_data(self, param, state_keep_mask):
        state = self.optimizer.state[param]
        for key in state:
            if key in ("exp_avg", "exp_avg_sq", "max_exp_avg_sq"):
                state[key] *= state_keep_mask
            elif key == "step":
                pass  # shared step count: bias correction of the fresh blocks is slightly off, as in the reference
            else:
                raise Exception(f"Unknown key in Adam parameter state {key}")


class SparseOptimizer(torch.optim.Optimizer):
    """``SparseOptimizer([BlockSparseMatrix, ...], lr=0.1, method="magnitude", ...)``; call ``step()``
    once per training step (reference ``sparse_optimizer.py:158-304``)."""

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
    ):
        if not 0.0 < lr:
            raise ValueError("Invalid learning rate: {}".format(lr))
        defaults = dict(
            lr=lr,
            method=method,
            new_coefficients_scale=new_coefficients_scale,
            new_coefficients_distribution=new_coefficients_distribution,
        )
        super().__init__([{"sparse_objects": sparse_objects}], defaults)
        self.attached_optimizers = []

    @staticmethod
    def sparse_objects(model):
        return [m for _, m in model.named_modules() if isinstance(m, BlockSparseMatrix)]

    def attach_optimizer(self, optimizer):
        if optimizer in self.attached_optimizers:
            return
        self.attached_optimizers.append(optimizer)

    def add_param_group(self, sparse_objects_group):
        assert isinstance(sparse_objects_group, dict), "param group must be a dict"
        for k in sparse_objects_group:
            if k != "sparse_objects" and k not in self.allowed_keys:
                raise Exception("Unknown cleaning parameter %s" % k)

        objs = sparse_objects_group["sparse_objects"]
        objs = [objs] if isinstance(objs, BlockSparseMatrix) else list(objs)
        sparse_objects_group["sparse_objects"] = objs
        for p in objs:
            if not isinstance(p, BlockSparseMatrix):
                raise Exception("I don't know how to clean this type of object: %s" % p)

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

        known = set()
        for group in self.param_groups:
            known.update(group["sparse_objects"])
        if not known.isdisjoint(objs):
            raise ValueError("some parameters appear in more than one parameter group")
        self.param_groups.append(sparse_objects_group)

    def clean(self, p, method, clean_ratio, new_coefficients_scale, new_coefficients_distribution):
        if not isinstance(p, BlockSparseMatrix):
            raise Exception("I don't know how to clean this : %s" % p)
        if method != "magnitude":
            raise Exception(f"Unknowncleaning method {method}")
        strategy = MagnitudeSparseOptimizerStrategy(
            clean_ratio,
            new_coefficients_distribution=new_coefficients_distribution,
            new_coefficients_scale=new_coefficients_scale,
        )
        keep = strategy.run(p)

        if self.attached_optimizers:
            found = False
            for optimizer in self.attached_optimizers:
                if not AdamOptimizerStateUpdater.is_compatible(optimizer):
                    raise Exception(f"unsupported optimizer {optimizer.__class__}")
                found = AdamOptimizerStateUpdater(optimizer, p).update_state(keep) or found
            if not found:
                raise Exception(f"Could not find sparse object {p} in optimizers {self.attached_optimizers}")

    def step(self):
        for group in self.param_groups:
            ratio = group["lr"]
            if ratio == 0.0:
                continue
            for p in group["sparse_objects"]:
                self.clean(
                    p,
                    clean_ratio=ratio,
                    method=group["method"],
                    new_coefficients_scale=group["new_coefficients_scale"],
                    new_coefficients_distribution=group["new_coefficients_distribution"],
                )
