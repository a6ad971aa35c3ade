"""Drop-in ``nn.Linear`` with a block-sparse weight and its autograd function.

Mirrors ``pytorch_block_sparse/block_sparse_linear.py`` of the reference: same constructor
arguments, same initialisation rules, same three contractions per layer --

* forward ``y = x @ W.T + b``      (reference ``block_sparse_linear.py:40``, ``:229-233``)
* dgrad   ``dx = dy @ W``           (``:80``)
* wgrad   ``dW = dy.T @ x`` at W's non-zero blocks, in ``data`` layout (``:123``)

-- each served by a CUDA kernel behind the C-ABI.  Differences, all invisible in values:
the bias is added in the forward kernel's epilogue instead of a separate elementwise pass,
dgrad no longer copies the weights transposed per call, and the reference's
``assert not (grad == 0).all()`` device->host sync after wgrad is not kept.
"""
import math
from typing import Tuple

import torch
import torch.autograd
import torch.nn as nn

from . import native
from .block_sparse import BlockSparseMatrix, BlockSparseMatrixBase, BlockSparseMatrixEmulator


class BlockSparseLinearFunction(torch.autograd.Function):
    """``apply(input, weight_data, weight[, bias[, residual[, activation]]])``.

    ``weight_data`` is ``weight.get_differentiable_data()`` passed separately so that the
    Parameter receives the gradient (reference ``block_sparse_linear.py:15-53``, ``:154``).
    The optional arguments are fused into the forward kernel's epilogue:
    ``y = act(x @ W.T + bias + residual)`` with ``activation`` ``None`` or ``"gelu"`` (erf form).
    With an activation the kernel also writes the pre-activation sum, which backward needs.
    """

    @staticmethod
    def forward(ctx, input, weight_data, weight, *extras):
        assert isinstance(weight, BlockSparseMatrixBase)
        bias = extras[0] if len(extras) > 0 else None
        residual = extras[1] if len(extras) > 1 else None
        activation = extras[2] if len(extras) > 2 else None
        ctx.weight = weight
        ctx.n_extra = len(extras)
        ctx.has_bias = bias is not None
        ctx.has_residual = residual is not None
        ctx.activation = activation
        # The weights are packed once per forward -- never from a cache keyed on autograd's version counter,
        # which writes through ``.data`` do not bump -- and backward reuses these images, i.e. the weights
        # the forward saw.
        ctx.packed = weight.packed_weights() if isinstance(weight, BlockSparseMatrix) else None
        fused = residual is not None or activation is not None
        if not fused:
            ctx.save_for_backward(input, weight_data)
            return weight.reverse_matmul(input, transpose=True, bias=bias, packed=ctx.packed)
        if not (isinstance(weight, BlockSparseMatrix) and ctx.packed.images is not None):
            # emulated block shapes and the exact-fp32 CUDA-core precision have no fused epilogue
            pre = weight.reverse_matmul(input, transpose=True, bias=bias, packed=ctx.packed)
            if residual is not None:
                pre = pre + residual
            out = torch.nn.functional.gelu(pre) if activation == "gelu" else pre
        else:
            # needs_input_grad reports the inputs' requires_grad flags even when no graph is being recorded (and
            # the grad mode cannot be asked here: it is always off inside forward); the layer's forward therefore
            # takes the inference path itself when gradients are disabled
            need_pre = activation is not None and any(ctx.needs_input_grad)
            out, pre = weight.reverse_matmul_fused(
                input, bias=bias, residual=residual, activation=activation, packed=ctx.packed, keep_pre=need_pre
            )
        ctx.save_for_backward(input, weight_data, pre if activation is not None else None)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        saved = ctx.saved_tensors
        input = saved[0]
        weight = ctx.weight
        if ctx.activation == "gelu":
            grad_output = torch.ops.aten.gelu_backward(grad_output.contiguous(), saved[2].view_as(grad_output))
        grad_input = grad_weight = grad_bias = grad_residual = None
        # the weight gradient first: in data-parallel training its all-reduce can then overlap the input gradient
        if ctx.needs_input_grad[1]:
            grad_weight = weight.matmul_with_output_sparse_support(grad_output, input)
        if ctx.needs_input_grad[0]:
            grad_input = weight.reverse_matmul(grad_output, transpose=False, packed=ctx.packed)
            assert grad_input.shape == input.shape
        if ctx.has_bias and ctx.needs_input_grad[3]:
            grad_bias = grad_output.reshape(-1, grad_output.shape[-1]).sum(0, dtype=torch.float32)
        if ctx.has_residual and ctx.needs_input_grad[4]:
            grad_residual = grad_output
        return (grad_input, grad_weight, None, grad_bias, grad_residual, None)[: 3 + ctx.n_extra]


class BlockSparseLinear(nn.Module):
    """Block-sparse replacement of ``torch.nn.Linear`` (reference ``block_sparse_linear.py:157-233``).

    ``density`` fixes the block count as ``int(density * in * out / (bh * bw))``.  Built from
    ``torch_nn_linear`` it takes that layer's sizes and bias, fills ``data`` through
    ``from_dense`` and rescales by ``1/sqrt(density)``.  Square blocks of 32, 64, 96, 128 ... run on the
    tensor-core kernels; other block shapes use the dense-masked emulator class (the reference sends
    everything but 32x32 there).  Parameters live on ``"cuda"``.
    """

    OPTIMIZED_BLOCK_SIZE = 32

    def __init__(
        self,
        in_features: int,
        out_features: int,
        bias: bool = True,
        density: float = 0.5,
        torch_nn_linear=None,
        verbose: bool = False,
        block_shape: Tuple[int, int] = (32, 32),
        activation=None,
    ):
        super().__init__()
        self.fn = BlockSparseLinearFunction.apply
        self.verbose = verbose
        self.block_shape = block_shape
        if activation not in (None, "gelu"):
            raise Exception(f"BlockSparseLinear invalid activation={activation}, expected None or 'gelu'")
        self.activation = activation  # not in the reference: applied inside the forward kernel's epilogue
        # 32x32 blocks and larger square multiples of 32 run on the CUDA kernels (the latter through their
        # 32x32 expansion); every other block shape uses the dense-masked emulator, as in the reference
        self._optimized = (
            block_shape[0] == block_shape[1] and block_shape[0] % self.OPTIMIZED_BLOCK_SIZE == 0 and block_shape[0] > 0
        )

        if torch_nn_linear is not None:
            in_features = torch_nn_linear.in_features
            out_features = torch_nn_linear.out_features
            bias = torch_nn_linear.bias is not None

        if in_features % block_shape[1] != 0:
            raise Exception(f"BlockSparseLinear invalid in_features={in_features}, should be multiple of {block_shape[1]}")
        if out_features % block_shape[0] != 0:
            raise Exception(f"BlockSparseLinear invalid in_features={in_features}, should be multiple of {block_shape[0]}")
        if density < 0 or density > 1:
            raise Exception(f"BlockSparseLinear invalid density={density}")

        self.block_count = int(density * (in_features * out_features / (block_shape[0] * block_shape[1])))
        self.in_features = in_features
        self.out_features = out_features

        matrix_cls = BlockSparseMatrix if self._optimized else BlockSparseMatrixEmulator
        if torch_nn_linear is not None:
            with torch.no_grad():
                weight = matrix_cls.from_dense(torch_nn_linear.weight.to("cuda"), block_shape, self.block_count)
            weight.multiply_(1.0 / math.sqrt(density))
        else:
            weight = matrix_cls.randn(
                (out_features, in_features), self.block_count, blocks=None, block_shape=block_shape, device="cuda"
            )
        self.weight = weight

        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, device="cuda"))
            if torch_nn_linear is not None:
                with torch.no_grad():
                    self.bias.copy_(torch_nn_linear.bias)
        else:
            self.register_parameter("bias", None)

    def forward(self, x, residual=None):
        """``act(x @ W.T + bias + residual)``; ``residual`` (not in the reference) has the output's shape and is
        added in the kernel's epilogue, like the bias and the layer's ``activation``."""
        if self._optimized:
            if residual is None and self.activation is None:
                return self.fn(x, self.weight.get_differentiable_data(), self.weight, self.bias)
            if (not torch.is_grad_enabled() and isinstance(self.weight, BlockSparseMatrix)
                    and native.resolve_precision(None) != native.PREC_FP32_SIMT):
                # inference: no pre-activation tensor is kept (and bf16 tensors stay bf16)
                return self.weight.reverse_matmul_fused(x, bias=self.bias, residual=residual, activation=self.activation)[0]
            return self.fn(x, self.weight.get_differentiable_data(), self.weight, self.bias, residual, self.activation)
        x = self.fn(x, self.weight.get_differentiable_data(), self.weight)
        if self.bias is not None:
            x = x + self.bias
        if residual is not None:
            x = x + residual
        return torch.nn.functional.gelu(x) if self.activation == "gelu" else x

    def extra_repr(self):
        return "in_features={}, out_features={}, bias={}, block_count={}".format(
            self.in_features, self.out_features, self.bias is not None, self.block_count
        )


class PseudoBlockSparseLinear(torch.nn.Module):
    """Pure-torch twin of a :class:`BlockSparseLinear` for debugging (reference ``block_sparse_linear.py:236-262``)."""

    def __init__(self, block_sparse_linear):
        super().__init__()
        matrix = block_sparse_linear.weight.cuda()
        self.weight = torch.nn.Parameter(matrix.to_dense())
        mask = matrix.to_dense(data_replace=torch.ones_like(matrix.data)) == 1
        if block_sparse_linear.bias is not None:
            self.bias = torch.nn.Parameter(block_sparse_linear.bias)
        else:
            self.register_parameter("bias", None)
        self.register_buffer("mask", mask)
        self.in_features = block_sparse_linear.in_features
        self.out_features = block_sparse_linear.out_features
        self.density = mask.sum().item() / (mask.shape[0] * mask.shape[1])

    def forward(self, input):
        return torch.nn.functional.linear(input, self.weight * self.mask, self.bias)

    def extra_repr(self):
        return "in_features={}, out_features={}, bias={}, fill_ratio={}".format(
            self.in_features, self.out_features, self.bias is not None, self.density
        )
