"""Output residual add, y = x + residual (+ bias): mirror of `novadit/ops/residual.py:8-25`.

The reference routes CUDA tensors to `novadit_cuda.fused_out_residual_forward`, which raises there
(`csrc/ops/residual_kernel.cu:3-8`); here the kernel exists (one pass, fp32 sum, one rounding) and the function is
differentiable: dx = dresidual = dy, dbias = sum of dy over batch and sequence.
"""
from __future__ import annotations

import torch

from . import require_cuda_extension


def out_residual_ref(x, residual, bias=None):
    """PyTorch definition, reference novadit/ops/residual.py:8-15."""
    if bias is not None:
        return x + residual + bias.view(1, 1, -1)
    return x + residual


class _FusedOutResidualFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, bias):
        ext = require_cuda_extension("fused_out_residual", x, "out_residual_ref")
        ctx.has_bias = bias is not None
        return ext.fused_out_residual_forward(x, residual, bias)

    @staticmethod
    def backward(ctx, dy):
        d_bias = dy.sum(dim=(0, 1)) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return (dy if ctx.needs_input_grad[0] else None, dy if ctx.needs_input_grad[1] else None, d_bias)


def fused_out_residual(x, residual, bias=None):
    """x, residual [B,S,H] (CUDA, one dtype of fp32 / fp16 / bf16), bias [H] or None."""
    require_cuda_extension("fused_out_residual", x, "out_residual_ref")
    return _FusedOutResidualFunction.apply(x, residual, bias)
