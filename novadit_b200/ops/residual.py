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


def gated_residual_ref(x, branch, gate):
    """y = x + gate[:, None, :] * branch (the adaLN-Zero residual of DiT blocks; not an operator of the reference)."""
    return x + gate.unsqueeze(1) * branch


class _FusedGatedResidualFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, branch, gate):
        from .. import capi

        require_cuda_extension("fused_gated_residual", x, "gated_residual_ref")
        branch, gate = branch.contiguous(), gate.contiguous()
        ctx.save_for_backward(branch, gate)
        return capi.gated_residual_fwd(x.contiguous(), branch, gate)

    @staticmethod
    def backward(ctx, dy):
        from .. import capi

        branch, gate = ctx.saved_tensors
        dbranch, part = capi.gated_residual_bwd(dy.contiguous(), branch, gate)
        return dy, dbranch, part.sum(dim=1).to(gate.dtype)


def fused_gated_residual(x, branch, gate):
    """x, branch [B,S,H], gate [B,H] (CUDA, one dtype of fp32 / fp16 / bf16); differentiable in all three."""
    require_cuda_extension("fused_gated_residual", x, "gated_residual_ref")
    return _FusedGatedResidualFunction.apply(x, branch, gate)
