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
        ext = require_cuda_extension("fused_gated_residual", x, "gated_residual_ref")
        branch, gate = branch.contiguous(), gate.contiguous()
        ctx.save_for_backward(branch, gate)
        return ext.fused_gated_residual_forward(x.contiguous(), branch, gate)

    @staticmethod
    def backward(ctx, dy):
        ext = require_cuda_extension("fused_gated_residual", dy, "gated_residual_ref")
        branch, gate = ctx.saved_tensors
        _, dbranch, dgate = ext.fused_gated_residual_backward(dy.contiguous(), None, branch, gate)
        return dy, dbranch, dgate.to(gate.dtype)


def fused_gated_residual(x, branch, gate):
    """x, branch [B,S,H], gate [B,H] (CUDA, one dtype of fp32 / fp16 / bf16); differentiable in all three."""
    require_cuda_extension("fused_gated_residual", x, "gated_residual_ref")
    return _FusedGatedResidualFunction.apply(x, branch, gate)


def residual_adaln_ref(x, branch, gate, scale, shift, eps: float = 1e-5):
    """PyTorch definition of the fused residual + AdaLN: (x_new, y) with x_new = x + gate * branch (gate None: x +
    branch) in x's dtype and y = adaln_ref(x_new, scale, shift, eps)."""
    from .adaln import adaln_ref

    x_new = gated_residual_ref(x, branch, gate) if gate is not None else x + branch
    return x_new, adaln_ref(x_new, scale, shift, eps)


def residual_adarmsnorm_ref(x, branch, gate, scale, shift, eps: float = 1e-5):
    from .adarmsnorm import adarmsnorm_ref

    x_new = gated_residual_ref(x, branch, gate) if gate is not None else x + branch
    return x_new, adarmsnorm_ref(x_new, scale, shift, eps)


class _FusedResidualNormFunction(torch.autograd.Function):
    """(x, branch, gate, scale, shift) -> (x_new, y): the gated residual of a block and the AdaLN / AdaRMSNorm of the
    next branch in ONE forward kernel. Backward: the one-pass norm backward on x_new, then one kernel that adds the
    gradient arriving along the residual stream, scales it by the gate for the branch and sums dgate."""

    @staticmethod
    def forward(ctx, x, branch, gate, scale, shift, eps, rms):
        ext = require_cuda_extension("fused_residual_adaln", x, "residual_adaln_ref")
        fwd = ext.fused_residual_adarmsnorm_forward if rms else ext.fused_residual_adaln_forward
        gate_c = gate.contiguous() if gate is not None else None
        branch_c = branch.contiguous()
        out = fwd(x.contiguous(), branch_c, gate_c, scale, shift, eps)
        x_new, y, scale_c = out[0], out[1], out[2]
        ctx.rms, ctx.has_gate = rms, gate is not None
        ctx.scale_shape, ctx.shift_shape = scale.shape, shift.shape
        ctx.save_for_backward(x_new, branch_c, gate_c if gate is not None else scale_c, scale_c, *out[3:])
        return x_new, y

    @staticmethod
    def backward(ctx, d_xnew, dy):
        ext = require_cuda_extension("fused_residual_adaln", dy, "residual_adaln_ref")
        x_new, branch, gate, scale_c, *stats = ctx.saved_tensors
        dy = dy.contiguous()
        if ctx.rms:
            dx_n, dscale, dshift = ext.fused_adarmsnorm_backward(dy, x_new, scale_c, stats[0])
        else:
            dx_n, dscale, dshift = ext.fused_adaln_backward(dy, x_new, scale_c, stats[0], stats[1])
        if ctx.has_gate:
            dsum, dbranch, dgate = ext.fused_gated_residual_backward(dx_n, d_xnew.contiguous(), branch, gate)
            dgate = dgate.to(gate.dtype)
        else:
            dsum = dx_n + d_xnew
            dbranch, dgate = dsum, None
        return (dsum, dbranch, dgate, dscale.to(scale_c.dtype).reshape(ctx.scale_shape),
                dshift.to(scale_c.dtype).reshape(ctx.shift_shape), None, None)


def fused_residual_adaln(x, branch, gate, scale, shift, eps: float = 1e-5):
    """(x_new, y): x_new = x + gate[b] * branch (gate [B, H]; None: x + branch), y = AdaLN(x_new) * (1 + scale) + shift.
    One pass over x and branch instead of a residual kernel and a norm kernel; differentiable in all five tensors.
    The operators are the reference's (`novadit/ops/residual.py:8-25`, `novadit/ops/adaln.py:56-80`); the fusion has
    no counterpart there."""
    require_cuda_extension("fused_residual_adaln", x, "residual_adaln_ref")
    return _FusedResidualNormFunction.apply(x, branch, gate, scale, shift, eps, False)


def fused_residual_adarmsnorm(x, branch, gate, scale, shift, eps: float = 1e-5):
    """AdaRMSNorm counterpart of `fused_residual_adaln`."""
    require_cuda_extension("fused_residual_adarmsnorm", x, "residual_adarmsnorm_ref")
    return _FusedResidualNormFunction.apply(x, branch, gate, scale, shift, eps, True)
