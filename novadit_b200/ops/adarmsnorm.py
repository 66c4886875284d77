"""Fused AdaRMSNorm: y = x / sqrt(mean(x^2) + eps) * (1 + scale) + shift.

Mirrors the reference's `novadit/ops/adarmsnorm.py` (autograd Function :8-47, public functions
:72-94); no PyTorch fallback, one-pass backward when every input needs a gradient.
"""
from __future__ import annotations

import torch

from . import require_cuda_extension
from .adaln import _broadcast_modulation


class _FusedAdaRMSNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, shift, eps):
        ext = require_cuda_extension("fused_adarmsnorm", x, "adarmsnorm_ref")
        y, scale_contig, inv_rms = ext.fused_adarmsnorm_forward(x, scale, shift, eps)
        ctx.save_for_backward(x, scale_contig, inv_rms)
        ctx.scale_shape = scale.shape
        ctx.shift_shape = shift.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = require_cuda_extension("fused_adarmsnorm", dy, "adarmsnorm_ref")
        x, scale, inv_rms = ctx.saved_tensors
        dy = dy.contiguous()
        need_dx = ctx.needs_input_grad[0]
        need_dp = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
        dx = dscale = dshift = None
        if need_dx and need_dp:
            dx, dscale, dshift = ext.fused_adarmsnorm_backward(dy, x, scale, inv_rms)
        elif need_dx:
            dx = ext.fused_adarmsnorm_backward_dx(dy, x, scale, inv_rms)
        elif need_dp:
            dscale, dshift = ext.fused_adarmsnorm_backward_dparam(dy, x, inv_rms)
        dscale = dscale.reshape(ctx.scale_shape) if ctx.needs_input_grad[1] else None
        dshift = dshift.reshape(ctx.shift_shape) if ctx.needs_input_grad[2] else None
        return dx, dscale, dshift, None


def adarmsnorm_ref(x, scale, shift, eps: float = 1e-5):
    """PyTorch definition; same function as the reference's `adarmsnorm_ref`,
    novadit/ops/adarmsnorm.py:56-69. Never called by the fused path."""
    xf = x.float()
    rms = torch.sqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    y = (xf / rms) * (1.0 + _broadcast_modulation(x, scale).float()) + _broadcast_modulation(x, shift).float()
    return y.to(dtype=x.dtype)


def fused_adarmsnorm(x, scale, shift, eps: float = 1e-5):
    require_cuda_extension("fused_adarmsnorm", x, "adarmsnorm_ref")
    return _FusedAdaRMSNormFunction.apply(x, scale, shift, eps)


@torch.no_grad()
def fused_adarmsnorm_inference(x, scale, shift, eps: float = 1e-5):
    ext = require_cuda_extension("fused_adarmsnorm_inference", x, "adarmsnorm_ref")
    return ext.fused_adarmsnorm_forward_inference(x, scale, shift, eps)
