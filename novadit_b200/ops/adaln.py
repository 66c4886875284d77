"""Fused AdaLN: y = LayerNorm(x) * (1 + scale) + shift, per-sample modulation, no affine.

Mirrors the reference's `novadit/ops/adaln.py` (public functions :72-121, autograd Function
:8-47). Differences: the fused functions never fall back to PyTorch, and when x, scale and
shift all need gradients the backward runs ONE kernel that produces dx and the fp32
dscale/dshift in a single pass over dy and x instead of two kernels.
"""
from __future__ import annotations

import torch

from . import require_cuda_extension


class _FusedAdaLNFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, shift, eps):
        ext = require_cuda_extension("fused_adaln", x, "adaln_ref")
        y, scale_contig, mean, invstd = ext.fused_adaln_forward(x, scale, shift, eps)
        ctx.save_for_backward(x, scale_contig, mean, invstd)
        ctx.scale_shape = scale.shape
        ctx.shift_shape = shift.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = require_cuda_extension("fused_adaln", dy, "adaln_ref")
        x, scale, mean, invstd = ctx.saved_tensors
        dy = dy.contiguous()
        need_dx = ctx.needs_input_grad[0]
        need_dp = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
        dx = dscale = dshift = None
        if need_dx and need_dp:
            dx, dscale, dshift = ext.fused_adaln_backward(dy, x, scale, mean, invstd)
        elif need_dx:
            dx = ext.fused_adaln_backward_dx(dy, x, scale, mean, invstd)
        elif need_dp:
            dscale, dshift = ext.fused_adaln_backward_dparam(dy, x, mean, invstd)
        # fp32 parameter gradients; autograd casts them when accumulating into half-precision leaves
        dscale = dscale.reshape(ctx.scale_shape) if ctx.needs_input_grad[1] else None
        dshift = dshift.reshape(ctx.shift_shape) if ctx.needs_input_grad[2] else None
        return dx, dscale, dshift, None


def _broadcast_modulation(x: torch.Tensor, tensor: torch.Tensor) -> torch.Tensor:
    while tensor.dim() < x.dim():
        tensor = tensor.unsqueeze(1)
    return tensor


def adaln_ref(x, scale, shift, eps: float = 1e-5):
    """PyTorch definition (fp32 inside, result in x.dtype); same function as the reference's
    `adaln_ref`, novadit/ops/adaln.py:56-69. Never called by the fused path."""
    xf = x.float()
    mean = xf.mean(dim=-1, keepdim=True)
    var = xf.var(dim=-1, unbiased=False, keepdim=True)
    xhat = (xf - mean) * torch.rsqrt(var + eps)
    y = xhat * (1.0 + _broadcast_modulation(x, scale).float()) + _broadcast_modulation(x, shift).float()
    return y.to(dtype=x.dtype)


def fused_adaln(x, scale, shift, eps: float = 1e-5):
    """x [B,S,H]; scale, shift [B,H] or [B,1,H]; CUDA fp16/bf16/fp32. Differentiable."""
    require_cuda_extension("fused_adaln", x, "adaln_ref")
    return _FusedAdaLNFunction.apply(x, scale, shift, eps)


@torch.no_grad()
def fused_adaln_inference(x, scale, shift, eps: float = 1e-5):
    """Forward only: returns y and writes no statistics."""
    ext = require_cuda_extension("fused_adaln_inference", x, "adaln_ref")
    return ext.fused_adaln_forward_inference(x, scale, shift, eps)


@torch.no_grad()
def fused_adaln_e4m3(x, scale, shift, eps: float, q_scale, amax=None):
    """Forward only, FP8 e4m3 output for an FP8 consumer (`fused_fc1_bias_act_fp8`-style GEMMs): returns
    q = saturate_e4m3(y / q_scale) with the shape of x. `q_scale` is a 1-element fp32 CUDA tensor (delayed scaling:
    derived from an earlier step's maximum as amax / 448); `amax`, when given, is a 1-element fp32 CUDA tensor that
    receives max(amax, max |y|) of this call. No counterpart in the reference (it has no FP8 path)."""
    ext = require_cuda_extension("fused_adaln_e4m3", x, "adaln_ref")
    return ext.fused_adaln_forward_e4m3(x.contiguous(), scale.contiguous(), shift.contiguous(), eps, q_scale, amax)[0]


def fused_adaln_backward_dx(dy, x, scale, mean, invstd):
    ext = require_cuda_extension("fused_adaln_backward_dx", x, "adaln_ref")
    return ext.fused_adaln_backward_dx(dy, x, scale, mean, invstd)


def fused_adaln_backward_dparam(dy, x, mean, invstd):
    """Returns (dscale, dshift), both [B,H] fp32 whatever the input dtype."""
    ext = require_cuda_extension("fused_adaln_backward_dparam", x, "adaln_ref")
    return tuple(ext.fused_adaln_backward_dparam(dy, x, mean, invstd))
