"""Fused gated activation y = up * act(gate), `up, gate = x.chunk(2, -1)`, act = SiLU or tanh-GELU.

Mirrors the reference's `novadit/ops/gate_act.py` (autograd Functions :32-71, public functions
:76-102); no PyTorch fallback.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import require_cuda_extension


def geglu_ref(z):
    """PyTorch definition, reference novadit/ops/gate_act.py:9-12."""
    z_up, z_gate = z.chunk(2, dim=-1)
    return z_up * F.gelu(z_gate, approximate="tanh")


def gate_act_ref(x, activation: str = "silu"):
    """PyTorch definition, reference novadit/ops/gate_act.py:15-27."""
    x_up, x_gate = x.chunk(2, dim=-1)
    if activation == "silu":
        return x_up * F.silu(x_gate)
    if activation == "gelu":
        return geglu_ref(x)
    raise ValueError(f"Unsupported activation: {activation}")


class _FusedGateActFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, act_id):
        ext = require_cuda_extension("fused_gate_act", x, "gate_act_ref")
        y = ext.fused_gate_act_forward(x, act_id)
        ctx.save_for_backward(x)
        ctx.act_id = act_id
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = require_cuda_extension("fused_gate_act", dy, "gate_act_ref")
        (x,) = ctx.saved_tensors
        return ext.fused_gate_act_backward(dy, x, ctx.act_id), None


class _FusedGeGLUFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z):
        ext = require_cuda_extension("fused_geglu", z, "geglu_ref")
        y = ext.fused_geglu_forward(z)
        ctx.save_for_backward(z)
        return y

    @staticmethod
    def backward(ctx, dy):
        ext = require_cuda_extension("fused_geglu", dy, "geglu_ref")
        (z,) = ctx.saved_tensors
        return ext.fused_geglu_backward(dy, z)


def fused_geglu(z):
    """z [B,S,2I] -> [B,S,I] = z_up * gelu_tanh(z_gate). Differentiable."""
    require_cuda_extension("fused_geglu", z, "geglu_ref")
    return _FusedGeGLUFunction.apply(z)


def fused_gate_act(x, activation: str = "silu"):
    if activation not in {"silu", "gelu"}:
        raise ValueError(f"Unsupported activation: {activation}")
    require_cuda_extension("fused_gate_act", x, "gate_act_ref")
    return _FusedGateActFunction.apply(x, 0 if activation == "silu" else 1)
