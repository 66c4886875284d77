"""Names the reference's `novadit.ops` exports that lie OUTSIDE the accelerated operator path.

They exist so that code written against the reference's package imports unchanged. The QKV
pack and the residual add are plain PyTorch here (the reference's native side for them is a stub
that raises: csrc/ops/qkv_pack_kernel.cu:5-10, csrc/ops/residual_kernel.cu:3-8), and the two
`torch.compile` comparison baselines of novadit/ops/norm_compile.py are not provided.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def qkv_pack_ref(qkv, num_heads: int, head_dim: int):
    """[B,S,3*h*d] -> q, k, v [B,S,h,d] (reference novadit/ops/qkv_pack.py:9-23)."""
    bsz, seq_len, three_hidden = qkv.shape
    hidden = num_heads * head_dim
    if three_hidden != 3 * hidden:
        raise ValueError(f"Expected last dim {3 * hidden}, got {three_hidden}")
    view = qkv.view(bsz, seq_len, 3, num_heads, head_dim)
    return view[:, :, 0].contiguous(), view[:, :, 1].contiguous(), view[:, :, 2].contiguous()


def fused_qkv_pack(qkv, num_heads: int, head_dim: int):
    return qkv_pack_ref(qkv, num_heads, head_dim)


def fused_qkv_linear_pack(x, weight, bias, num_heads: int, head_dim: int):
    return fused_qkv_pack(F.linear(x, weight, bias), num_heads=num_heads, head_dim=head_dim)


def out_residual_ref(x, residual, bias=None):
    """x + residual (+ bias) (reference novadit/ops/residual.py:8-15)."""
    if bias is not None:
        return x + residual + bias.view(1, 1, -1)
    return x + residual


def fused_out_residual(x, residual, bias=None):
    return out_residual_ref(x, residual, bias)


def adaln_compile(*args, **kwargs):
    raise NotImplementedError("the torch.compile comparison baseline is not part of this library; use fused_adaln")


def adarmsnorm_compile(*args, **kwargs):
    raise NotImplementedError("the torch.compile comparison baseline is not part of this library; use fused_adarmsnorm")
