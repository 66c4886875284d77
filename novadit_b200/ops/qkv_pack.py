"""QKV pack, [B,S,3*h*d] -> q, k, v [B,S,h,d]: mirror of `novadit/ops/qkv_pack.py:9-44`.

The reference routes CUDA tensors to `novadit_cuda.fused_qkv_pack_forward`, which raises there
(`csrc/ops/qkv_pack_kernel.cu:5-10`); here one kernel reads each qkv row once and writes the three contiguous
outputs, and its inverse serves as the backward.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import require_cuda_extension


def qkv_pack_ref(qkv, num_heads: int, head_dim: int):
    """PyTorch definition, reference novadit/ops/qkv_pack.py:9-23."""
    bsz, seq_len, three_hidden = qkv.shape
    hidden = num_heads * head_dim
    if three_hidden != 3 * hidden:
        raise ValueError(f"Expected last dim {3 * hidden}, got {three_hidden}")
    view = qkv.view(bsz, seq_len, 3, num_heads, head_dim)
    return view[:, :, 0].contiguous(), view[:, :, 1].contiguous(), view[:, :, 2].contiguous()


class _FusedQkvPackFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, num_heads, head_dim):
        ext = require_cuda_extension("fused_qkv_pack", qkv, "qkv_pack_ref")
        q, k, v = ext.fused_qkv_pack_forward(qkv, num_heads, head_dim)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        ext = require_cuda_extension("fused_qkv_pack", dq, "qkv_pack_ref")
        return ext.fused_qkv_pack_backward(dq, dk, dv), None, None


def fused_qkv_pack(qkv, num_heads: int, head_dim: int):
    if qkv.dim() != 3 or qkv.shape[-1] != 3 * num_heads * head_dim:
        raise ValueError(f"Expected last dim {3 * num_heads * head_dim}, got {tuple(qkv.shape)}")
    require_cuda_extension("fused_qkv_pack", qkv, "qkv_pack_ref")
    return _FusedQkvPackFunction.apply(qkv, num_heads, head_dim)


def fused_qkv_linear_pack(x, weight, bias, num_heads: int, head_dim: int):
    """reference novadit/ops/qkv_pack.py:36-44."""
    return fused_qkv_pack(F.linear(x, weight, bias), num_heads=num_heads, head_dim=head_dim)
