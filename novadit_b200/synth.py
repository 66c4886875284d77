"""Seeded synthetic inputs for the operator workloads.

Every tensor is drawn on the CPU in fp32 from one `torch.Generator` in a fixed
order and then cast, so the CPU checker and the GPU kernels always see the
same bits. The distributions are the ones the workload statements give:
activations and upstream gradients ~ N(0,1), modulation vectors ~ N(0,0.1),
FC1 weight and bias ~ N(0,0.02).
"""
from __future__ import annotations

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def norm_inputs(batch, seq, hidden, dtype=torch.bfloat16, seed=0, mod_std=0.1):
    """x, scale, shift, dy for AdaLN / AdaRMSNorm: x,dy [B,S,H] ~ N(0,1); scale,shift [B,H] ~ N(0,mod_std)."""
    g = _gen(seed)
    x = torch.randn(batch, seq, hidden, generator=g, dtype=torch.float32)
    scale = torch.randn(batch, hidden, generator=g, dtype=torch.float32) * mod_std
    shift = torch.randn(batch, hidden, generator=g, dtype=torch.float32) * mod_std
    dy = torch.randn(batch, seq, hidden, generator=g, dtype=torch.float32)
    return x.to(dtype), scale.to(dtype), shift.to(dtype), dy.to(dtype)


def gate_act_inputs(batch, seq, inter, dtype=torch.bfloat16, seed=0):
    """x [B,S,2I] ~ N(0,1), dy [B,S,I] ~ N(0,1)."""
    g = _gen(seed)
    x = torch.randn(batch, seq, 2 * inter, generator=g, dtype=torch.float32)
    dy = torch.randn(batch, seq, inter, generator=g, dtype=torch.float32)
    return x.to(dtype), dy.to(dtype)


def fc1_inputs(m, k, n, dtype=torch.bfloat16, seed=0):
    """X [M,K] ~ N(0,1), W [N,K] ~ N(0,0.02) (nn.Linear layout), bias [N] ~ N(0,0.02)."""
    g = _gen(seed)
    x = torch.randn(m, k, generator=g, dtype=torch.float32)
    w = torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02
    b = torch.randn(n, generator=g, dtype=torch.float32) * 0.02
    return x.to(dtype), w.to(dtype), b.to(dtype)
