"""Output residual add and QKV pack: kernels against the reference's PyTorch definitions."""
from __future__ import annotations

import pytest
import torch

import novadit_b200.ops as ops
from tests.helpers import HALF_REL_L2

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_l2(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(2, 8, 16), (3, 77, 1152), (1, 1, 8), (2, 5, 770), (4, 300, 4608)])
@pytest.mark.parametrize("with_bias", [True, False])
def test_out_residual(dtype, shape, with_bias):
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(shape, generator=gen).to(dtype)
    r = torch.randn(shape, generator=gen).to(dtype)
    b = torch.randn(shape[-1], generator=gen).to(dtype) if with_bias else None
    y = ops.fused_out_residual(x.to(DEV), r.to(DEV), None if b is None else b.to(DEV))
    want = x.double() + r.double() + (0 if b is None else b.double().view(1, 1, -1))  # exact sum, rounded once below
    assert y.shape == x.shape and y.dtype == dtype and y.is_contiguous()
    if dtype == torch.float32:
        assert rel_l2(y, want) < 1e-6
    else:
        # one rounding of the (exact in fp32) sum: within half a unit in the last place of the exact value
        half_ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11  # relative to the value, at most
        err = (y.cpu().double() - want).abs()
        assert bool((err <= half_ulp * want.abs() * 1.001 + 1e-7).all()) and rel_l2(y, want) < HALF_REL_L2
        # ... so at least as close to the exact sum as the reference's two roundings
        ref = ops.out_residual_ref(x, r, b)
        assert rel_l2(y, want) <= rel_l2(ref, want) + 1e-9


def test_out_residual_autograd():
    gen = torch.Generator().manual_seed(2)
    x, r = (torch.randn(2, 9, 64, generator=gen).to(DEV, torch.bfloat16).requires_grad_(True) for _ in range(2))
    b = torch.randn(64, generator=gen).to(DEV, torch.bfloat16).requires_grad_(True)
    dy = torch.randn(2, 9, 64, generator=gen).to(DEV, torch.bfloat16)
    got = torch.autograd.grad(ops.fused_out_residual(x, r, b), (x, r, b), dy)
    want = torch.autograd.grad(ops.out_residual_ref(x, r, b), (x, r, b), dy)
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    assert rel_l2(got[2], want[2]) < 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("b,s,heads,hd", [(2, 8, 2, 8), (3, 77, 16, 72), (1, 1, 1, 4), (2, 5, 5, 7), (4, 256, 16, 72)])
def test_qkv_pack_is_exact_and_contiguous(dtype, b, s, heads, hd):
    gen = torch.Generator().manual_seed(3)
    qkv = torch.randn(b, s, 3 * heads * hd, generator=gen).to(dtype)
    got = ops.fused_qkv_pack(qkv.to(DEV), heads, hd)
    want = ops.qkv_pack_ref(qkv, heads, hd)
    for g, w in zip(got, want):
        assert g.shape == (b, s, heads, hd) and g.is_contiguous()
        assert torch.equal(g.cpu(), w)
    # the backward is the inverse gather
    qd = qkv.to(DEV).requires_grad_(True)
    q, k, v = ops.fused_qkv_pack(qd, heads, hd)
    gq, gk, gv = (torch.randn(q.shape, generator=gen).to(DEV, dtype) for _ in range(3))
    (dqkv,) = torch.autograd.grad((q, k, v), (qd,), (gq, gk, gv))
    assert torch.equal(dqkv, torch.cat([gq.reshape(b, s, -1), gk.reshape(b, s, -1), gv.reshape(b, s, -1)], dim=-1))


def test_shape_errors_like_the_reference():
    with pytest.raises(ValueError, match="Expected last dim"):
        ops.fused_qkv_pack(torch.zeros(2, 4, 50, device=DEV), 2, 8)
    with pytest.raises(RuntimeError):
        ops.fused_out_residual(torch.zeros(2, 4, 8), torch.zeros(2, 4, 8))  # CPU tensors: no fallback
