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


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(2, 8, 16), (3, 77, 1152), (1, 1, 8), (2, 5, 770), (4, 256, 1152)])
def test_gated_residual_forward_backward(dtype, shape):
    gen = torch.Generator().manual_seed(5)
    b, s, h = shape
    x = torch.randn(shape, generator=gen).to(dtype)
    br = torch.randn(shape, generator=gen).to(dtype)
    gate = (torch.randn(b, h, generator=gen) * 0.5).to(dtype)
    dy = torch.randn(shape, generator=gen).to(dtype)
    xd, bd, gd = (t.to(DEV).requires_grad_(True) for t in (x, br, gate))
    y = ops.fused_gated_residual(xd, bd, gd)
    dx, dbr, dgate = torch.autograd.grad(y, (xd, bd, gd), dy.to(DEV))
    x64, b64, g64 = (t.double().requires_grad_(True) for t in (x, br, gate))
    want = ops.gated_residual_ref(x64, b64, g64)
    wdx, wdbr, wdg = torch.autograd.grad(want, (x64, b64, g64), dy.double())
    tol = 1e-6 if dtype == torch.float32 else HALF_REL_L2
    assert rel_l2(y, want) < tol and rel_l2(dbr, wdbr) < tol and rel_l2(dgate, wdg) < tol
    assert torch.equal(dx.cpu(), dy)
    if dtype != torch.float32:  # one rounding of the fp32 result
        half_ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
        err = (y.detach().cpu().double() - want.detach()).abs()
        assert bool((err <= half_ulp * want.detach().abs() * 1.001 + 1e-7).all())


def test_gated_residual_row_shard():
    from novadit_b200 import capi

    gen = torch.Generator().manual_seed(6)
    b, s, h = 3, 50, 256
    x, br, dy = (torch.randn(b, s, h, generator=gen).to(DEV, torch.bfloat16) for _ in range(3))
    gate = torch.randn(b, h, generator=gen).to(DEV, torch.bfloat16)
    full = capi.gated_residual_fwd(x, br, gate)
    dbr_full, part_full = capi.gated_residual_bwd(dy, br, gate)
    lo, hi = 37, 121
    sl = lambda t: t.reshape(-1, h)[lo:hi].contiguous()  # noqa: E731
    y = capi.gated_residual_fwd(sl(x), sl(br), gate, row_start=lo, seq_len=s)
    dbr, part = capi.gated_residual_bwd(sl(dy), sl(br), gate, row_start=lo, seq_len=s)
    assert torch.equal(y, sl(full)) and torch.equal(dbr, sl(dbr_full))
    # the shard touches samples 0..2; the middle sample is complete inside it
    assert torch.equal(part[1 - lo // s], part_full[1])
