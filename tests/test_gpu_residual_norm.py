"""The norm forward with the gated residual in front (`nd_adaln_fwd_residual` / `nd_adarms_fwd_residual`) and the
residual backward that adds the stream's gradient (`nd_gated_residual_bwd_add`), through the C ABI and through
`novadit_b200.ops`."""
from __future__ import annotations

import pytest
import torch

import novadit_b200.ops as ops
from novadit_b200 import capi, synth
from oracle import novadit_oracle as oracle
from tests.helpers import assert_half_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(b, s, h, dtype, seed):
    x, scale, shift, dy = synth.norm_inputs(b, s, h, dtype, seed)
    gen = torch.Generator().manual_seed(seed + 100)
    branch = torch.randn(b, s, h, generator=gen).to(dtype)
    gate = (torch.randn(b, h, generator=gen) * 0.5).to(dtype)
    return x, branch, gate, scale, shift, dy


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("use_gate", [True, False])
@pytest.mark.parametrize("shape,dtype", [
    ((32, 256, 1152), torch.bfloat16),   # workload config 2
    ((3, 77, 768), torch.float16),       # ragged groups, several samples per chunk
    ((2, 256, 768), torch.float32),      # workload config 1 on the GPU
    ((5, 9, 770), torch.bfloat16),       # rows not 16-byte vectorisable: the composed path
    ((2, 33, 4104), torch.bfloat16),     # wider than 512 vectors: the composed path
])
def test_one_pass_equals_the_two_kernels_bit_for_bit_and_the_oracle(kind, use_gate, shape, dtype):
    b, s, h = shape
    x, branch, gate, scale, shift, _ = _inputs(b, s, h, dtype, seed=7)
    xd, bd, gd, sd, hd = (t.to(DEV) for t in (x, branch, gate, scale, shift))
    out = capi.norm_fwd_residual(kind, xd, bd, gd if use_gate else None, sd, hd, 1e-6)
    # the composition the fused kernel replaces
    x_new = capi.gated_residual_fwd(xd, bd, gd) if use_gate else ops.fused_out_residual(xd, bd)
    ref = capi.norm_fwd(kind, x_new, sd, hd, 1e-6)
    assert torch.equal(out[0], x_new)
    for got, want in zip(out[1:], ref):
        assert torch.equal(got, want)
    # and the oracle: the residual stream in the input dtype, then the reference's norm of it
    xn = (x.float() + (gate.float()[:, None, :] if use_gate else 1.0) * branch.float()).to(dtype)
    fwd = oracle.adaln_fwd if kind == "layer" else oracle.adarms_fwd
    want_y = fwd(xn, scale, shift, 1e-6)[0]
    if dtype == torch.float32:
        assert oracle.rel_l2(out[1].cpu(), want_y) < 1e-5
    else:
        assert torch.equal(out[0].cpu(), xn)
        exact = fwd(xn, scale, shift, 1e-6, compute=torch.float64, round_out=False)[0]
        assert_half_parity(out[1].cpu(), want_y, f"{kind} y after the residual", exact=exact)


def test_residual_backward_with_the_streams_gradient_added():
    b, s, h = 4, 100, 1152
    x, branch, gate, _, _, dy = _inputs(b, s, h, torch.bfloat16, seed=3)
    dres = torch.roll(dy, 1, 0)
    dyd, drd, bd, gd = (t.to(DEV) for t in (dy, dres, branch, gate))
    dsum, dbranch, part = capi.gated_residual_bwd_add(dyd, drd, bd, gd)
    want_sum = dyd + drd  # the separate addition, one rounding
    assert torch.equal(dsum, want_sum)
    wb, wpart = capi.gated_residual_bwd(want_sum, bd, gd)
    assert torch.equal(dbranch, wb) and torch.equal(part, wpart)


@pytest.mark.parametrize("fused_op,ref_op", [("fused_residual_adaln", "residual_adaln_ref"),
                                             ("fused_residual_adarmsnorm", "residual_adarmsnorm_ref")])
@pytest.mark.parametrize("use_gate", [True, False])
def test_operator_is_differentiable_and_matches_the_pytorch_definition(fused_op, ref_op, use_gate):
    b, s, h = 3, 64, 1152
    x, branch, gate, scale, shift, dy = _inputs(b, s, h, torch.bfloat16, seed=11)
    d_xnew = torch.roll(dy, 2, 1).to(DEV)
    dy = dy.to(DEV)

    def run(fn, dtype):
        leaves = [t.to(DEV, dtype).requires_grad_(True) for t in (x, branch, gate, scale, shift)]
        xv, bv, gv, sv, hv = leaves
        x_new, y = fn(xv, bv, gv if use_gate else None, sv, hv, 1e-6)
        targets = [t for i, t in enumerate(leaves) if use_gate or i != 2]
        grads = torch.autograd.grad((x_new, y), targets, (d_xnew.to(dtype), dy.to(dtype)))
        return x_new, y, grads

    xf, yf, gf = run(getattr(ops, fused_op), torch.bfloat16)
    xr, yr, gr = run(getattr(ops, ref_op), torch.float32)  # fp32 evaluation of the same bf16 inputs
    assert oracle.rel_l2(xf.float().cpu(), xr.cpu()) < 1e-2 and oracle.rel_l2(yf.float().cpu(), yr.cpu()) < 1e-2
    for a, e in zip(gf, gr):
        assert oracle.rel_l2(a.float().cpu(), e.cpu()) < 1e-2
