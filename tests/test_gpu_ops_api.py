"""The `novadit.ops`-compatible Python API on CUDA tensors: the cases the reference's own test files pin
(tests/test_fused_adaln.py, test_fused_adarmsnorm.py, test_fused_gate_act.py, test_fused_fc1_bias_act.py),
with the reference's tolerances, against the oracle evaluated on the same bits."""
from __future__ import annotations

import pytest
import torch

import novadit_b200.ops as ops
from oracle import novadit_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, want, tol):
    torch.testing.assert_close(got.cpu().float(), want.cpu().float(), rtol=tol, atol=tol)


@pytest.mark.parametrize("name", ["adaln", "adarmsnorm"])
@pytest.mark.parametrize("dtype,shape,tol", [
    (torch.float16, (2, 3, 768), 1e-2), (torch.bfloat16, (2, 3, 768), 2e-2),
    (torch.float16, (2, 3, 770), 2e-2), (torch.bfloat16, (2, 3, 770), 3e-2),
])
@pytest.mark.parametrize("mod3d", [False, True])
def test_forward_and_inference_match_reference_function(name, dtype, shape, tol, mod3d):
    torch.manual_seed(0)
    b, s, h = shape
    x = torch.randn(b, s, h, device=DEV, dtype=dtype)
    mshape = (b, 1, h) if mod3d else (b, h)
    scale, shift = torch.randn(*mshape, device=DEV, dtype=dtype), torch.randn(*mshape, device=DEV, dtype=dtype)
    fused = ops.fused_adaln if name == "adaln" else ops.fused_adarmsnorm
    infer = ops.fused_adaln_inference if name == "adaln" else ops.fused_adarmsnorm_inference
    ofwd = oracle.adaln_fwd if name == "adaln" else oracle.adarms_fwd
    want = ofwd(x.cpu(), scale.cpu(), shift.cpu(), 1e-5)[0]
    out = fused(x, scale, shift, eps=1e-5)
    assert out.shape == x.shape and out.dtype == x.dtype
    _close(out, want, tol)
    assert torch.equal(infer(x, scale, shift, eps=1e-5), out)  # inference == training output


@pytest.mark.parametrize("dtype,h,tol", [(torch.float16, 768, 2e-2), (torch.bfloat16, 768, 4e-2),
                                         (torch.float16, 770, 3e-2), (torch.bfloat16, 770, 5e-2)])
def test_adaln_extension_entry_points_like_the_reference_tests(dtype, h, tol):
    """fused_adaln_forward statistics, backward_dx and backward_dparam (S = 257) through the pybind module."""
    torch.manual_seed(1)
    b, s = 2, 257
    x = torch.randn(b, s, h, device=DEV, dtype=dtype)
    scale, shift = torch.randn(b, h, device=DEV, dtype=dtype), torch.randn(b, h, device=DEV, dtype=dtype)
    dy = torch.randn_like(x)
    y, saved_scale, mean, invstd = ops.novadit_cuda.fused_adaln_forward(x, scale, shift, 1e-5)
    assert saved_scale.shape == scale.shape and mean.shape == (b, s) and invstd.dtype == torch.float32
    _, wmean, winvstd = oracle.adaln_fwd(x.cpu(), scale.cpu(), shift.cpu(), 1e-5)
    _close(mean, wmean, 1e-3)
    _close(invstd, winvstd, 1e-3)
    wdx, wds, wdh = oracle.adaln_bwd(dy.cpu(), x.cpu(), scale.cpu(), 1e-5)
    _close(ops.fused_adaln_backward_dx(dy, x, saved_scale, mean, invstd), wdx, tol)
    dscale, dshift = ops.fused_adaln_backward_dparam(dy, x, mean, invstd)
    assert dscale.shape == (b, h) and dscale.dtype == torch.float32 and dshift.dtype == torch.float32
    _close(dscale, wds, tol)
    _close(dshift, wdh, tol)


@pytest.mark.parametrize("name", ["adaln", "adarmsnorm"])
@pytest.mark.parametrize("needs", [(True, True, True), (True, False, False), (False, True, True), (False, False, True)])
def test_autograd_matches_reference_function(name, needs):
    torch.manual_seed(2)
    shape = (2, 3, 768)
    fused = ops.fused_adaln if name == "adaln" else ops.fused_adarmsnorm
    ref = ops.adaln_ref if name == "adaln" else ops.adarmsnorm_ref
    x = torch.randn(shape, device=DEV, dtype=torch.float16)
    scale = torch.randn(shape[0], shape[2], device=DEV, dtype=torch.float16)
    shift = torch.randn_like(scale)
    dy = torch.randn_like(x)
    leaves = [t.clone().requires_grad_(n) for t, n in zip((x, scale, shift), needs)]
    refs = [t.detach().cpu().float().requires_grad_(n) for t, n in zip((x, scale, shift), needs)]
    fused(*leaves).backward(dy)
    ref(*refs).backward(dy.cpu().float())
    for got, want, need in zip(leaves, refs, needs):
        if need:
            _close(got.grad, want.grad, 2e-2)
        else:
            assert got.grad is None


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("dtype,inter,tol", [(torch.float16, 768, 2e-2), (torch.bfloat16, 768, 2e-2),
                                             (torch.float32, 768, 1e-4), (torch.float16, 385, 2e-2),
                                             (torch.bfloat16, 385, 3e-2), (torch.float32, 385, 1e-4)])
def test_gate_act_forward_backward(act, dtype, inter, tol):
    torch.manual_seed(3)
    x = torch.randn(2, 4, 2 * inter, device=DEV, dtype=dtype, requires_grad=True)
    dy = torch.randn(2, 4, inter, device=DEV, dtype=dtype)
    y = ops.fused_gate_act(x, act)
    assert y.shape == (2, 4, inter) and y.dtype == dtype
    y.backward(dy)
    _close(y, oracle.gate_act_fwd(x.detach().cpu(), act), tol)
    _close(x.grad, oracle.gate_act_bwd(dy.cpu(), x.detach().cpu(), act), max(tol, 5e-4))
    if act == "gelu":
        assert torch.equal(ops.fused_geglu(x.detach()), y.detach())
    # a non-contiguous upstream gradient is accepted (the callee makes it contiguous)
    dy_t = torch.randn(2, inter, 4, device=DEV, dtype=dtype).transpose(1, 2)
    z = ops.novadit_cuda.fused_gate_act_backward(dy_t, x.detach(), 0 if act == "silu" else 1)
    _close(z, oracle.gate_act_bwd(dy_t.cpu().contiguous(), x.detach().cpu(), act), max(tol, 5e-4))


@pytest.mark.parametrize("dtype,b,s,h,i,act", [(torch.float16, 2, 128, 768, 768, "silu"),
                                               (torch.float16, 1, 64, 1152, 3072, "gelu"),
                                               (torch.bfloat16, 2, 64, 1152, 1152, "gelu")])
def test_fc1_bias_act_forward_and_autograd(dtype, b, s, h, i, act):
    torch.manual_seed(42)
    x = (torch.randn(b, s, h, device=DEV) ).to(dtype).requires_grad_(True)
    w = (torch.randn(2 * i, h, device=DEV) / h ** 0.5).to(dtype).requires_grad_(True)
    bias = (torch.randn(2 * i, device=DEV) * 0.1).to(dtype).requires_grad_(True)
    y = ops.fused_fc1_bias_act(x, w, bias, act)
    assert y.shape == (b, s, i) and y.dtype == dtype
    want = oracle.fc1_fwd(x.detach().cpu(), w.detach().cpu(), bias.detach().cpu(), act)
    tol = 3e-2 if dtype == torch.bfloat16 else 2e-2
    _close(y, want, tol)
    # the drop-in pybind entry takes the interleaved layout the reference's Python hands it
    y2 = ops.novadit_cuda.fused_fc1_bias_act_forward(x.detach(), ops.interleave_weight(w.detach()),
                                                     ops.interleave_bias(bias.detach()), 0 if act == "silu" else 1)
    _close(y2, want, tol)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, br = (t.detach().cpu().float().requires_grad_(True) for t in (x, w, bias))
    ops.fc1_bias_act_ref(xr, wr, br, act).backward(dy.cpu().float())
    for got, ref in ((x.grad, xr.grad), (w.grad, wr.grad), (bias.grad, br.grad)):
        assert oracle.rel_l2(got.cpu(), ref) < 2e-2


def test_fc1_fp8_api():
    torch.manual_seed(5)
    x = torch.randn(2, 256, 1152, device=DEV).bfloat16()
    w = (torch.randn(2 * 1152, 1152, device=DEV) * 0.02).bfloat16()
    bias = (torch.randn(2 * 1152, device=DEV) * 0.02).bfloat16()
    y = ops.fused_fc1_bias_act_fp8(x, w, bias, "gelu")
    qx, sx = oracle.quant_e4m3(x.cpu())
    qw, sw = oracle.quant_e4m3(w.cpu())
    want = oracle.fc1_fwd_fp8(qx, sx, qw, sw, bias.cpu(), "gelu", gated=True)
    assert oracle.rel_l2(y.cpu(), want) <= 3e-2
