"""AdaLN / AdaRMSNorm forward with FP8 e4m3 output and the AdaLN -> FC1 chain in FP8 (delayed scaling)."""
from __future__ import annotations

import pytest
import torch

from novadit_b200 import capi, synth
from oracle import novadit_oracle as oracle
from tests.helpers import FP8_REL_L2

pytestmark = pytest.mark.gpu
DEV = "cuda"


def oracle_y(kind, x, scale, shift, eps):
    if kind == "layer":
        return oracle.adaln_fwd(x, scale, shift, eps, compute=torch.float64, round_out=False)[0]
    return oracle.adarms_fwd(x, scale, shift, eps, compute=torch.float64, round_out=False)[0]


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("dtype,shape", [
    (torch.bfloat16, (4, 64, 1152)), (torch.float16, (3, 77, 768)), (torch.bfloat16, (2, 9, 128)),
    (torch.bfloat16, (2, 40, 1536)), (torch.float32, (2, 33, 768)),
])
def test_e4m3_output_matches_quantised_oracle(kind, dtype, shape):
    b, s, h = shape
    x, scale, shift, _ = synth.norm_inputs(b, s, h, dtype, 23)
    want = oracle_y(kind, x, scale, shift, 1e-6)
    true_amax = float(want.abs().max())
    q_scale = torch.tensor([true_amax / 448.0], dtype=torch.float32, device=DEV)
    amax = torch.zeros(1, dtype=torch.float32, device=DEV)
    out = capi.norm_fwd_e4m3(kind, x.to(DEV), scale.to(DEV), shift.to(DEV), 1e-6, q_scale, amax)
    out16 = capi.norm_fwd(kind, x.to(DEV), scale.to(DEV), shift.to(DEV), 1e-6)
    torch.cuda.synchronize()
    q = out[0]
    assert q.dtype == torch.float8_e4m3fn and q.shape == x.shape
    # the recorded maximum is the maximum of the fp32 values before any rounding
    assert abs(float(amax) - true_amax) <= 1e-5 * true_amax
    # statistics are those of the 16-bit forward (another kernel, another summation order: a few ulps)
    assert torch.allclose(out[-1], out16[-1], rtol=2e-6, atol=0)
    # de-quantised output: every element within half an e4m3 step of the exact value (3 mantissa bits: 2^-4 relative,
    # plus the subnormal step 2^-9 * scale), and a small relative L2 overall
    deq = q.float().cpu().double() * float(q_scale)
    err = (deq - want).abs()
    bound = want.abs() * 2.0 ** -4 * 1.001 + float(q_scale) * 2.0 ** -10 * 1.001 + 1e-7
    assert bool((err <= bound).all()), f"max excess {float((err - bound).max()):.3e}"
    assert oracle.rel_l2(deq.float(), want.float()) < 4e-2
    # and it equals, code for code up to rare ties, the oracle's quantisation of the exact values
    codes = (want / float(q_scale)).float().clamp(-448, 448).to(torch.float8_e4m3fn)
    same = (codes.view(torch.uint8) == q.cpu().view(torch.uint8)).float().mean()
    assert float(same) > 0.999


def test_amax_accumulates_and_saturation_clamps():
    x, scale, shift, _ = synth.norm_inputs(2, 16, 256, torch.bfloat16, 5)
    q_scale = torch.tensor([1e-3], dtype=torch.float32, device=DEV)  # far too small: everything saturates
    amax = torch.tensor([123.0], dtype=torch.float32, device=DEV)   # an earlier, larger maximum stays
    q, _, _ = capi.norm_fwd_e4m3("layer", x.to(DEV), scale.to(DEV), shift.to(DEV), 1e-6, q_scale, amax)
    torch.cuda.synchronize()
    assert float(amax) == 123.0
    assert bool(torch.isfinite(q.float()).all()) and float(q.float().abs().max()) == 448.0


def test_unsupported_width_is_refused():
    x, scale, shift, _ = synth.norm_inputs(1, 4, 2048, torch.bfloat16, 1)
    q_scale = torch.ones(1, dtype=torch.float32, device=DEV)
    with pytest.raises(capi.NovaditError):
        capi.norm_fwd_e4m3("layer", x.to(DEV), scale.to(DEV), shift.to(DEV), 1e-6, q_scale)


def test_adaln_to_fc1_chain_in_fp8():
    """AdaLN writes e4m3 with last step's scale; FC1 consumes it: against the fp32 pipeline on de-quantised operands."""
    b, s, h, n = 4, 128, 1152, 2304
    x, scale, shift, _ = synth.norm_inputs(b, s, h, torch.bfloat16, 3)
    _, w, bias = synth.fc1_inputs(8, h, n, torch.bfloat16, 4)
    y_exact = oracle_y("layer", x, scale, shift, 1e-6)
    q_scale = torch.tensor([float(y_exact.abs().max()) * 1.05 / 448.0], dtype=torch.float32, device=DEV)  # a stale scale
    amax = torch.zeros(1, dtype=torch.float32, device=DEV)
    q, _, _ = capi.norm_fwd_e4m3("layer", x.to(DEV), scale.to(DEV), shift.to(DEV), 1e-6, q_scale, amax)
    qw, sw = capi.quantize_e4m3(w.to(DEV))
    out = capi.fc1_fwd(q.reshape(b * s, h), qw, bias.to(DEV), "gelu", 1, alpha_dev=torch.cat([q_scale, sw]),
                       out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    oqw, osw = oracle.quant_e4m3(w)
    want = oracle.fc1_fwd_fp8(q.reshape(b * s, h).cpu(), float(q_scale), oqw, osw, bias, "gelu", gated=True)
    assert oracle.rel_l2(out.cpu(), want) < 5e-3  # the kernel's own error on identical FP8 operands
    full = oracle.fc1_fwd(y_exact.reshape(b * s, h).float(), w.float(), bias.float(), "gelu", gated=True,
                          compute=torch.float32, out_dtype=torch.float32)
    print("chain vs unquantised fp32 pipeline, rel_l2:", oracle.rel_l2(out.cpu().float(), full))
