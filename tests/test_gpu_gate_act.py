"""Gated-activation CUDA kernels against the CPU oracle and the reference's golden vectors (through the C ABI)."""
from __future__ import annotations

import pytest
import torch

from novadit_b200 import capi, synth
from oracle import novadit_oracle as oracle
from tests import golden_io
from tests.helpers import assert_half_parity, assert_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"
GATE = golden_io.load("gate_act_golden")


def assert_gate_parity(got, want, what):
    if want.dtype == torch.float32:
        # the reference's own fp32 tolerances: 1e-4 forward, 5e-4 backward (tests/test_fused_gate_act.py)
        torch.testing.assert_close(got.cpu(), want, rtol=1e-4, atol=1e-4, msg=lambda m: what + ": " + m)
    else:
        assert_half_parity(got, want, what)


@pytest.mark.parametrize("case", sorted(GATE))
def test_matches_reference_golden_vectors(case):
    g = GATE[case]
    dtype = golden_io.DTYPES[g["dtype"]]
    b, s, i = (int(v) for v in g["shape"])
    x, dy = synth.gate_act_inputs(b, s, i, dtype, int(g["seed"]))
    y = capi.gate_act_fwd(x.to(DEV), g["act"])
    dz = capi.gate_act_bwd(dy.to(DEV), x.to(DEV), g["act"])
    assert_gate_parity(y, golden_io.unpack(g["y"], dtype).reshape(b, s, i), case + " y")
    assert_gate_parity(dz, golden_io.unpack(g["dz"], dtype).reshape(b, s, 2 * i), case + " dz")


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("dtype,shape", [
    (torch.float16, (2, 4, 768)), (torch.bfloat16, (2, 4, 768)), (torch.float32, (2, 4, 768)),
    (torch.float16, (2, 4, 385)), (torch.bfloat16, (2, 4, 385)), (torch.float32, (2, 4, 385)),  # ragged I
    (torch.bfloat16, (1, 1, 8)), (torch.bfloat16, (3, 7, 4608)), (torch.bfloat16, (1, 5, 20000)),
])
def test_matches_oracle(act, dtype, shape):
    b, s, i = shape
    x, dy = synth.gate_act_inputs(b, s, i, dtype, seed=40 + i % 13)
    y = capi.gate_act_fwd(x.to(DEV), act)
    dz = capi.gate_act_bwd(dy.to(DEV), x.to(DEV), act)
    assert_gate_parity(y, oracle.gate_act_fwd(x, act, compute=torch.float64), f"{act} {dtype} {shape} y")
    assert_gate_parity(dz, oracle.gate_act_bwd(dy, x, act, compute=torch.float64), f"{act} {dtype} {shape} dz")


@pytest.mark.parametrize("act", ["silu", "gelu"])
def test_config3_slice_bf16(act):
    """Workload config 3 row width (I = 4608) on 2048 of its 32768 rows, against the oracle."""
    x, dy = synth.gate_act_inputs(1, 2048, 4608, torch.bfloat16, seed=3)
    y = capi.gate_act_fwd(x.to(DEV), act)
    dz = capi.gate_act_bwd(dy.to(DEV), x.to(DEV), act)
    assert_half_parity(y, oracle.gate_act_fwd(x, act), f"config3 {act} y")
    assert_half_parity(dz, oracle.gate_act_bwd(dy, x, act), f"config3 {act} dz")


@pytest.mark.parametrize("act", ["silu", "gelu"])
def test_config3_full_size_properties(act):
    """Full config 3 (B=8, S=4096, I=4608): rows are independent and the op is linear in `up` and in dy."""
    b, s, i = 8, 4096, 4608
    g = torch.Generator(device=DEV).manual_seed(11)
    x = torch.randn(b, s, 2 * i, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    dy = torch.randn(b, s, i, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    y = capi.gate_act_fwd(x, act)
    dz = capi.gate_act_bwd(dy, x, act)
    # doubling `up` (exact in bf16) doubles y and the gate half of dz, leaves the up half of dz unchanged
    x2 = x.clone()
    x2[..., :i] *= 2
    assert torch.equal(capi.gate_act_fwd(x2, act), y * 2)
    dz2 = capi.gate_act_bwd(dy, x2, act)
    assert torch.equal(dz2[..., :i], dz[..., :i]) and torch.equal(dz2[..., i:], dz[..., i:] * 2)
    # doubling dy doubles dz
    assert torch.equal(capi.gate_act_bwd(dy * 2, x, act), dz * 2)
    # a sample of rows equals the same rows computed alone, and the oracle
    rows = torch.randint(0, b * s, (128,), generator=g, device=DEV)
    xs = x.reshape(-1, 2 * i)[rows].contiguous()
    assert torch.equal(capi.gate_act_fwd(xs.unsqueeze(0), act)[0], y.reshape(-1, i)[rows])
    assert_half_parity(y.reshape(-1, i)[rows].cpu(), oracle.gate_act_fwd(xs.cpu(), act), "sampled rows y")
    dys = dy.reshape(-1, i)[rows].contiguous()
    assert_half_parity(dz.reshape(-1, 2 * i)[rows].cpu(), oracle.gate_act_bwd(dys.cpu(), xs.cpu(), act), "sampled rows dz")


def test_extreme_gate_values_do_not_produce_nan():
    x = torch.tensor([[[1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, -80.0, 80.0, -1e4, 1e4, 0.0, -0.0, 30.0, -30.0]]],
                     dtype=torch.float32)
    dy = torch.ones(1, 1, 8)
    for act in ("silu", "gelu"):
        y = capi.gate_act_fwd(x.to(DEV), act).cpu()
        dz = capi.gate_act_bwd(dy.to(DEV), x.to(DEV), act).cpu()
        assert torch.isfinite(y).all() and torch.isfinite(dz).all()
        torch.testing.assert_close(y, oracle.gate_act_fwd(x, act, compute=torch.float64), rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(dz, oracle.gate_act_bwd(dy, x, act, compute=torch.float64), rtol=5e-4, atol=5e-4)


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("dtype,inter", [(torch.bfloat16, 4608), (torch.float16, 200), (torch.float32, 33)])
def test_gate_first_layout_is_the_same_backward_with_halves_swapped(act, dtype, inter):
    """Rows [gate | up] (FC1's pre-activation) give, half for half, the bits of the [up | gate] backward."""
    x, dy = synth.gate_act_inputs(2, 37, inter, dtype, seed=9)
    xd, gd = x.to(DEV), dy.to(DEV)
    dz = capi.gate_act_bwd(gd, xd, act)
    z = torch.cat([xd[..., inter:], xd[..., :inter]], dim=-1).contiguous()
    dz_gf = capi.gate_act_bwd(gd, z, act, gate_first=True)
    torch.cuda.synchronize()
    assert torch.equal(dz_gf[..., :inter], dz[..., inter:]) and torch.equal(dz_gf[..., inter:], dz[..., :inter])
