"""Shared helpers of the parity tests."""
from __future__ import annotations

import torch

from oracle import novadit_oracle as oracle

# Parity bars of the workload statement.
HALF_MAX_ABS = 2e-2   # bf16 / fp16 outputs: max |got - want|
HALF_REL_L2 = 1e-2    # bf16 / fp16 outputs: relative L2
F32_REL_L2 = 1e-4     # fp32 dscale / dshift: relative L2
FP8_REL_L2 = 3e-2     # FP8 FC1 against an fp32 GEMM of the de-quantised operands


def _ulp(v: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Spacing of `dtype` numbers at |v| (v in fp64)."""
    mant = 8 if dtype == torch.bfloat16 else 11
    exp = torch.floor(torch.log2(v.abs().clamp_min(1e-30)))
    return torch.pow(torch.tensor(2.0, dtype=torch.float64), exp - (mant - 1))


def assert_half_parity(got: torch.Tensor, want: torch.Tensor, what: str, exact: torch.Tensor | None = None) -> None:
    """bf16/fp16 bar: max_abs <= 2e-2 and relative L2 <= 1e-2 against the oracle's rounded output.

    One exception, only when `exact` (the oracle's UNROUNDED fp64 value) is given: an element may
    differ from `want` by one rounding step if the exact value sits within 1% of a step of the
    midpoint between the two candidates. There both neighbours are correct roundings of values
    that fp32 arithmetic cannot tell apart, and above |y| = 4 one bf16 step (3.1e-2) is already
    larger than the max_abs bar, so without this rule the bar would measure luck, not error.
    """
    got, want = got.detach().cpu(), want.detach().cpu()
    assert got.shape == want.shape and got.dtype == want.dtype, f"{what}: shape/dtype {got.shape} {got.dtype}"
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite output"
    rl = oracle.rel_l2(got, want)
    assert rl <= HALF_REL_L2, f"{what}: rel_l2 {rl:.3e}"
    diff = (got.double() - want.double()).abs()
    bad = diff > HALF_MAX_ABS
    if bool(bad.any()) and exact is not None:
        ex = exact.detach().cpu().double().reshape(got.shape)
        step = _ulp(ex[bad], got.dtype)
        mid = (got.double()[bad] + want.double()[bad]) / 2
        one_step = (diff[bad] <= step * 1.001)
        near_tie = ((ex[bad] - mid).abs() <= 0.01 * step)
        ok = one_step & near_tie
        assert bool(ok.all()), (f"{what}: {int((~ok).sum())} element(s) beyond max_abs {HALF_MAX_ABS} that are not "
                                f"rounding near-ties (max_abs {float(diff.max()):.3e})")
        print(f"{what}: {int(bad.sum())} rounding near-tie(s) out of {got.numel()} elements")
        return
    assert not bool(bad.any()), f"{what}: max_abs {float(diff.max()):.3e} rel_l2 {rl:.3e}"


def assert_f32_parity(got: torch.Tensor, want: torch.Tensor, what: str, tol: float = F32_REL_L2) -> None:
    got, want = got.detach().cpu(), want.detach().cpu()
    assert got.shape == want.shape and got.dtype == torch.float32, f"{what}: shape/dtype {got.shape} {got.dtype}"
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    rl = oracle.rel_l2(got, want)
    assert rl <= tol, f"{what}: rel_l2 {rl:.3e}"


def assert_parity(got, want, what):
    if want.dtype == torch.float32:
        assert_f32_parity(got, want, what, tol=1e-5)
    else:
        assert_half_parity(got, want, what)
