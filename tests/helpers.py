"""Shared helpers of the parity tests."""
from __future__ import annotations

import torch

from oracle import novadit_oracle as oracle

# Parity bars of the workload statement.
HALF_MAX_ABS = 2e-2   # bf16 / fp16 outputs: max |got - want|
HALF_REL_L2 = 1e-2    # bf16 / fp16 outputs: relative L2
F32_REL_L2 = 1e-4     # fp32 dscale / dshift: relative L2
FP8_REL_L2 = 3e-2     # FP8 FC1 against an fp32 GEMM of the de-quantised operands


def assert_half_parity(got: torch.Tensor, want: torch.Tensor, what: str) -> None:
    got, want = got.detach().cpu(), want.detach().cpu()
    assert got.shape == want.shape and got.dtype == want.dtype, f"{what}: shape/dtype {got.shape} {got.dtype}"
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite output"
    ma, rl = oracle.max_abs(got, want), oracle.rel_l2(got, want)
    assert ma <= HALF_MAX_ABS and rl <= HALF_REL_L2, f"{what}: max_abs {ma:.3e} rel_l2 {rl:.3e}"


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
