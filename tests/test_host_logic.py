"""Host-side logic that needs no GPU: the operator API surface, error behaviour, weight helpers."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import novadit_b200.ops as ops
from tests import golden_io

REFERENCE_EXPORTS = [  # novadit/ops/__init__.py:46-76 of the reference
    "HAS_NOVADIT_CUDA", "NOVADIT_CUDA_IMPORT_ERROR", "adarmsnorm_ref", "adaln_ref", "fused_adaln",
    "fused_adaln_inference", "fused_adaln_backward_dparam", "fused_adaln_backward_dx", "fused_adarmsnorm",
    "fused_adarmsnorm_inference", "fused_geglu", "fused_gate_act", "gate_act_ref", "geglu_ref", "fc1_bias_act_ref",
    "fused_fc1_bias_act", "interleave_weight", "un_interleave_weight", "interleave_bias", "un_interleave_bias",
    "split_gated_weight", "fused_out_residual", "fused_qkv_linear_pack", "fused_qkv_pack", "adaln_compile",
    "adarmsnorm_compile", "novadit_cuda", "out_residual_ref", "qkv_pack_ref",
]
PYBIND_EXPORTS = [  # csrc/bindings.cpp:85-116 of the reference
    "fused_adaln_forward", "fused_adaln_forward_inference", "fused_adaln_backward_dx", "fused_adaln_backward_dparam",
    "fused_qkv_pack_forward", "fused_out_residual_forward", "fused_geglu_forward", "fused_geglu_backward",
    "fused_gate_act_forward", "fused_gate_act_backward", "fused_adarmsnorm_forward",
    "fused_adarmsnorm_forward_inference", "fused_adarmsnorm_backward_dx", "fused_adarmsnorm_backward_dparam",
    "fused_fc1_bias_act_forward",
]


def test_ops_api_surface_matches_reference():
    for name in REFERENCE_EXPORTS:
        assert hasattr(ops, name), name
        assert name in ops.__all__, name


def test_extension_exports_the_reference_pybind_names():
    assert ops.HAS_NOVADIT_CUDA, f"extension not importable: {ops.NOVADIT_CUDA_IMPORT_ERROR!r}"
    for name in PYBIND_EXPORTS:
        assert hasattr(ops.novadit_cuda, name), name


def test_fused_ops_refuse_cpu_tensors_instead_of_falling_back():
    x = torch.randn(2, 4, 16)
    s = torch.randn(2, 16)
    for fn in (ops.fused_adaln, ops.fused_adaln_inference, ops.fused_adarmsnorm, ops.fused_adarmsnorm_inference):
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            fn(x, s, s)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.fused_gate_act(x, "silu")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.fused_geglu(x)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.fused_fc1_bias_act(x.bfloat16(), torch.randn(8, 16).bfloat16())
    with pytest.raises(ValueError):
        ops.fused_gate_act(x, "relu")


def test_extension_validates_like_the_reference():
    ext = ops.novadit_cuda
    x = torch.randn(2, 4, 16)
    with pytest.raises(RuntimeError, match="x must be a CUDA tensor"):
        ext.fused_adaln_forward(x, torch.randn(2, 16), torch.randn(2, 16), 1e-5)
    with pytest.raises(RuntimeError, match="z must be a CUDA tensor"):
        ext.fused_geglu_forward(x)
    with pytest.raises(RuntimeError, match="qkv must be a CUDA tensor"):
        ext.fused_qkv_pack_forward(x, 2, 8)
    with pytest.raises(RuntimeError, match="must be CUDA tensors"):
        ext.fused_out_residual_forward(x, x, None)


def test_ref_functions_shapes_and_formula():
    x = torch.randn(2, 8, 16, dtype=torch.bfloat16)
    for shape in [(2, 16), (2, 1, 16)]:
        s, h = torch.randn(*shape, dtype=torch.bfloat16), torch.randn(*shape, dtype=torch.bfloat16)
        assert ops.adaln_ref(x, s, h).shape == x.shape and ops.adaln_ref(x, s, h).dtype == x.dtype
        assert ops.adarmsnorm_ref(x, s, h).shape == x.shape
    z = torch.randn(2, 8, 128)
    assert ops.geglu_ref(z).shape == (2, 8, 64)
    torch.testing.assert_close(ops.gate_act_ref(z, "gelu"), ops.geglu_ref(z))
    w, b = torch.randn(64, 32), torch.randn(64)
    assert ops.fc1_bias_act_ref(torch.randn(2, 4, 32), w, b, "silu").shape == (2, 4, 32)


def test_interleave_helpers_match_reference_known_answers():
    g = np.load(golden_io.GOLDEN_DIR + "/interleave_golden.npz")
    w, b = torch.from_numpy(g["w"]), torch.from_numpy(g["b"])
    wi = ops.interleave_weight(w)
    assert torch.equal(wi, torch.from_numpy(g["w_inter"]))
    assert torch.equal(ops.interleave_bias(b), torch.from_numpy(g["b_inter"]))
    assert torch.equal(ops.un_interleave_weight(wi), w) and torch.equal(torch.from_numpy(g["w_round"]), w)
    assert torch.equal(ops.un_interleave_bias(ops.interleave_bias(b)), b)
    sg, sv = ops.split_gated_weight(wi)
    assert torch.equal(sg, torch.from_numpy(g["split_gate"])) and torch.equal(sv, torch.from_numpy(g["split_value"]))
    # same known answers the reference's tests spell out: row 1 of the interleaved weight is value row 0
    assert torch.equal(wi[1], w[3]) and torch.equal(wi[2], w[1])
    with pytest.raises(ValueError):
        ops.split_gated_weight(torch.randn(5, 4))
