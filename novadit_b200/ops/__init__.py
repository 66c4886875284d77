"""`novadit.ops`-compatible operator API backed by the sm_100a kernels.

Same public names as the reference's `novadit/ops/__init__.py:46-76`. The
`fused_*` functions run ONLY the CUDA kernels (through the `novadit_cuda`
extension, itself a thin layer over the C ABI): a CPU tensor or a missing
extension raises instead of falling back to PyTorch. The `*_ref` functions are
the plain PyTorch definitions the reference also exports; nothing in the fused
path calls them.
"""
from __future__ import annotations

import importlib

importlib.import_module("torch")  # load torch's shared libraries before the native extension

try:
    from .. import novadit_cuda  # type: ignore

    HAS_NOVADIT_CUDA = True
    NOVADIT_CUDA_IMPORT_ERROR = None
except Exception as exc:  # the extension is not built: every fused_* call will raise
    novadit_cuda = None
    HAS_NOVADIT_CUDA = False
    NOVADIT_CUDA_IMPORT_ERROR = exc


def require_cuda_extension(op: str, tensor, ref_name: str):
    """Return the extension module or raise: the fused operators have no fallback."""
    if novadit_cuda is None:
        raise RuntimeError(
            f"{op}: the novadit_cuda extension is not available ({NOVADIT_CUDA_IMPORT_ERROR!r}); "
            "build it with `python -m novadit_b200.build`")
    if not tensor.is_cuda:
        raise RuntimeError(
            f"{op} runs only on CUDA tensors (no CPU fallback); use {ref_name} for a PyTorch evaluation")
    return novadit_cuda


from .adaln import (  # noqa: E402
    adaln_ref,
    fused_adaln,
    fused_adaln_backward_dparam,
    fused_adaln_backward_dx,
    fused_adaln_e4m3,
    fused_adaln_inference,
)
from .adarmsnorm import adarmsnorm_ref, fused_adarmsnorm, fused_adarmsnorm_inference  # noqa: E402
from .fc1_bias_act import (  # noqa: E402
    fc1_bias_act_ref,
    fused_fc1_bias_act,
    fused_fc1_bias_act_fp8,
    quantize_e4m3,
    interleave_bias,
    interleave_weight,
    split_gated_weight,
    un_interleave_bias,
    un_interleave_weight,
)
from .gate_act import fused_gate_act, fused_geglu, gate_act_ref, geglu_ref  # noqa: E402
from .outside_path import adaln_compile, adarmsnorm_compile  # noqa: E402
from .qkv_pack import fused_qkv_linear_pack, fused_qkv_pack, qkv_pack_ref  # noqa: E402
from .residual import (  # noqa: E402
    fused_gated_residual,
    fused_out_residual,
    fused_residual_adaln,
    fused_residual_adarmsnorm,
    gated_residual_ref,
    out_residual_ref,
    residual_adaln_ref,
    residual_adarmsnorm_ref,
)

__all__ = [
    "HAS_NOVADIT_CUDA",
    "NOVADIT_CUDA_IMPORT_ERROR",
    "adarmsnorm_ref",
    "adaln_ref",
    "fused_adaln",
    "fused_adaln_e4m3",
    "fused_adaln_inference",
    "fused_adaln_backward_dparam",
    "fused_adaln_backward_dx",
    "fused_adarmsnorm",
    "fused_adarmsnorm_inference",
    "fused_geglu",
    "fused_gate_act",
    "gate_act_ref",
    "geglu_ref",
    "fc1_bias_act_ref",
    "fused_fc1_bias_act",
    "fused_fc1_bias_act_fp8",
    "interleave_weight",
    "un_interleave_weight",
    "interleave_bias",
    "un_interleave_bias",
    "split_gated_weight",
    "fused_gated_residual",
    "fused_residual_adaln",
    "fused_residual_adarmsnorm",
    "residual_adaln_ref",
    "residual_adarmsnorm_ref",
    "quantize_e4m3",
    "fused_out_residual",
    "gated_residual_ref",
    "fused_qkv_linear_pack",
    "fused_qkv_pack",
    "adaln_compile",
    "adarmsnorm_compile",
    "novadit_cuda",
    "out_residual_ref",
    "qkv_pack_ref",
]
