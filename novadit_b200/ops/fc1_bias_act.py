"""Fused FC1: z = x @ W^T + b, W [2I, H] with rows [gate | value], y = value * act(gate).

Mirrors the reference's `novadit/ops/fc1_bias_act.py` (reference function :55-68, autograd Function
:213-285, helpers :30-52 and :329-347, public function :350-368). The forward is ONE tcgen05 kernel
with the bias, activation and gating in its epilogue; the weight is consumed as stored (no
per-call interleave copy, no JIT). The backward keeps the reference's formulation
(novadit/ops/fc1_bias_act.py:248-285) - recompute z, activation backward, dx = dz W, dW = dz^T x - with the
recomputation and the activation backward in ONE tcgen05 launch (the forward main loop with a backward epilogue;
z never reaches memory). dx, dW and dbias are library calls; the job of the reference's CuTe-DSL backward-dx
kernel (:288-326) is also available on this library's tcgen05 GEMM as `fused_fc1_bias_act_backward_dx`.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import require_cuda_extension


def interleave_weight(weight):
    """[gate block | value block] rows -> (gate0, value0, gate1, value1, ...)."""
    inter = weight.shape[0] // 2
    return torch.stack([weight[:inter], weight[inter:]], dim=1).reshape(2 * inter, -1).contiguous()


def un_interleave_weight(weight):
    return torch.cat([weight[0::2], weight[1::2]], dim=0).contiguous()


def interleave_bias(bias):
    inter = bias.shape[0] // 2
    return torch.stack([bias[:inter], bias[inter:]], dim=1).reshape(2 * inter).contiguous()


def un_interleave_bias(bias):
    return torch.cat([bias[0::2], bias[1::2]], dim=0).contiguous()


def split_gated_weight(weight):
    """Interleaved [2I, H] weight -> (w_gate [I,H], w_value [I,H]), both contiguous."""
    if weight.dim() != 2 or weight.shape[0] % 2 != 0:
        raise ValueError(f"weight must have shape [2*I, H] with an even first dim, got {tuple(weight.shape)}")
    return weight[0::2].contiguous(), weight[1::2].contiguous()


def fc1_bias_act_ref(x, weight, bias=None, activation: str = "silu"):
    """PyTorch definition, reference novadit/ops/fc1_bias_act.py:55-68."""
    z = F.linear(x, weight, bias)
    z_gate, z_value = z.chunk(2, dim=-1)
    if activation == "silu":
        return z_value * F.silu(z_gate)
    if activation == "gelu":
        return z_value * F.gelu(z_gate, approximate="tanh")
    raise ValueError(f"Unsupported activation: {activation}")


class _FusedFc1BiasActFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, act_id):
        ext = require_cuda_extension("fused_fc1_bias_act", x, "fc1_bias_act_ref")
        y = ext.fused_fc1_bias_act_forward_stacked(x.contiguous(), weight.contiguous(),
                                                   None if bias is None else bias.contiguous(), act_id)
        ctx.save_for_backward(x, weight, bias)
        ctx.act_id = act_id
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias = ctx.saved_tensors
        ext = require_cuda_extension("fused_fc1_bias_act", x, "fc1_bias_act_ref")
        inter, hidden = weight.shape[0] // 2, weight.shape[1]
        want_db = bias is not None and ctx.needs_input_grad[2]
        d_b = None
        if hidden % 8 == 0 and inter % 8 == 0:
            # z recomputed and differentiated inside one tcgen05 launch: it never reaches memory; dbias is summed
            # in the same epilogue, so dz is not read a second time for it
            if want_db:
                dz, d_b = ext.fused_fc1_bias_act_backward_dz_dbias(x, weight, bias, dy, ctx.act_id)
            else:
                dz = ext.fused_fc1_bias_act_backward_dz(x, weight, bias, dy, ctx.act_id)
        else:
            z = F.linear(x, weight, bias)  # recomputed, as in the reference
            dz = ext.fused_gate_act_backward_gate_first(dy.contiguous(), z, ctx.act_id)  # one pass, not ~8 eager ones
        if hidden % 8 == 0 and inter % 4 == 0:
            # dx = dz W and dW = dz^T x on the tcgen05 GEMMs that read W, dz and x in place (MN-major operands);
            # dbias by the two-stage column sum where the dz launch has not produced it: no library GEMM or
            # reduction in the backward pass
            dx = ext.fused_fc1_bias_act_backward_dx(dz, weight) if ctx.needs_input_grad[0] else None
            d_w = ext.fused_fc1_bias_act_backward_dw(dz, x) if ctx.needs_input_grad[1] else None
            if want_db and d_b is None:
                d_b = ext.fused_fc1_bias_act_backward_dbias(dz)
            return dx, d_w, d_b, None
        # rows the copy engine cannot walk (pitches that are not multiples of 16 bytes): PyTorch's GEMMs
        m = x.shape[0] * x.shape[1]
        dz_flat, x_flat = dz.reshape(m, -1), x.reshape(m, -1)
        dx = (dz_flat @ weight).reshape(x.shape)
        d_w = dz_flat.T @ x_flat
        if want_db and d_b is None:
            d_b = dz_flat.sum(dim=0)
        return dx, d_w, d_b, None


def fused_fc1_bias_act(x, weight, bias=None, activation: str = "silu"):
    """x [B,S,H], weight [2I,H], bias [2I] or None (all fp16 or all bf16, CUDA) -> y [B,S,I]."""
    if activation not in {"silu", "gelu"}:
        raise ValueError(f"Unsupported activation: {activation}")
    require_cuda_extension("fused_fc1_bias_act", x, "fc1_bias_act_ref")
    if x.dtype not in (torch.float16, torch.bfloat16) or weight.dtype != x.dtype or (
            bias is not None and bias.dtype != x.dtype):
        raise RuntimeError("fused_fc1_bias_act needs x, weight and bias of one dtype, fp16 or bf16")
    return _FusedFc1BiasActFunction.apply(x, weight, bias, 0 if activation == "silu" else 1)


@torch.no_grad()
def fused_fc1_bias_act_fp8(x, weight, bias=None, activation: str = "gelu", gated: bool = True,
                           weight_q=None):
    """FP8 e4m3 forward with per-tensor amax scales (no counterpart in the reference).

    x and weight are quantised on the device (amax -> scale -> saturating e4m3), the GEMM runs
    in `kind::f8f6f4` with fp32 accumulation, and the two de-quantisation scales are applied in
    the epilogue before bias and activation. Pass `weight_q=(q, scale)` from an earlier
    `quantize_e4m3(weight)` to skip re-quantising a static weight. x [B, S, H] (or [M, H]); returns bf16/fp16.
    """
    ext = require_cuda_extension("fused_fc1_bias_act_fp8", x, "fc1_bias_act_ref")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("fused_fc1_bias_act_fp8 needs fp16 or bf16 activations (the output takes their dtype)")
    x3 = x.contiguous() if x.dim() == 3 else x.contiguous().unsqueeze(0)
    qx, sx = ext.quantize_e4m3(x3)
    qw, sw = weight_q if weight_q is not None else ext.quantize_e4m3(weight.contiguous())
    y = ext.fused_fc1_bias_act_forward_fp8(qx, qw, bias, torch.cat([sx, sw]), 0 if activation == "silu" else 1,
                                           bool(gated), x.dtype == torch.bfloat16)
    return y if x.dim() == 3 else y.squeeze(0)


@torch.no_grad()
def quantize_e4m3(x):
    """Per-tensor amax scaling to e4m3 on the device: (q, scale) with scale = amax / 448 as a 1-element fp32 tensor."""
    ext = require_cuda_extension("quantize_e4m3", x, "torch.Tensor.to(torch.float8_e4m3fn)")
    return tuple(ext.quantize_e4m3(x.contiguous()))
