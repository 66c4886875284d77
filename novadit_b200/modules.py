"""The DiT-XL/2 block-stack harness of workload config 5, built on the REFERENCE's own block modules.

Nothing of `novadit/modules` is re-typed here. `reference_modules()` imports the reference's `novadit.modules`
(`NovaDiTBlock`, `NovaDiTAttention`, `NovaDiTMLP`: `novadit/modules/dit_block.py:11-71`, `dit_attention.py:10-80`,
`dit_mlp.py:9-57`) after making this library's extension importable as `novadit_cuda`, the name the reference's
`novadit/ops/__init__.py:10-18` looks for - which is the whole drop-in: the reference's Python, unchanged, runs on
these kernels. The `novadit` package must be importable (installed, on `PYTHONPATH`, or unpacked under
`baseline/_ref` next to this package).

What the reference does not have, and this module adds around its blocks, is the adaLN-Zero conditioning of DiT
(workload config 5): SiLU -> Linear(H, 6H), zero-initialised, giving shift / scale / gate for the attention and the
MLP branch, with the gated residual `x + gate * branch` as one kernel. An `AdaLNZeroBlock` drives the SUBMODULES
of one reference `NovaDiTBlock` (`_adaln`, `attn`, `mlp`) because the reference block's own forward has neither a
gate nor a conditioning input. With `use_fused=False` every operator is the reference's PyTorch `*_ref`
definition: that stack is the parity twin and the timing baseline of the harness.
"""
from __future__ import annotations

import importlib
import os
import sys

import torch
import torch.nn.functional as F
from torch import nn

from . import ops

_REF_INSTALL = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


def reference_modules():
    """The reference's `novadit.modules`, importing its `novadit.ops` on top of THIS library's extension."""
    if ops.novadit_cuda is None:
        raise RuntimeError(f"the novadit_cuda extension is not built: {ops.NOVADIT_CUDA_IMPORT_ERROR!r}")
    sys.modules.setdefault("novadit_cuda", ops.novadit_cuda)  # the top-level name the reference imports
    try:
        mods = importlib.import_module("novadit.modules")
    except ImportError:
        if not os.path.isdir(os.path.join(_REF_INSTALL, "novadit")):
            raise RuntimeError(
                "the block-stack harness stacks the reference's own NovaDiTBlock: make the `novadit` package "
                "importable (pip install it, put it on PYTHONPATH, or install it into baseline/_ref)") from None
        sys.path.append(_REF_INSTALL)
        mods = importlib.import_module("novadit.modules")
    ref_ops = importlib.import_module("novadit.ops")
    if not ref_ops.HAS_NOVADIT_CUDA or ref_ops.novadit_cuda is not ops.novadit_cuda:
        raise RuntimeError("novadit.ops did not pick up this library's novadit_cuda extension "
                           f"({ref_ops.NOVADIT_CUDA_IMPORT_ERROR!r})")
    return mods


class _GateFirstRefMLP(nn.Module):
    """PyTorch twin of the reference MLP with `use_fused_fc1_bias_act=True`. The reference's two MLP paths are
    different functions of the same weights: `fused_fc1_bias_act` gates with the FIRST half of fc1's output
    (value * act(gate), `novadit/ops/fc1_bias_act.py:55-68`), `fc1` + gate-act with the SECOND
    (`novadit/ops/gate_act.py:9-27`), and the module has no switch that evaluates the first one in PyTorch. This
    wrapper does, with the reference's own `fc1_bias_act_ref` and the wrapped module's parameters."""

    def __init__(self, mlp: nn.Module) -> None:
        super().__init__()
        self.mlp = mlp

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ref_ops = importlib.import_module("novadit.ops")
        m = self.mlp
        return m.fc2(ref_ops.fc1_bias_act_ref(x, m.fc1.weight, m.fc1.bias, m.activation))


class _FusedFc1MLP(nn.Module):
    """The reference MLP's fused-FC1 path with a backward pass that runs. The reference's
    `_FusedFc1BiasActFunction.backward` (`novadit/ops/fc1_bias_act.py:248-268`) re-enters autograd
    (`z.requires_grad_(True)` ... `y_ref.backward(dy)`) without enabling grad mode, which is off inside a
    Function's backward: under an ordinary `loss.backward()` it raises "element 0 of tensors does not require
    grad". So the training stack evaluates `fused_fc1_bias_act` through this library's mirror of the operator
    (same forward kernel, backward on the tcgen05 dz kernel) on the wrapped reference module's parameters; the
    reference's own Function is exercised forward-only by the drop-in test."""

    def __init__(self, mlp: nn.Module) -> None:
        super().__init__()
        self.mlp = mlp

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        m = self.mlp
        return m.fc2(ops.fused_fc1_bias_act(x, m.fc1.weight, m.fc1.bias, m.activation))


class AdaLNZeroBlock(nn.Module):
    """One DiT block with adaLN-Zero conditioning around the parts of an unchanged reference `NovaDiTBlock`."""

    def __init__(self, hidden_size: int, num_heads: int, mlp_ratio: float = 4.0, use_fused: bool = True,
                 use_fused_fc1_bias_act: bool = True, activation: str = "gelu", zero_init: bool = True,
                 device=None, dtype=None) -> None:
        super().__init__()
        ref = reference_modules()
        self.use_fused = use_fused
        self.body = ref.NovaDiTBlock(hidden_size, num_heads, mlp_ratio, attention_backend="sdpa",
                                     use_fused_adaln=use_fused, use_fused_qkv_pack=use_fused,
                                     use_fused_out_residual=use_fused, use_fused_gate_act=use_fused,
                                     device=device, dtype=dtype)
        self.body.mlp.activation = activation  # the reference block does not pass it to its MLP (dit_block.py:40-48)
        # `use_fused_fc1_bias_act` selects the MLP's function (gate = first half of fc1's output) for the fused and
        # the PyTorch stack alike; `use_fused` selects who evaluates it
        if use_fused_fc1_bias_act:
            self.mlp_branch = _FusedFc1MLP(self.body.mlp) if use_fused else _GateFirstRefMLP(self.body.mlp)
        else:
            self.mlp_branch = self.body.mlp
        self.modulation = nn.Linear(hidden_size, 6 * hidden_size, device=device, dtype=dtype)
        if zero_init:
            nn.init.zeros_(self.modulation.weight)
            nn.init.zeros_(self.modulation.bias)

    def forward(self, x: torch.Tensor, cond: torch.Tensor) -> torch.Tensor:
        shift_a, scale_a, gate_a, shift_m, scale_m, gate_m = self.modulation(F.silu(cond)).chunk(6, dim=-1)
        body = self.body
        residual = ops.fused_gated_residual if self.use_fused else ops.gated_residual_ref
        x = residual(x, body.attn(body._adaln(x, scale_a.contiguous(), shift_a.contiguous())), gate_a)
        x = residual(x, self.mlp_branch(body._adaln(x, scale_m.contiguous(), shift_m.contiguous())), gate_m)
        return x


class DiTStack(nn.Module):
    """`depth` adaLN-Zero blocks over a latent [B, S, H] and a conditioning vector [B, H] (DiT-XL/2: depth 28,
    H = 1152, 16 heads, mlp_ratio 4). `zero_init=False` draws the modulation weights N(0, 0.02) so that branches
    and their gradients are not identically zero (the meaningful parity check)."""

    def __init__(self, hidden_size: int = 1152, num_heads: int = 16, depth: int = 28, mlp_ratio: float = 4.0,
                 use_fused: bool = True, use_fused_fc1_bias_act: bool = True, activation: str = "gelu",
                 zero_init: bool = True, device=None, dtype=None) -> None:
        super().__init__()
        self.blocks = nn.ModuleList([
            AdaLNZeroBlock(hidden_size, num_heads, mlp_ratio, use_fused, use_fused_fc1_bias_act, activation,
                           zero_init, device, dtype)
            for _ in range(depth)
        ])

    def forward(self, x: torch.Tensor, cond: torch.Tensor) -> torch.Tensor:
        if not (self.blocks and self.blocks[0].use_fused):
            for block in self.blocks:
                x = block(x, cond)
            return x
        # Fused stack: the gated residual of a branch and the AdaLN of the NEXT branch are one kernel
        # (`ops.fused_residual_adaln`), also across block boundaries, so a block's MLP residual is applied by the
        # next block's first norm; only the very first norm and the very last residual run on their own. Same
        # values as block-by-block evaluation: the fused kernel rounds the residual stream exactly where the
        # separate kernel does.
        pending = None  # (branch, gate) whose residual has not been added to x yet
        for block in self.blocks:
            shift_a, scale_a, gate_a, shift_m, scale_m, gate_m = block.modulation(F.silu(cond)).chunk(6, dim=-1)
            body = block.body
            if pending is None:
                h = body._adaln(x, scale_a.contiguous(), shift_a.contiguous())
            else:
                x, h = ops.fused_residual_adaln(x, pending[0], pending[1], scale_a.contiguous(), shift_a.contiguous())
            x, h = ops.fused_residual_adaln(x, body.attn(h), gate_a, scale_m.contiguous(), shift_m.contiguous())
            pending = (block.mlp_branch(h), gate_m)
        return ops.fused_gated_residual(x, pending[0], pending[1])


@torch.no_grad()
def init_stack_(stack: DiTStack, seed: int = 0, std: float = 0.02, zero_init: bool = True) -> None:
    """Deterministic N(0, std) weights drawn on the CPU in fp32 in module order (biases zero, modulation layers zero
    when `zero_init`), so that two stacks built with the same seed hold the same bits."""
    gen = torch.Generator().manual_seed(seed)
    for name, p in stack.named_parameters():
        if name.endswith("bias") or (zero_init and ".modulation." in name):
            p.zero_()
        else:
            p.copy_((torch.randn(p.shape, generator=gen, dtype=torch.float32) * std).to(p.dtype))
