"""Host-side mirror of `novadit/modules` plus the DiT-XL/2 block-stack harness of workload config 5.

`NovaDiTAttention`, `NovaDiTMLP` and `NovaDiTBlock` take the reference's constructor arguments and have its
forward signatures (`novadit/modules/dit_attention.py:10-80`, `dit_mlp.py:9-57`, `dit_block.py:11-71`), with the
operators coming from `novadit_b200.ops`. Differences, on purpose:

* attention always runs through `F.scaled_dot_product_attention` (the reference's "sdpa" backend,
  `novadit/attention/sdpa.py:7-27`); its flash-attn dispatch is outside the operator path;
* `use_fused_fc1_bias_act` is a constructor argument of the block (the reference has it on the MLP only,
  `dit_mlp.py:18`, and never passes it from the block);
* `use_fused_qkv_pack` / `use_fused_out_residual` select this library's kernels for the QKV split and the
  output residual add (in the reference the operators behind them raise on CUDA tensors: `ops/qkv_pack.py`,
  `ops/residual.py`).

`AdaLNZeroBlock` / `DiTStack` are the harness of config 5, which the reference does not have: the adaLN-Zero
conditioning of DiT (SiLU -> Linear(H, 6H), zero-initialised, giving shift / scale / gate for the attention and
the MLP branch) around an unchanged `NovaDiTBlock` body, stacked `depth` times. With `use_fused=False` every
operator is the PyTorch `*_ref` definition: that stack is the parity oracle and the timing baseline of the
harness.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from . import ops


class NovaDiTAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int | None = None, qkv_bias: bool = True,
                 out_bias: bool = True, dropout_p: float = 0.0, causal: bool = False,
                 attention_backend: str = "sdpa", use_fused_qkv_pack: bool = True,
                 use_fused_out_residual: bool = True, add_residual: bool = False, device=None, dtype=None) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.head_dim = head_dim or hidden_size // num_heads
        self.dropout_p, self.causal, self.add_residual = dropout_p, causal, add_residual
        self.use_fused_qkv_pack, self.use_fused_out_residual = use_fused_qkv_pack, use_fused_out_residual
        if self.num_heads * self.head_dim != hidden_size:
            raise ValueError("hidden_size must equal num_heads * head_dim")
        if attention_backend not in ("auto", "sdpa"):
            raise ValueError("only the sdpa attention backend is available here")
        self.qkv_proj = nn.Linear(hidden_size, 3 * hidden_size, bias=qkv_bias, **kw)
        self.out_proj = nn.Linear(hidden_size, hidden_size, bias=out_bias, **kw)

    def forward(self, x: torch.Tensor, attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        b, s, _ = x.shape
        qkv = self.qkv_proj(x)
        if self.use_fused_qkv_pack and qkv.is_cuda:
            q, k, v = ops.fused_qkv_pack(qkv, self.num_heads, self.head_dim)
        else:
            q, k, v = qkv.view(b, s, 3, self.num_heads, self.head_dim).unbind(dim=2)
        out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                             attn_mask=attention_mask,
                                             dropout_p=self.dropout_p if self.training else 0.0,
                                             is_causal=self.causal)
        out = self.out_proj(out.transpose(1, 2).reshape(b, s, self.hidden_size))
        if not self.add_residual:
            return F.dropout(out, self.dropout_p, self.training) if self.dropout_p > 0 else out
        if self.dropout_p == 0.0 and self.use_fused_out_residual and out.is_cuda:
            return ops.fused_out_residual(out, x, None)
        return x + F.dropout(out, self.dropout_p, self.training)


class NovaDiTMLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", bias: bool = True,
                 dropout_p: float = 0.0, use_fused_gate_act: bool = True, use_fused_fc1_bias_act: bool = False,
                 add_residual: bool = False, device=None, dtype=None, fc1_gate_first: bool = False) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.activation, self.dropout_p, self.add_residual = activation, dropout_p, add_residual
        self.use_fused_gate_act, self.use_fused_fc1_bias_act = use_fused_gate_act, use_fused_fc1_bias_act
        # The reference's two MLP paths are different functions of the same weights: `fused_fc1_bias_act` gates
        # with the FIRST half of fc1's output (value * act(gate), ops/fc1_bias_act.py:55-68), `fc1` + gate-act
        # with the SECOND (up * act(gate), ops/gate_act.py). `fc1_gate_first` makes the unfused path evaluate the
        # first convention (through `fc1_bias_act_ref`), so that a fused-FC1 stack has a PyTorch twin.
        self.fc1_gate_first = fc1_gate_first
        self.fc1 = nn.Linear(hidden_size, 2 * intermediate_size, bias=bias, **kw)
        self.fc2 = nn.Linear(intermediate_size, hidden_size, bias=bias, **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        residual = x
        if self.use_fused_fc1_bias_act:
            x = ops.fused_fc1_bias_act(x, self.fc1.weight, self.fc1.bias, self.activation)
        elif self.fc1_gate_first:
            x = ops.fc1_bias_act_ref(x, self.fc1.weight, self.fc1.bias, self.activation)
        else:
            x = self.fc1(x)
            x = (ops.fused_gate_act if self.use_fused_gate_act else ops.gate_act_ref)(x, activation=self.activation)
        x = self.fc2(x)
        if self.dropout_p > 0:
            x = F.dropout(x, self.dropout_p, self.training)
        return residual + x if self.add_residual else x


class NovaDiTBlock(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, mlp_ratio: float = 4.0, dropout_p: float = 0.0,
                 attention_backend: str = "sdpa", use_fused_adaln: bool = True, use_fused_qkv_pack: bool = True,
                 use_fused_out_residual: bool = True, use_fused_gate_act: bool = True,
                 use_fused_fc1_bias_act: bool = False, activation: str = "silu", device=None, dtype=None,
                 fc1_gate_first: bool = False) -> None:
        super().__init__()
        self.use_fused_adaln = use_fused_adaln
        self.attn = NovaDiTAttention(hidden_size, num_heads, dropout_p=dropout_p, attention_backend=attention_backend,
                                     use_fused_qkv_pack=use_fused_qkv_pack,
                                     use_fused_out_residual=use_fused_out_residual, add_residual=False,
                                     device=device, dtype=dtype)
        self.mlp = NovaDiTMLP(hidden_size, int(hidden_size * mlp_ratio), activation=activation, dropout_p=dropout_p,
                              use_fused_gate_act=use_fused_gate_act, use_fused_fc1_bias_act=use_fused_fc1_bias_act,
                              add_residual=False, device=device, dtype=dtype, fc1_gate_first=fc1_gate_first)

    def _adaln(self, x, scale, shift):
        return (ops.fused_adaln if self.use_fused_adaln else ops.adaln_ref)(x, scale, shift)

    def forward(self, x, attn_scale, attn_shift, mlp_scale, mlp_shift, attention_mask=None):
        x = x + self.attn(self._adaln(x, attn_scale, attn_shift), attention_mask=attention_mask)
        x = x + self.mlp(self._adaln(x, mlp_scale, mlp_shift))
        return x


class AdaLNZeroBlock(nn.Module):
    """One DiT block with adaLN-Zero conditioning around the body of `NovaDiTBlock`."""

    def __init__(self, hidden_size: int, num_heads: int, mlp_ratio: float = 4.0, use_fused: bool = True,
                 use_fused_fc1_bias_act: bool = True, activation: str = "gelu", zero_init: bool = True,
                 device=None, dtype=None) -> None:
        super().__init__()
        self.use_fused = use_fused
        # `use_fused_fc1_bias_act` selects the MLP's function (gate = first half of fc1's output) for the fused and
        # the PyTorch stack alike; `use_fused` selects who evaluates it
        self.body = NovaDiTBlock(hidden_size, num_heads, mlp_ratio, use_fused_adaln=use_fused,
                                 use_fused_qkv_pack=False, use_fused_out_residual=use_fused,
                                 use_fused_gate_act=use_fused, use_fused_fc1_bias_act=use_fused and use_fused_fc1_bias_act,
                                 activation=activation, device=device, dtype=dtype,
                                 fc1_gate_first=use_fused_fc1_bias_act)
        self.modulation = nn.Linear(hidden_size, 6 * hidden_size, device=device, dtype=dtype)
        if zero_init:
            nn.init.zeros_(self.modulation.weight)
            nn.init.zeros_(self.modulation.bias)

    def forward(self, x: torch.Tensor, cond: torch.Tensor) -> torch.Tensor:
        shift_a, scale_a, gate_a, shift_m, scale_m, gate_m = self.modulation(F.silu(cond)).chunk(6, dim=-1)
        body = self.body
        residual = ops.fused_gated_residual if self.use_fused else ops.gated_residual_ref
        x = residual(x, body.attn(body._adaln(x, scale_a.contiguous(), shift_a.contiguous())), gate_a)
        x = residual(x, body.mlp(body._adaln(x, scale_m.contiguous(), shift_m.contiguous())), gate_m)
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
        for block in self.blocks:
            x = block(x, cond)
        return x


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
