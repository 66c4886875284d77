"""The DiT block-stack harness (adaLN-Zero around the reference's own NovaDiTBlock): the stack on fused operators
against the same stack on the reference's PyTorch definitions. Needs the reference's Python package (an install
under baseline/_ref or an importable `novadit`); skipped without it."""
from __future__ import annotations

import importlib.util
import os

import pytest
import torch

from novadit_b200.modules import DiTStack, init_stack_, reference_modules

pytestmark = pytest.mark.gpu
DEV = "cuda"
_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if importlib.util.find_spec("novadit") is None and not os.path.isdir(os.path.join(_ROOT, "baseline", "_ref", "novadit")):
    pytest.skip("the reference's Python package is not importable", allow_module_level=True)


def rel_l2(a, b):
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def step(stack, x, cond, dy):
    y = stack(x, cond)
    return y, torch.autograd.grad(y, (x, cond, *stack.parameters()), dy)


@pytest.mark.parametrize("activation", ["gelu", "silu"])
@pytest.mark.parametrize("fused_fc1", [True, False])
def test_fused_stack_matches_pytorch_stack(activation, fused_fc1):
    h, heads, depth, b, s = 256, 4, 3, 3, 80
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(b, s, h, generator=gen).to(DEV, torch.bfloat16).requires_grad_(True)
    cond = torch.randn(b, h, generator=gen).to(DEV, torch.bfloat16).requires_grad_(True)
    dy = torch.randn(b, s, h, generator=gen).to(DEV, torch.bfloat16)
    stacks = []
    for fused in (True, False):
        st = DiTStack(h, heads, depth, use_fused=fused, use_fused_fc1_bias_act=fused_fc1, activation=activation,
                      zero_init=False, device=DEV, dtype=torch.bfloat16)
        init_stack_(st, seed=11, zero_init=False)
        stacks.append(st)
    yf, gf = step(stacks[0], x, cond, dy)
    yr, gr = step(stacks[1], x, cond, dy)
    # two bf16 pipelines that round at different points: a few bf16 steps per block, not more
    assert rel_l2(yf, yr) < 2e-2
    assert rel_l2(gf[0], gr[0]) < 3e-2 and rel_l2(gf[1], gr[1]) < 3e-2
    for (name, _), a, e in zip(stacks[0].named_parameters(), gf[2:], gr[2:]):
        assert rel_l2(a, e) < 5e-2, name


def test_zero_initialised_stack_is_the_identity():
    h, heads = 128, 2
    st = DiTStack(h, heads, depth=2, use_fused=True, zero_init=True, device=DEV, dtype=torch.bfloat16)
    init_stack_(st, seed=0, zero_init=True)
    x = torch.randn(2, 16, h, device=DEV).to(torch.bfloat16).requires_grad_(True)
    cond = torch.randn(2, h, device=DEV).to(torch.bfloat16).requires_grad_(True)
    y = st(x, cond)
    assert torch.equal(y, x)
    (dx,) = torch.autograd.grad(y, (x,), torch.ones_like(y))
    assert torch.equal(dx, torch.ones_like(dx))


def test_the_stack_is_made_of_the_reference_blocks():
    ref = reference_modules()
    st = DiTStack(128, 2, depth=1, use_fused=True, device=DEV, dtype=torch.bfloat16)
    body = st.blocks[0].body
    assert type(body) is ref.NovaDiTBlock and type(body).__module__ == "novadit.modules.dit_block"
    assert type(body.mlp).__module__ == "novadit.modules.dit_mlp" and body.mlp.use_fused_gate_act
    import novadit.ops as ref_ops
    import novadit_b200.ops as ops
    assert ref_ops.HAS_NOVADIT_CUDA and ref_ops.novadit_cuda is ops.novadit_cuda
