"""The DiT block-stack harness: the stack on fused operators against the same stack on the PyTorch definitions."""
from __future__ import annotations

import pytest
import torch

from novadit_b200.modules import DiTStack, NovaDiTBlock, init_stack_

pytestmark = pytest.mark.gpu
DEV = "cuda"


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


def test_block_has_the_reference_signature():
    blk = NovaDiTBlock(128, 2, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(2, 8, 128, device=DEV).to(torch.bfloat16)
    m = [torch.randn(2, 128, device=DEV).to(torch.bfloat16) * 0.1 for _ in range(4)]
    y = blk(x, *m)
    ref = NovaDiTBlock(128, 2, use_fused_adaln=False, use_fused_gate_act=False, device=DEV, dtype=torch.bfloat16)
    ref.load_state_dict(blk.state_dict())
    assert rel_l2(y, ref(x, *m)) < 2e-2
