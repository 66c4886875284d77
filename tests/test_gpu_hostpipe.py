"""Host-buffer pipeline: results of overlapped steps equal those of the same steps run one by one."""
from __future__ import annotations

import pytest
import torch

import novadit_b200.ops as ops
from novadit_b200 import synth
from novadit_b200.hostpipe import HostPipeline, adaln_train_step

pytestmark = pytest.mark.gpu
DEV = "cuda"


def direct(host, eps):
    x, scale, shift, dy = (t.to(DEV) for t in host)
    x.requires_grad_(True)
    scale.requires_grad_(True)
    shift.requires_grad_(True)
    y = ops.fused_adaln(x, scale, shift, eps)
    y.backward(dy)
    return [t.cpu() for t in (y.detach(), x.grad, scale.grad, shift.grad)]


def test_overlapped_steps_match_serial_steps():
    eps = 1e-6
    batches = [[t.pin_memory() for t in synth.norm_inputs(4, 96, 1152, torch.bfloat16, seed=s)] for s in range(7)]
    want = [direct(b, eps) for b in batches]
    pipe = HostPipeline(adaln_train_step(eps), DEV, depth=3)
    got = {}
    tickets = []
    for i, b in enumerate(batches):  # more steps than slots: every slot is reused, results read late
        tickets.append(pipe.submit(b))
        if i >= 2:
            t = tickets[i - 2]
            got[t] = [o.clone() for o in pipe.result(t)]
    for t in tickets[-2:]:
        got[t] = [o.clone() for o in pipe.result(t)]
    pipe.drain()
    for t, w in zip(tickets, want):
        for g, e in zip(got[t], w):
            assert torch.equal(g, e), f"step {t}: pipelined result differs from the serial one"


def test_rejects_pageable_host_memory_and_stale_tickets():
    pipe = HostPipeline(adaln_train_step(), DEV, depth=2)
    batch = list(synth.norm_inputs(1, 8, 128, torch.bfloat16, seed=0))
    with pytest.raises(ValueError):
        pipe.submit(batch)  # not pinned
    pinned = [t.pin_memory() for t in batch]
    t0 = pipe.submit(pinned)
    pipe.submit(pinned)
    pipe.submit(pinned)
    with pytest.raises(ValueError):
        pipe.result(t0)  # its slot has been reused
    pipe.drain()
