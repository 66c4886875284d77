"""The no-allocation AdaLN backward (`nd_adaln_bwd_noalloc`) against the regular entry point.

It exists for callers that cannot give the library scratch memory (all device memory already in
their own pool, allocations forbidden by a plugin host, or a call site such as a stream capture
where cudaMalloc is not allowed), so its partial sums go through a fixed array inside the library.
The file name keeps this test last in collection order.
"""
from __future__ import annotations

import pytest
import torch

from novadit_b200 import capi, synth

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(b, s, h, seed):
    x, scale, shift, dy = (t.to(DEV) for t in synth.norm_inputs(b, s, h, torch.bfloat16, seed))
    _, mean, invstd = capi.norm_fwd("layer", x, scale, shift, 1e-6)
    return x, scale, dy, mean, invstd


def _noalloc_bwd(x, scale, dy, mean, invstd):
    b, s, h = x.shape
    dx = torch.empty_like(x)
    dscale = torch.full((b, h), float("nan"), dtype=torch.float32, device=DEV)
    dshift = torch.full((b, h), float("nan"), dtype=torch.float32, device=DEV)
    rc = capi.lib().nd_adaln_bwd_noalloc(capi.ND_BF16, dy.data_ptr(), x.data_ptr(), scale.data_ptr(), mean.data_ptr(),
                                         invstd.data_ptr(), dx.data_ptr(), dscale.data_ptr(), dshift.data_ptr(),
                                         b * s, 0, s, h, torch.cuda.current_stream().cuda_stream)
    capi.check(rc, "nd_adaln_bwd_noalloc")
    torch.cuda.synchronize()
    return dx, dscale, dshift


def test_no_alloc_backward_equals_regular_backward_twice_in_a_row():
    # two different problems back to back: the second call finds the first one's leftovers in the scratch
    for b, s, h, seed in [(32, 256, 1152, 0), (3, 77, 768, 1)]:
        x, scale, dy, mean, invstd = _inputs(b, s, h, seed)
        want_dx, want_ds, want_dh = capi.norm_bwd("layer", dy, x, scale, mean, invstd)
        torch.cuda.synchronize()
        got_dx, got_ds, got_dh = _noalloc_bwd(x, scale, dy, mean, invstd)
        # same kernels and the same fixed summation order: the results are bit-identical
        assert torch.equal(got_dx, want_dx)
        assert torch.equal(got_ds, want_ds) and torch.equal(got_dh, want_dh)


def test_no_alloc_backward_refuses_what_does_not_fit():
    L = capi.lib()
    assert L.nd_noalloc_scratch_bytes() == 16 << 20
    # hidden = 4096 needs (148 * 8 + B) slots of 32 KiB: far more than the built-in 16 MiB
    rows, s, h = 64, 8, 4096
    assert L.nd_norm_dparam_ws_bytes(rows, 0, s, h) > L.nd_noalloc_scratch_bytes()
    # real tensors of the right sizes: if the size check ever regressed, the call would run on valid memory and
    # show up as a wrong return code, not as a device fault
    x, scale, dy, mean, invstd = _inputs(rows // s, s, h, 2)
    dx = torch.empty_like(x)
    dscale = torch.zeros(rows // s, h, dtype=torch.float32, device=DEV)
    dshift = torch.zeros_like(dscale)
    rc = L.nd_adaln_bwd_noalloc(capi.ND_BF16, dy.data_ptr(), x.data_ptr(), scale.data_ptr(), mean.data_ptr(),
                                invstd.data_ptr(), dx.data_ptr(), dscale.data_ptr(), dshift.data_ptr(), rows, 0, s, h,
                                torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == -6 and b"too large" in L.nd_status_string(rc)
    assert L.nd_adaln_bwd_noalloc(capi.ND_BF16, None, None, None, None, None, None, None, None, 0, 0, s, h, None) == 0
