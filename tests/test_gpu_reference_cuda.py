"""This library against the REFERENCE's own CUDA kernels on the same GPU and the same seeded inputs.

The reference's extension is compiled from its sources by oracle/build_ref_cuda.py into oracle/_ref/ (module
`novadit_cuda_ref`, bindings `csrc/bindings.cpp:85-116`). It is the second pin of the oracle: the reference's
kernels must sit within the same bars of the oracle as this library's, and the two GPU implementations within
those bars of each other. Skipped when the extension has not been built (no checkout of the reference at hand).
"""
from __future__ import annotations

import importlib.util
import os

import pytest
import torch

from novadit_b200 import capi, synth
from oracle import novadit_oracle as oracle
from oracle.build_ref_cuda import out_path
from tests.helpers import HALF_MAX_ABS, HALF_REL_L2, F32_REL_L2

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ref():
    path = out_path()
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/novadit_cuda_ref is not built")
    spec = importlib.util.spec_from_file_location("novadit_cuda_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def close(a, b, what, max_abs=HALF_MAX_ABS, rel=HALF_REL_L2):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    ma, rl = oracle.max_abs(a, b), oracle.rel_l2(a, b)
    # two independently rounded 16-bit results may differ by one step (3.1e-2 above |v| = 4): allow that
    assert ma <= 2 * max_abs and rl <= rel, f"{what}: max_abs {ma:.3e} rel_l2 {rl:.3e}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(2, 256, 768), (32, 256, 1152), (3, 77, 1152)])
def test_adaln(ref, dtype, shape):
    b, s, h = shape
    x, scale, shift, dy = synth.norm_inputs(b, s, h, dtype, seed=11)
    xd, sd, hd, gd = (t.to(DEV) for t in (x, scale, shift, dy))
    ry, _, rmean, rinv = ref.fused_adaln_forward(xd, sd, hd, 1e-6)
    rdx = ref.fused_adaln_backward_dx(gd, xd, sd, rmean, rinv)
    rds, rdh = ref.fused_adaln_backward_dparam(gd, xd, rmean, rinv)
    my, mmean, minv = capi.norm_fwd("layer", xd, sd, hd, 1e-6)
    mdx, mds, mdh = capi.norm_bwd("layer", gd, xd, sd, mmean, minv)
    torch.cuda.synchronize()
    wy, wmean, winv = oracle.adaln_fwd(x, scale, shift, 1e-6)
    wdx, wds, wdh = oracle.adaln_bwd(dy, x, scale, 1e-6)
    for name, r, m, w in (("y", ry, my, wy), ("dx", rdx, mdx, wdx)):
        close(r, w, f"reference kernel vs oracle {name}")
        close(m, r, f"this library vs reference kernel {name}")
    for name, r, m, w in (("mean", rmean, mmean, wmean), ("invstd", rinv, minv, winv), ("dscale", rds, mds, wds),
                          ("dshift", rdh, mdh, wdh)):
        # the reference's kernels use the one-pass variance E[x^2] - mean^2 under --use_fast_math: looser on stats
        assert oracle.rel_l2(r.float().cpu().reshape(w.shape), w) <= 1e-3, f"reference kernel vs oracle {name}"
        assert oracle.rel_l2(m.float().cpu().reshape(w.shape), w) <= F32_REL_L2, f"this library vs oracle {name}"


@pytest.mark.parametrize("shape", [(2, 256, 768), (32, 256, 1152)])
def test_adarmsnorm(ref, shape):
    b, s, h = shape
    x, scale, shift, dy = synth.norm_inputs(b, s, h, torch.bfloat16, seed=12)
    xd, sd, hd, gd = (t.to(DEV) for t in (x, scale, shift, dy))
    ry, _, rinv = ref.fused_adarmsnorm_forward(xd, sd, hd, 1e-6)
    rdx = ref.fused_adarmsnorm_backward_dx(gd, xd, sd, rinv)
    rds, rdh = ref.fused_adarmsnorm_backward_dparam(gd, xd, rinv)
    my, minv = capi.norm_fwd("rms", xd, sd, hd, 1e-6)
    mdx, mds, mdh = capi.norm_bwd("rms", gd, xd, sd, None, minv)
    torch.cuda.synchronize()
    wy, winv = oracle.adarms_fwd(x, scale, shift, 1e-6)
    wdx, wds, wdh = oracle.adarms_bwd(dy, x, scale, 1e-6)
    for name, r, m, w in (("y", ry, my, wy), ("dx", rdx, mdx, wdx)):
        close(r, w, f"reference kernel vs oracle {name}")
        close(m, r, f"this library vs reference kernel {name}")
    for name, r, m, w in (("inv_rms", rinv, minv, winv), ("dscale", rds, mds, wds), ("dshift", rdh, mdh, wdh)):
        assert oracle.rel_l2(r.float().cpu().reshape(w.shape), w) <= 1e-3, f"reference kernel vs oracle {name}"
        assert oracle.rel_l2(m.float().cpu().reshape(w.shape), w) <= F32_REL_L2, f"this library vs oracle {name}"


@pytest.mark.parametrize("act,act_id", [("silu", 0), ("gelu", 1)])
def test_gate_act(ref, act, act_id):
    x, dy = synth.gate_act_inputs(2, 512, 4608, torch.bfloat16, seed=13)
    xd, gd = x.to(DEV), dy.to(DEV)
    ry = ref.fused_gate_act_forward(xd, act_id)
    rdz = ref.fused_gate_act_backward(gd, xd, act_id)
    my = capi.gate_act_fwd(xd, act)
    mdz = capi.gate_act_bwd(gd, xd, act)
    torch.cuda.synchronize()
    wy, wdz = oracle.gate_act_fwd(x, act), oracle.gate_act_bwd(dy, x, act)
    for name, r, m, w in (("y", ry, my, wy), ("dz", rdz, mdz, wdz)):
        close(r, w, f"reference kernel vs oracle {act} {name}")
        close(m, r, f"this library vs reference kernel {act} {name}")


def _graph_ms(fn, reps=10):
    """Milliseconds per call of fn(), replayed from a CUDA graph and timed with CUDA events."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def test_speed_beside_the_reference_kernels(ref, record_property):
    """The reference's kernels (built for sm_100) and this library's through the same pybind interface, outputs
    allocated by the call, on the same buffers: gate-act forward + backward at workload config 3 (inputs far
    larger than L2) and the AdaLN step at config 2 over 8 rotating buffer sets. The margins are wide on purpose (a
    shared GPU): gate-act must not be slower than the reference's kernel by more than 3 %, AdaLN at least twice as
    fast as its three launches."""
    import novadit_b200.ops as ops

    mine = ops.novadit_cuda
    x, dy = synth.gate_act_inputs(32, 1024, 4608, torch.bfloat16, seed=3)
    xd, gd = x.to(DEV), dy.to(DEV)
    for act, act_id in (("silu", 0), ("gelu", 1)):
        t_ref = _graph_ms(lambda: (ref.fused_gate_act_forward(xd, act_id), ref.fused_gate_act_backward(gd, xd, act_id)))
        t_mine = _graph_ms(lambda: (mine.fused_gate_act_forward(xd, act_id), mine.fused_gate_act_backward(gd, xd, act_id)))
        record_property(f"gate_act_{act}_fwd_bwd_ms_reference_vs_this", (t_ref, t_mine))
        assert t_mine <= 1.03 * t_ref, f"gate-act {act}: this library {t_mine * 1e3:.1f} us, reference {t_ref * 1e3:.1f} us"
    del xd, gd
    b, s, h = 32, 256, 1152
    x, scale, shift, dy = synth.norm_inputs(b, s, h, torch.bfloat16, seed=0)
    sets = [(torch.roll(x, i, 1).to(DEV), scale.to(DEV), shift.to(DEV), torch.roll(dy, i, 1).to(DEV)) for i in range(8)]

    def three_launches(mod):
        def run():
            for xs, sc, sh, g in sets:
                _, _, mean, inv = mod.fused_adaln_forward(xs, sc, sh, 1e-6)
                mod.fused_adaln_backward_dx(g, xs, sc, mean, inv)
                mod.fused_adaln_backward_dparam(g, xs, mean, inv)
        return run

    t_ref = _graph_ms(three_launches(ref)) / 8
    t_mine = _graph_ms(three_launches(mine)) / 8
    record_property("adaln_fwd_dx_dparam_ms_reference_vs_this", (t_ref, t_mine))
    assert t_mine <= 0.5 * t_ref, f"AdaLN step: this library {t_mine * 1e3:.1f} us, reference {t_ref * 1e3:.1f} us"
