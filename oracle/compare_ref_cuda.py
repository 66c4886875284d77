"""Speed of the REFERENCE's own CUDA kernels beside this library's, on the same GPU, shapes and buffers.

    python oracle/compare_ref_cuda.py            # needs oracle/_ref/novadit_cuda_ref*.so (oracle/build_ref_cuda.py)

Test infrastructure (a comparator for the design notes), not part of the product and not used by bench.py.
Both sides run through the same kind of entry point - the 15-function pybind interface
(`csrc/bindings.cpp:85-116`; this repository's `novadit_cuda` mirrors it), outputs allocated by the call as the
reference's API does - with every step replayed from a CUDA graph over 8 rotating buffer sets (605 MB, larger
than 4x the L2) and timed with CUDA events. The reference's backward is its two launches (dx, dparam); this
library is timed both that way and with its one-pass backward. Bytes are the algorithmic bytes of the step
(every tensor moved once), so the GB/s of the two sides are directly comparable.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from novadit_b200 import synth  # noqa: E402
from oracle.build_ref_cuda import out_path  # noqa: E402

NSETS = 8


def load_reference():
    spec = importlib.util.spec_from_file_location("novadit_cuda_ref", out_path())
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def time_graph(fn, reps=20) -> float:
    """Milliseconds per call of fn() (fn runs all NSETS sets), replayed from a CUDA graph."""
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


def main() -> None:
    import novadit_b200.ops as ops

    if not ops.HAS_NOVADIT_CUDA:
        raise SystemExit("novadit_cuda (this repository's extension) is not built")
    mine = ops.novadit_cuda
    ref = load_reference()
    dev = "cuda"
    b, s, h, e = 32, 256, 1152, 2
    rows = b * s
    step_bytes = (2 * rows * h * e + 2 * b * h * e + 2 * rows * 4) + (3 * rows * h * e + b * h * e + 2 * rows * 4 + 2 * b * h * 4)
    x, scale, shift, dy = synth.norm_inputs(b, s, h, torch.bfloat16, seed=0)
    sets = [(torch.roll(x, i, 1).to(dev), scale.to(dev), shift.to(dev), torch.roll(dy, i, 1).to(dev)) for i in range(NSETS)]

    def adaln_two_launch(mod):
        def run():
            for xs, sc, sh, g in sets:
                y, _, mean, inv = mod.fused_adaln_forward(xs, sc, sh, 1e-6)
                mod.fused_adaln_backward_dx(g, xs, sc, mean, inv)
                mod.fused_adaln_backward_dparam(g, xs, mean, inv)
        return run

    def adaln_one_pass():
        for xs, sc, sh, g in sets:
            y, _, mean, inv = mine.fused_adaln_forward(xs, sc, sh, 1e-6)
            mine.fused_adaln_backward(g, xs, sc, mean, inv)

    def rms_two_launch(mod):
        def run():
            for xs, sc, sh, g in sets:
                y, _, inv = mod.fused_adarmsnorm_forward(xs, sc, sh, 1e-6)
                mod.fused_adarmsnorm_backward_dx(g, xs, sc, inv)
                mod.fused_adarmsnorm_backward_dparam(g, xs, inv)
        return run

    print(f"device: {torch.cuda.get_device_name(0)}; config 2: x [{b},{s},{h}] bf16, {step_bytes} algorithmic bytes per step")
    for name, fn, nbytes in (
        ("AdaLN fwd + dx + dparam, reference kernels", adaln_two_launch(ref), step_bytes),
        ("AdaLN fwd + dx + dparam, this library (same three calls)", adaln_two_launch(mine), step_bytes),
        ("AdaLN fwd + one-pass backward, this library", adaln_one_pass, step_bytes),
        ("AdaRMSNorm fwd + dx + dparam, reference kernels", rms_two_launch(ref), step_bytes - 2 * rows * 4),
        ("AdaRMSNorm fwd + dx + dparam, this library", rms_two_launch(mine), step_bytes - 2 * rows * 4),
    ):
        ms = time_graph(fn) / NSETS
        print(f"{name}: {ms * 1e3:.1f} us per step, {nbytes / ms / 1e6:.0f} GB/s")
    del sets

    # gate-act, config 3: [8 * 4096, 2 * 4608] bf16 (604 MB input: larger than L2 by itself)
    rows, inter = 8 * 4096, 4608
    xg, dyg = synth.gate_act_inputs(1, 2048, inter, torch.bfloat16, seed=3)
    xg = xg.to(dev).repeat(rows // 2048, 1, 1).reshape(8, rows // 8, 2 * inter).contiguous()
    dyg = dyg.to(dev).repeat(rows // 2048, 1, 1).reshape(8, rows // 8, inter).contiguous()
    nbytes = 8 * rows * inter * e
    for act_id, act in ((0, "SiLU"), (1, "GELU-tanh")):
        for name, mod in (("reference kernels", ref), ("this library", mine)):
            def run(mod=mod, act_id=act_id):
                mod.fused_gate_act_forward(xg, act_id)
                mod.fused_gate_act_backward(dyg, xg, act_id)
            ms = time_graph(run, reps=10)
            print(f"gate-act {act} fwd + bwd, {name}: {ms * 1e3:.1f} us, {nbytes / ms / 1e6:.0f} GB/s")


if __name__ == "__main__":
    main()
