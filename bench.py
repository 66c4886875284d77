"""Benchmark of the operator hot path: AdaLN forward + backward at the DiT-XL/2 shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one pass of the hot path over one batch of synthetic input: AdaLN forward
(y + fp32 statistics) followed by the one-pass backward (dx + fp32 dscale/dshift) on
x [B=32, S=256, H=1152] bf16, eps 1e-6 (workload config 2). The headline metric is algorithmic
HBM bytes per second. With N > 1 every rank runs its own batch of that shape (rows sharded, no
data-path collective: whole samples per GPU), so scaling is weak and the value is the sum over
ranks divided by the slowest rank's time.

Timing: CUDA events on the launching stream, barrier + synchronize on both sides, max over
ranks. The 76 MB working set of one step would sit in the 126 MB L2, so the steps rotate through
8 independent buffer sets (605 MB): every step reads its inputs from HBM. Steps are replayed
from CUDA graphs because one step is ~20 us of GPU work.

The JSON line also carries: `roofline` for the dominant kernel (the fused backward), `e2e`
(the same step through the public `novadit_b200.ops` API from pinned HOST buffers, copies inside
the timed region), `cpu_baseline` (the CPU oracle's restatement of the reference's PyTorch path,
timed on this box's cores), `clocks`, and `extras` with the other operators of the path
(AdaRMSNorm, gate-act at config 3, FC1 at config 4 in bf16 and FP8).

`--impl reference` times the reference's own CPU implementation of the step (the oracle port:
the reference is Python and is not installed on the benchmark box) and prints the same line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "adaln_fwd_bwd_hbm_gbs"
UNIT = "GB/s"
B, S, H = 32, 256, 1152          # workload config 2
EPS = 1e-6
NSETS = 8                         # rotating buffer sets (8 x 75.6 MB > 4 x L2)
E = 2                             # bytes per bf16 element
ROWS = B * S
# algorithmic bytes of one launch (compulsory traffic, every tensor moved once)
FWD_BYTES = 2 * ROWS * H * E + 2 * B * H * E + 2 * ROWS * 4                       # 37 961 728
BWD_BYTES = 3 * ROWS * H * E + B * H * E + 2 * ROWS * 4 + 2 * B * H * 4           # 57 057 280
STEP_BYTES = FWD_BYTES + BWD_BYTES                                                # 95 019 008
WORKLOAD = "config2: AdaLN fwd+bwd, x [32,256,1152] bf16, eps 1e-6"   # the same string in both arms
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "norm_config2_traffic.json")


def measured_traffic() -> tuple[int | None, dict | None]:
    """DRAM bytes per launch of the dominant kernel from the tracked ncu record (read + written), and the record
    itself (it names the capture's command and the commit it was taken at). None when the file is absent."""
    try:
        with open(TRAFFIC_FILE) as f:
            rec = json.load(f)
        return int(rec["dram_bytes_read"]) + int(rec["dram_bytes_write"]), rec
    except Exception:
        return None, None


def measured_peaks() -> tuple[float, float, str]:
    """(HBM GB/s, bf16 TFLOP/s burst, source) from MEASURED_PEAKS.json, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def measured_sustained_tflops(burst: float) -> float:
    """bf16 TFLOP/s of a seconds-long cuBLAS loop under the power cap (MEASURED_PEAKS.json), else 0.88 x burst."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"])
    except Exception:
        return 0.88 * burst


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only) every 10 ms in a thread."""

    def __init__(self, index: int) -> None:
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self) -> None:
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.01)

    def start(self) -> None:
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
        med = int(statistics.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------ CPU arm (reference path on host cores)
def cpu_reference_step_time(steps: int, warmup: int, budget_s: float | None = None) -> tuple[float, int, int]:
    """Median seconds of one fwd+bwd step of the reference's PyTorch CPU path (oracle port) at config 2.

    Returns (median seconds per step, steps run, threads). With `budget_s` the loop stops early once
    that much time has been spent (the bounded sample of the GPU arm's `cpu_baseline`)."""
    from novadit_b200 import synth
    from oracle import novadit_oracle as oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    x, scale, shift, dy = synth.norm_inputs(B, S, H, torch.bfloat16, seed=0)
    for _ in range(max(1, warmup)):
        oracle.cpu_path_norm_fwd_bwd(x, scale, shift, dy, EPS, "layer")
    times = []
    t_begin = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        oracle.cpu_path_norm_fwd_bwd(x, scale, shift, dy, EPS, "layer")
        times.append(time.perf_counter() - t0)
        if budget_s is not None and time.perf_counter() - t_begin > budget_s:
            break
    return statistics.median(times), len(times), threads


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # under torchrun rank 0 alone runs the CPU arm
    steps = max(1, min(args.steps, 200))  # ~80 ms per step on 8 cores: bounded to stay within minutes
    sec, ran, threads = cpu_reference_step_time(steps, max(1, min(args.warmup, 5)))
    value = STEP_BYTES / sec / 1e9
    sample = f"{ran} full steps of config 2 (B={B}, S={S}, H={H} bf16 inputs, fp32 math), median"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": ran, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD}, "setup": {"where": "host CPU"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
def event_time_ms(fn, stream) -> float:
    """Run fn() bracketed by CUDA events on `stream`; returns elapsed milliseconds."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    fn()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def capture(fn) -> torch.cuda.CUDAGraph:
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


def replay_steps(big, singles, k: int) -> None:
    """Exactly k steps: whole-rotation graphs (NSETS steps each) plus single-step graphs for the remainder."""
    for _ in range(k // NSETS):
        big.replay()
    for i in range(k % NSETS):
        singles[i].replay()


GRAPH_STEPS = 256  # steps per graph of the timed region (a whole number of rotations)


class StepGraphs:
    """Graphs that replay EXACTLY k steps with no single-step launches: k // 256 replays of a 256-step graph and
    one graph holding the remaining k % 256 steps (graph launches cost the host ~10 us each, which shows when a
    graph holds one 27 us step)."""

    def __init__(self, work: "NormWorkload", k: int) -> None:
        self.whole = k // GRAPH_STEPS
        rest = k % GRAPH_STEPS
        self.big = capture(lambda: [work.step(work.sets[i % NSETS]) for i in range(GRAPH_STEPS)]) if self.whole else None
        self.rest = capture(lambda: [work.step(work.sets[i % NSETS]) for i in range(rest)]) if rest else None

    def replay(self) -> None:
        for _ in range(self.whole):
            self.big.replay()
        if self.rest is not None:
            self.rest.replay()


class NormWorkload:
    """NSETS independent buffer sets of the config-2 shape and the graphs that run them."""

    def __init__(self, kind: str, dev) -> None:
        from novadit_b200 import capi, synth

        self.capi, self.kind = capi, kind
        x, scale, shift, dy = synth.norm_inputs(B, S, H, torch.bfloat16, seed=0)
        self.sets = []
        for i in range(NSETS):
            # every set gets distinct bits (roll) so that no two sets can alias in a cache
            xs, gs = torch.roll(x, i, 1).to(dev), torch.roll(dy, i, 1).to(dev)
            self.sets.append({
                "x": xs, "dy": gs, "scale": scale.to(dev), "shift": shift.to(dev),
                "y": torch.empty_like(xs), "dx": torch.empty_like(xs),
                "mean": torch.empty(B, S, dtype=torch.float32, device=dev),
                "invstd": torch.empty(B, S, dtype=torch.float32, device=dev),
                "dscale": torch.empty(B, H, dtype=torch.float32, device=dev),
                "dshift": torch.empty(B, H, dtype=torch.float32, device=dev),
            })

    def fwd(self, s) -> None:
        self.capi.norm_fwd(self.kind, s["x"], s["scale"], s["shift"], EPS, y=s["y"],
                           mean=s["mean"] if self.kind == "layer" else None, invstd=s["invstd"])

    def bwd(self, s) -> None:
        self.capi.norm_bwd(self.kind, s["dy"], s["x"], s["scale"], s["mean"] if self.kind == "layer" else None,
                           s["invstd"], dx=s["dx"], dscale=s["dscale"], dshift=s["dshift"])

    def step(self, s) -> None:
        self.fwd(s)
        self.bwd(s)

    def graphs(self):
        for s in self.sets[:2]:
            self.step(s)  # allocate the workspace and load the kernels before capture
        torch.cuda.synchronize()
        big = capture(lambda: [self.step(s) for s in self.sets])
        singles = [capture(lambda s=s: self.step(s)) for s in self.sets]
        fwd_only = capture(lambda: [self.fwd(s) for s in self.sets])
        bwd_only = capture(lambda: [self.bwd(s) for s in self.sets])
        return big, singles, fwd_only, bwd_only


def time_graph_loop(graph, reps: int, stream) -> float:
    """Average milliseconds of one replay of `graph` over `reps` back-to-back replays."""
    for _ in range(3):
        graph.replay()
    return event_time_ms(lambda: [graph.replay() for _ in range(reps)], stream) / reps


def bench_extras(dev, stream, hbm_peak: float, tf_peak: float, tf_sustained: float) -> dict:
    """The other operators of the path, each timed alone (cold inputs by rotation or size > L2)."""
    from novadit_b200 import capi, synth

    out = {}
    # AdaRMSNorm, same shape and rotation as the headline
    rms = NormWorkload("rms", dev)
    big, _, _, _ = rms.graphs()
    ms = time_graph_loop(big, 20, stream) / NSETS
    rms_bytes = STEP_BYTES - 2 * ROWS * 4  # no mean array in either pass
    out["adarmsnorm_fwd_bwd"] = {"GB/s": rms_bytes / ms / 1e6, "ms_per_step": ms,
                                 "frac_of_hbm_peak": rms_bytes / ms / 1e6 / hbm_peak}
    del rms, big

    # the same step in eager PyTorch on this GPU (`adaln_ref` + autograd: what the reference runs on a GPU without its
    # extension), over the same rotation of buffer sets
    import novadit_b200.ops as ops

    work = NormWorkload("layer", dev)

    def eager_steps():
        for st in work.sets:
            xg, sg, hg = st["x"].requires_grad_(True), st["scale"].requires_grad_(True), st["shift"].requires_grad_(True)
            torch.autograd.grad(ops.adaln_ref(xg, sg, hg, EPS), (xg, sg, hg), st["dy"])

    for _ in range(2):
        eager_steps()
    torch.cuda.synchronize()
    ms = event_time_ms(lambda: [eager_steps() for _ in range(3)], stream) / (3 * NSETS)
    out["adaln_fwd_bwd_pytorch_eager_cuda"] = {"GB/s": STEP_BYTES / ms / 1e6, "ms_per_step": ms}
    del work

    # the gated residual in front of the norm: one launch (x_new = x + gate * branch, then AdaLN of x_new) against
    # the two launches it replaces, over the same rotation of buffer sets (branch = the set's dy tensor)
    work = NormWorkload("layer", dev)
    gate = (torch.randn(B, H, device=dev) * 0.5).to(torch.bfloat16)

    def fused_all():
        for st in work.sets:
            capi.norm_fwd_residual("layer", st["x"], st["dy"], gate, st["scale"], st["shift"], EPS)

    def split_all():
        for st in work.sets:
            xn = capi.gated_residual_fwd(st["x"], st["dy"], gate)
            capi.norm_fwd("layer", xn, st["scale"], st["shift"], EPS)

    fused_all()
    split_all()
    ms_f = time_graph_loop(capture(fused_all), 20, stream) / NSETS
    ms_s = time_graph_loop(capture(split_all), 20, stream) / NSETS
    res_bytes = 4 * ROWS * H * 2  # x, branch in; x_new, y out
    out["residual_adaln_fwd_fused"] = {"ms": ms_f, "GB/s": res_bytes / ms_f / 1e6,
                                       "two_launches_ms": ms_s, "speedup_vs_two_launches": ms_s / ms_f}
    del work

    # the same kernels on 16 x the rows (B = 512: 131 072 rows, 302 MB per tensor, two buffer sets): where launch
    # and first-byte latency stop mattering
    big_b = 16 * B
    xb = torch.randn(big_b, S, H, device=dev).to(torch.bfloat16)
    gb = torch.randn(big_b, S, H, device=dev).to(torch.bfloat16)
    sb = (torch.randn(big_b, H, device=dev) * 0.1).to(torch.bfloat16)
    hb = (torch.randn(big_b, H, device=dev) * 0.1).to(torch.bfloat16)
    big_sets = []
    for _ in range(2):
        big_sets.append({"x": xb.clone(), "dy": gb.clone(), "y": torch.empty_like(xb), "dx": torch.empty_like(xb),
                         "mean": torch.empty(big_b, S, dtype=torch.float32, device=dev),
                         "invstd": torch.empty(big_b, S, dtype=torch.float32, device=dev),
                         "dscale": torch.empty(big_b, H, dtype=torch.float32, device=dev),
                         "dshift": torch.empty(big_b, H, dtype=torch.float32, device=dev)})
    del xb, gb

    def big_step():
        for st in big_sets:
            capi.norm_fwd("layer", st["x"], sb, hb, EPS, y=st["y"], mean=st["mean"], invstd=st["invstd"])
            capi.norm_bwd("layer", st["dy"], st["x"], sb, st["mean"], st["invstd"], dx=st["dx"], dscale=st["dscale"],
                          dshift=st["dshift"])

    big_step()
    ms = time_graph_loop(capture(big_step), 5, stream) / 2
    big_bytes = 16 * STEP_BYTES
    out["adaln_fwd_bwd_131072_rows"] = {"GB/s": big_bytes / ms / 1e6, "ms_per_step": ms,
                                        "frac_of_hbm_peak": big_bytes / ms / 1e6 / hbm_peak}
    del big_sets

    # gate-act, workload config 3: x [8, 4096, 2*4608] bf16 (604 MB, far larger than L2)
    rows, inter = 8 * 4096, 4608
    x, dy = synth.gate_act_inputs(1, 2048, inter, torch.bfloat16, seed=3)
    xg = x.to(dev).repeat(rows // 2048, 1, 1).reshape(rows, 2 * inter).contiguous()
    dyg = dy.to(dev).repeat(rows // 2048, 1, 1).reshape(rows, inter).contiguous()
    yg, dzg = torch.empty_like(dyg), torch.empty_like(xg)
    for act in ("silu", "gelu"):
        capi.gate_act_fwd(xg, act, y=yg)
        capi.gate_act_bwd(dyg, xg, act, dz=dzg)
        g = capture(lambda: (capi.gate_act_fwd(xg, act, y=yg), capi.gate_act_bwd(dyg, xg, act, dz=dzg)))
        ms = time_graph_loop(g, 10, stream)
        nbytes = 8 * rows * inter * E  # fwd 3 + bwd 5 tensors of rows x I
        out[f"gate_act_{act}_fwd_bwd"] = {"GB/s": nbytes / ms / 1e6, "ms_per_step": ms,
                                         "frac_of_hbm_peak": nbytes / ms / 1e6 / hbm_peak}
    del xg, dyg, yg, dzg

    # FC1, workload config 4: M=8192, K=1152, N=4608, bias, GELU-tanh; gated (reference semantics) and plain
    m, k, n = 8192, 1152, 4608
    xf, wf, bf = (t.to(dev) for t in synth.fc1_inputs(m, k, n, torch.bfloat16, seed=0))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    flops = 2.0 * m * k * n
    qx, sx = capi.quantize_e4m3(xf)
    qw, sw = capi.quantize_e4m3(wf)
    scales = torch.cat([sx, sw])
    # Library comparators on the same box, timed the same way: cuBLASLt bf16 (F.linear + eager GELU gating, what the
    # reference's fc1_bias_act_ref runs on a GPU) at this shape, and an FP8 e4m3 GEMM of 8192^3 through
    # torch._scaled_mm as the measured FP8 peak (no FP8 figure exists among the driver-measured peaks).
    import torch.nn.functional as F

    def ref_gated():
        z = F.linear(xf, wf, bf)
        return z[:, n // 2:] * F.gelu(z[:, :n // 2], approximate="tanh")

    ref_gated()
    ms = time_graph_loop(capture(ref_gated), 20, stream)
    out["fc1_bf16_gated_pytorch_cublaslt"] = {"TFLOP/s": flops / ms / 1e9, "ms": ms}
    ms = time_graph_loop(capture(lambda: F.linear(xf, wf, bf)), 20, stream)
    out["fc1_bf16_gemm_only_cublaslt"] = {"TFLOP/s": flops / ms / 1e9, "ms": ms}
    fp8_peak = None
    try:
        big = 8192
        a8 = torch.randn(big, big, device=dev).to(torch.float8_e4m3fn)
        b8 = torch.randn(big, big, device=dev).to(torch.float8_e4m3fn).t()  # column-major second operand
        one = torch.ones((), device=dev)
        mm = lambda: torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # noqa: E731
        mm()
        ms = time_graph_loop(capture(mm), 10, stream)
        fp8_peak = 2 * big ** 3 / ms / 1e9
        out["fp8_peak_measured_scaled_mm_8192"] = {"TFLOP/s": fp8_peak, "ms": ms}
        del a8, b8
    except Exception as exc:  # the comparator is informative only
        out["fp8_peak_measured_scaled_mm_8192"] = {"unavailable": str(exc).splitlines()[0][:120]}
    for name, gated in (("gated", 1), ("plain", 0)):
        y = torch.empty(m, n // 2 if gated else n, dtype=torch.bfloat16, device=dev)
        capi.fc1_fwd(xf, wf, bf, "gelu", gated, y=y, status=status)
        g = capture(lambda: capi.fc1_fwd(xf, wf, bf, "gelu", gated, y=y, status=status))
        ms = time_graph_loop(g, 50, stream)
        out[f"fc1_bf16_{name}"] = {"TFLOP/s": flops / ms / 1e9, "ms": ms, "frac_of_bf16_peak": flops / ms / 1e9 / tf_peak}
        capi.fc1_fwd(qx, qw, bf, "gelu", gated, alpha_dev=scales, out_dtype=torch.bfloat16, y=y, status=status)
        g = capture(lambda: capi.fc1_fwd(qx, qw, bf, "gelu", gated, alpha_dev=scales, out_dtype=torch.bfloat16,
                                         y=y, status=status))
        ms = time_graph_loop(g, 50, stream)
        out[f"fc1_fp8_{name}"] = {"TFLOP/s": flops / ms / 1e9, "ms": ms,
                                  "frac_of_2x_bf16_peak": flops / ms / 1e9 / (2 * tf_peak),
                                  "frac_of_measured_fp8_peak": flops / ms / 1e9 / fp8_peak if fp8_peak else None,
                                  "frac_of_nominal_4500": flops / ms / 1e9 / 4500.0}
    g = capture(lambda: capi.quantize_e4m3(xf))
    out["fp8_quantise_x_ms"] = time_graph_loop(g, 20, stream)
    del xf, wf, bf, qx, qw, y

    # FC1 backward at the DiT-XL/2 MLP shape (M = 8192 tokens, H = 1152, 2I = 9216): the activation backward with
    # recomputation (one tcgen05 launch), dx = dz W and dW = dz^T x on the tcgen05 GEMM that reads its operands in
    # place, dbias; each next to the library call the reference's backward makes for it
    mt, hh, n2 = 8192, 1152, 9216
    xb_, wb_, bb_ = (t.to(dev) for t in synth.fc1_inputs(mt, hh, n2, torch.bfloat16, seed=1))
    dyb = torch.randn(mt, n2 // 2, device=dev).to(torch.bfloat16)
    dzb = capi.fc1_bwd_dz(xb_, wb_, bb_, dyb, "gelu", status=status)
    gf = 2.0 * mt * hh * n2
    ms = time_graph_loop(capture(lambda: capi.fc1_bwd_dz(xb_, wb_, bb_, dyb, "gelu", status=status)), 20, stream)
    out["fc1_bwd_dz_recompute"] = {"TFLOP/s": gf / ms / 1e9, "ms": ms}
    capi.fc1_bwd_dz_dbias(xb_, wb_, bb_, dyb, "gelu", status=status)
    ms = time_graph_loop(capture(lambda: capi.fc1_bwd_dz_dbias(xb_, wb_, bb_, dyb, "gelu", status=status)), 20, stream)
    out["fc1_bwd_dz_recompute_with_dbias"] = {"TFLOP/s": gf / ms / 1e9, "ms": ms}
    for name, fn, lib in (("dx", lambda: capi.fc1_bwd_gemm(dzb, wb_, "dx", status=status), lambda: dzb @ wb_),
                          ("dw", lambda: capi.fc1_bwd_gemm(dzb, xb_, "dw", status=status), lambda: dzb.t() @ xb_)):
        fn()
        lib()
        ms = time_graph_loop(capture(fn), 20, stream)
        ms_lib = time_graph_loop(capture(lib), 20, stream)
        # the same GEMM on whole 128 x 192 single-CTA tiles (what a call without a workspace runs)
        whole = (lambda nm: lambda: capi.fc1_bwd_gemm(dzb, wb_ if nm == "dx" else xb_, nm, status=status,
                                                      workspace=False))(name)
        whole()
        ms_whole = time_graph_loop(capture(whole), 20, stream)
        out[f"fc1_bwd_{name}"] = {"TFLOP/s": gf / ms / 1e9, "ms": ms, "frac_of_bf16_peak": gf / ms / 1e9 / tf_peak,
                                  "whole_single_cta_tiles_ms": ms_whole,
                                  "library_gemm_ms": ms_lib, "speedup_vs_library": ms_lib / ms}
    capi.colsum(dzb)
    ms = time_graph_loop(capture(lambda: capi.colsum(dzb)), 20, stream)
    ms_lib = time_graph_loop(capture(lambda: dzb.sum(dim=0)), 20, stream)
    out["fc1_bwd_dbias"] = {"ms": ms, "GB/s": mt * n2 * 2 / ms / 1e6, "library_sum_ms": ms_lib}
    del xb_, wb_, bb_, dyb, dzb

    # FC1, the large case of workload config 4: M=32768, K=3072, N=12288 (2.47 TFLOP per launch, ~2 ms: a kernel
    # this long runs under the power cap, so its fraction is taken of the SUSTAINED bf16 figure)
    m, k, n = 32768, 3072, 12288
    flops = 2.0 * m * k * n
    xl = torch.randn(m, k, device=dev).to(torch.bfloat16)
    wl = (torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16)
    bl = (torch.randn(n, device=dev) * 0.02).to(torch.bfloat16)
    qxl, sxl = capi.quantize_e4m3(xl)
    qwl, swl = capi.quantize_e4m3(wl)
    scales_l = torch.cat([sxl, swl])
    for name, gated in (("gated", 1), ("plain", 0)):
        yl = torch.empty(m, n // 2 if gated else n, dtype=torch.bfloat16, device=dev)
        capi.fc1_fwd(xl, wl, bl, "gelu", gated, y=yl, status=status)
        ms = time_graph_loop(capture(lambda: capi.fc1_fwd(xl, wl, bl, "gelu", gated, y=yl, status=status)), 10, stream)
        out[f"fc1_large_bf16_{name}"] = {"TFLOP/s": flops / ms / 1e9, "ms": ms,
                                         "frac_of_bf16_sustained": flops / ms / 1e9 / tf_sustained,
                                         "frac_of_bf16_peak": flops / ms / 1e9 / tf_peak}
        capi.fc1_fwd(qxl, qwl, bl, "gelu", gated, alpha_dev=scales_l, out_dtype=torch.bfloat16, y=yl, status=status)
        ms = time_graph_loop(capture(lambda: capi.fc1_fwd(qxl, qwl, bl, "gelu", gated, alpha_dev=scales_l,
                                                          out_dtype=torch.bfloat16, y=yl, status=status)), 10, stream)
        out[f"fc1_large_fp8_{name}"] = {"TFLOP/s": flops / ms / 1e9, "ms": ms,
                                        "frac_of_measured_fp8_peak": flops / ms / 1e9 / fp8_peak if fp8_peak else None,
                                        "frac_of_2x_bf16_sustained": flops / ms / 1e9 / (2 * tf_sustained)}
        del yl
    ms = time_graph_loop(capture(lambda: F.linear(xl, wl, bl)), 10, stream)
    out["fc1_large_bf16_gemm_only_cublaslt"] = {"TFLOP/s": flops / ms / 1e9, "ms": ms}
    out["fc1_status_word"] = int(status.item())
    return out


def bench_sharded(dev, stream, rank: int, world: int, hbm_peak: float, tf_peak: float) -> dict | None:
    """The multi-GPU cases of the path, run by EVERY rank and reduced to rank 0 (max of the per-rank device times):
    (i) strong scaling of the fixed config-2 tensor (8192 rows / N per rank, whole samples, no collective),
    (ii) a tensor whose samples span ranks (B = 2, S = 4096; B = 1, S = 8192 on two ranks), where the packed
    fp32 dscale/dshift go through ONE NCCL all-reduce - checked against the unsharded result and for bitwise
    reproducibility, (iii) FC1 of config 4 with the weights replicated, rows per rank (weak) and rows sharded
    (strong). With one rank (i) and (iii) are the one-GPU numbers and (ii) runs without a collective."""
    import torch.distributed as dist

    from novadit_b200 import capi, shard as sh, synth

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(flag: bool) -> bool:
        if world == 1:
            return flag
        t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    out = {}
    # (i) strong scaling: this rank's block of the ONE config-2 tensor; enough rotating sets that inputs stay cold
    x, scale, shift, dy = synth.norm_inputs(B, S, H, torch.bfloat16, seed=0)
    s = sh.make_shard(ROWS, S, world, rank)
    xs, gs = x.reshape(-1, H)[s.start:s.end], dy.reshape(-1, H)[s.start:s.end]
    sd, hd = scale.to(dev), shift.to(dev)
    nsets = NSETS * world
    sets = []
    for i in range(nsets):
        xi = torch.roll(xs, i, 0).to(dev).contiguous()
        sets.append({"x": xi, "dy": torch.roll(gs, i, 0).to(dev).contiguous(), "y": torch.empty_like(xi),
                     "dx": torch.empty_like(xi), "mean": torch.empty(s.count, dtype=torch.float32, device=dev),
                     "invstd": torch.empty(s.count, dtype=torch.float32, device=dev),
                     "dscale": torch.zeros(B, H, dtype=torch.float32, device=dev),
                     "dshift": torch.zeros(B, H, dtype=torch.float32, device=dev)})

    def shard_step(st):
        capi.norm_fwd("layer", st["x"], sd, hd, EPS, y=st["y"], mean=st["mean"], invstd=st["invstd"],
                      row_start=s.start, seq_len=S)
        capi.norm_bwd("layer", st["dy"], st["x"], sd, st["mean"], st["invstd"], dx=st["dx"], dscale=st["dscale"],
                      dshift=st["dshift"], row_start=s.start, seq_len=S, batch=B)

    shard_step(sets[0])
    torch.cuda.synchronize()
    g = capture(lambda: [shard_step(st) for st in sets])
    if world > 1:
        dist.barrier()
    ms = max_over_ranks(statistics.median(time_graph_loop(g, 10, stream) for _ in range(5)) / nsets)
    out["adaln_config2_strong"] = {"rows_per_gpu": s.count, "ms_per_step": ms, "GB/s": STEP_BYTES / ms / 1e6,
                                   "frac_of_n_x_hbm_peak": STEP_BYTES / ms / 1e6 / (world * hbm_peak),
                                   "collective": "none (whole samples per GPU)"}
    del sets, g

    # (ii) samples that span ranks: the all-reduce carries data
    b2, s2 = (2, 4096) if world != 2 else (1, 8192)
    x, scale, shift, dy = synth.norm_inputs(b2, s2, H, torch.bfloat16, seed=5)
    rows2 = b2 * s2
    s = sh.make_shard(rows2, s2, world, rank)
    xs = x.reshape(-1, H)[s.start:s.end].to(dev).contiguous()
    gs = dy.reshape(-1, H)[s.start:s.end].to(dev).contiguous()
    sd, hd = scale.to(dev), shift.to(dev)
    _, mean, invstd = capi.norm_fwd("layer", xs, sd, hd, EPS, row_start=s.start, seq_len=s2)
    runs = []
    for _ in range(2):
        dx, ds, dh = sh.norm_backward_sharded("layer", gs, xs, sd, mean, invstd, s, b2)
        torch.cuda.synchronize()
        runs.append((dx.clone(), ds.clone(), dh.clone()))
    reproducible = all_true(all(torch.equal(p, q) for p, q in zip(*runs)))
    # the unsharded result of one GPU (every rank computes it: the tensor is 19 MB)
    xf, gf = x.reshape(-1, H).to(dev), dy.reshape(-1, H).to(dev)
    _, mf, rf = capi.norm_fwd("layer", xf, sd, hd, EPS, seq_len=s2)
    wdx, wds, wdh = capi.norm_bwd("layer", gf, xf, sd, mf, rf, seq_len=s2, batch=b2)

    def rel_l2(a, b):
        return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))

    mine = list(s.samples())
    errs = [rel_l2(runs[0][1][mine], wds[mine]), rel_l2(runs[0][2][mine], wdh[mine])]
    err = max_over_ranks(max(errs))
    dx_equal = all_true(torch.equal(runs[0][0], wdx[s.start:s.end]))
    if err > 1e-4 or not reproducible:
        raise AssertionError(f"sharded backward: rel-L2 {err:.3e} (bar 1e-4), reproducible {reproducible}")
    reps = 20

    def sharded_steps():
        for _ in range(reps):
            capi.norm_fwd("layer", xs, sd, hd, EPS, mean=mean, invstd=invstd, row_start=s.start, seq_len=s2)
            sh.norm_backward_sharded("layer", gs, xs, sd, mean, invstd, s, b2)

    sharded_steps()
    if world > 1:
        dist.barrier()
    ms = max_over_ranks(statistics.median(event_time_ms(sharded_steps, stream) for _ in range(5)) / reps)
    packed = torch.zeros(2, b2, H, dtype=torch.float32, device=dev)
    ar_ms = 0.0
    if world > 1:
        def reduces():
            for _ in range(reps):
                dist.all_reduce(packed)
        reduces()
        dist.barrier()
        ar_ms = max_over_ranks(statistics.median(event_time_ms(reduces, stream) for _ in range(5)) / reps)
    step_bytes2 = 5 * rows2 * H * E
    out["adaln_straddling"] = {"shape": [b2, s2, H], "rows_per_gpu": s.count,
                               "collective": "NCCL all_reduce of [2,B,H] fp32" if sh.needs_allreduce(rows2, s2, world) else "none",
                               "ms_per_step": ms, "GB/s": step_bytes2 / ms / 1e6, "allreduce_alone_ms": ar_ms,
                               "allreduce_bytes": packed.numel() * 4, "dparam_rel_l2_vs_unsharded": err,
                               "dx_bitwise_equal_unsharded": dx_equal, "bitwise_reproducible": reproducible,
                               "launch": "eager (20 steps per sample, median of 5)"}
    del xf, gf, wdx, runs

    # (iii) FC1 of config 4, weights replicated
    m, k, n = 8192, 1152, 4608
    xc, wc, bc = (t.to(dev) for t in synth.fc1_inputs(m, k, n, torch.bfloat16, seed=0))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for name, rows_here in (("weak", m), ("strong", m // world)):
        xr = xc[:rows_here].contiguous()
        yr = torch.empty(rows_here, n // 2, dtype=torch.bfloat16, device=dev)
        capi.fc1_fwd(xr, wc, bc, "gelu", 1, y=yr, status=status)
        g = capture(lambda: capi.fc1_fwd(xr, wc, bc, "gelu", 1, y=yr, status=status))
        if world > 1:
            dist.barrier()
        ms = max_over_ranks(statistics.median(time_graph_loop(g, 50, stream) for _ in range(3)))
        total = 2.0 * rows_here * k * n * world
        out[f"fc1_bf16_gated_{name}"] = {"rows_per_gpu": rows_here, "ms": ms, "TFLOP/s_all_gpus": total / ms / 1e9,
                                         "frac_of_n_x_bf16_peak": total / ms / 1e9 / (world * tf_peak)}
        del g
    out["fc1_status_word"] = int(status.item())
    del xc, wc, bc
    out["dit_stack_config5"] = bench_dit_stack(dev, rank, world, max_over_ranks)
    return out if rank == 0 else None


def bench_dit_stack(dev, rank: int, world: int, max_over_ranks) -> dict:
    """Workload config 5: one training step (forward + backward with respect to x, c and every parameter) of the
    DiT-XL/2 block stack - depth 28, hidden 1152, 16 heads, MLP ratio 4, adaLN-Zero modulation, x [32,256,1152] bf16
    per GPU, random-init weights N(0, 0.02) - built from the REFERENCE's own NovaDiTBlock modules running on this
    library's extension (novadit_b200/modules.py). The batch is sharded: every rank steps its own 32 samples, no
    gradient all-reduce (that is ordinary data parallelism, outside the operator path). Rank 0 also steps the same
    stack on the reference's PyTorch operator definitions for the parity figures and the speed-up."""
    try:
        from novadit_b200.modules import DiTStack, init_stack_, reference_modules

        reference_modules()
    except Exception as exc:
        return {"unavailable": str(exc).splitlines()[0][:160]}
    dt = torch.bfloat16
    gen = torch.Generator().manual_seed(1000 + rank)
    x = torch.randn(B, S, H, generator=gen).to(dev, dt).requires_grad_(True)
    cond = torch.randn(B, H, generator=gen).to(dev, dt).requires_grad_(True)
    dy = torch.randn(B, S, H, generator=gen).to(dev, dt)

    def build(fused: bool):
        stack = DiTStack(H, 16, 28, use_fused=fused, zero_init=False, device=dev, dtype=dt)
        init_stack_(stack, seed=0, zero_init=False)
        targets = (x, cond, *stack.parameters())

        def step():
            y = stack(x, cond)
            return y, torch.autograd.grad(y, targets, dy)

        return step

    def median_ms(step, warm: int, iters: int) -> float:
        for _ in range(warm):
            step()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    fused_step = build(True)
    ms = max_over_ranks(median_ms(fused_step, 2, 5))
    res = {"ms_per_step": ms, "tokens_per_s_all_gpus": world * B * S / ms * 1e3, "tokens_per_gpu": B * S,
           "blocks": "reference novadit.modules.NovaDiTBlock x 28 on novadit_cuda of this library"}
    if rank == 0:
        yf, gf = fused_step()
        ref_step = build(False)
        ref_ms = median_ms(ref_step, 1, 3)
        yr, gr = ref_step()

        def rel(a, b):
            a, b = a.detach().float(), b.detach().float()
            return float((a - b).norm() / b.norm().clamp_min(1e-30))

        res.update({"pytorch_operators_ms_per_step_rank0": ref_ms, "speedup_vs_pytorch_operators": ref_ms / ms,
                    "parity_rel_l2": {"y": rel(yf, yr), "dx": rel(gf[0], gr[0]), "dcond": rel(gf[1], gr[1]),
                                      "param_grads": rel(torch.cat([g.flatten() for g in gf[2:]]),
                                                         torch.cat([g.flatten() for g in gr[2:]]))}})
    return res


def bench_e2e(dev, k: int) -> dict:
    """The same step through the public API (`novadit_b200.ops.fused_adaln` + autograd) from pinned HOST
    buffers, the way a caller without device-resident activations uses the library: `HostPipeline` uploads
    x, scale, shift, dy, runs the step and downloads y, dx, dscale, dshift, with the three phases of consecutive
    steps on three streams. Every step's host->device and device->host copies are inside the timed region, which
    ends when the last step's results are in host memory."""
    from novadit_b200 import synth
    from novadit_b200.hostpipe import HostPipeline, adaln_train_step, bind_host_thread_to_gpu

    cpus_before = os.sched_getaffinity(0)
    bound = bind_host_thread_to_gpu(dev.index or 0)  # pinned buffers below land on the GPU's NUMA node
    host = [t.pin_memory() for t in synth.norm_inputs(B, S, H, torch.bfloat16, seed=0)]
    pipe = HostPipeline(adaln_train_step(EPS), dev, depth=3)
    for _ in range(12):  # untimed: pinned result buffers, allocator pools and copy paths reach their steady state
        last = pipe.submit(host)
    outs = pipe.result(last)
    pipe.drain()
    t0 = time.perf_counter()
    for _ in range(k):
        pipe.submit(host)
    pipe.drain()
    sec = (time.perf_counter() - t0) / k
    os.sched_setaffinity(0, cpus_before)  # the CPU baseline leg gets every core back
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = sum(t.numel() * t.element_size() for t in outs)
    return {"seconds_per_step": sec, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "pipeline": "3 streams, 3 steps in flight", "host_thread_bound_to_gpu_numa_node": bound}


def run_gpu_arm(args) -> None:
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the operators have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    hbm_peak, tf_peak, peak_src = measured_peaks()
    tf_sustained = measured_sustained_tflops(tf_peak)
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    stream = torch.cuda.current_stream()

    work = NormWorkload("layer", dev)
    big, singles, fwd_only, bwd_only = work.graphs()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Load phase: the warm-up steps, extended to ~0.4 s of continuous launches so that the clock samples
    # taken from here to the end of the timed region are samples under load.
    sampler = ClockSampler(local)
    replay_steps(big, singles, warmup)
    torch.cuda.synchronize()
    sampler.start()
    t_load = time.perf_counter()
    while time.perf_counter() - t_load < 0.4:
        for _ in range(50):
            big.replay()
        torch.cuda.synchronize()

    # Timed region: exactly `steps` steps between two events, barrier + synchronize on both sides. One untimed
    # rotation is queued right before the first event so that the first timed step does not start on an idle GPU,
    # and the region is repeated: the per-rank median is reported (then the maximum over ranks).
    est_s = steps * 30e-6
    repeats = 25 if est_s * 25 <= 5.0 else max(3, int(5.0 / est_s))
    timed = StepGraphs(work, steps)
    timed.replay()  # first launch of the new graphs, untimed
    samples_ms = []
    for _ in range(repeats):
        barrier()
        big.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        timed.replay()
        e1.record(stream)
        barrier()
        samples_ms.append(e0.elapsed_time(e1))
    elapsed_ms = statistics.median(samples_ms)

    # Per-kernel durations for the roofline (same buffers, same rotation), still under the sampler.
    reps = max(4, min(200, steps // NSETS + 1))
    fwd_ms = time_graph_loop(fwd_only, reps, stream) / NSETS
    bwd_ms = time_graph_loop(bwd_only, reps, stream) / NSETS
    clocks = sampler.stop()

    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / steps
    value = world * STEP_BYTES / (ms_per_step * 1e-3) / 1e9

    e2e = bench_e2e(dev, max(3, min(steps, 30)))
    e2e_sec = e2e.pop("seconds_per_step")
    if world > 1:
        t = torch.tensor([e2e_sec], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_sec = float(t.item())
    e2e_line = {"value": world * STEP_BYTES / e2e_sec / 1e9, "unit": UNIT, **e2e}

    extras, cpu_line = None, None
    multi = None
    if not args.no_extras:
        multi = bench_sharded(dev, stream, rank, world, hbm_peak, tf_peak)  # every rank takes part
    if rank == 0 and not args.no_extras:
        extras = bench_extras(dev, stream, hbm_peak, tf_peak, tf_sustained)
        extras["adaln_fwd_kernel"] = {"ms": fwd_ms, "GB/s": FWD_BYTES / fwd_ms / 1e6,
                                      "frac_of_hbm_peak": FWD_BYTES / fwd_ms / 1e6 / hbm_peak}
        extras["sharded"] = multi
    if rank == 0 and world == 1 and not args.no_cpu:
        sec, ran, threads = cpu_reference_step_time(200, 1, budget_s=10.0)
        cpu_line = {"value": STEP_BYTES / sec / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
                    "sample": f"{ran} full config-2 steps (about 10 s) of the reference's PyTorch CPU path, median"}
    barrier()

    if rank == 0:
        achieved = BWD_BYTES / bwd_ms / 1e6
        traffic, traffic_rec = measured_traffic()
        fc1 = (extras or {}).get("fc1_bf16_gated")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD},
            "setup": {"per_gpu": "one config-2 batch per GPU", "global_rows": world * ROWS,
                      "parallelism": f"rows sharded over {world} GPU(s), no collective",
                      "cold_cache": f"{NSETS} rotating buffer sets (605 MB > 4x L2)", "launch": "CUDA graphs",
                      "repeats": repeats, "timed": "median over repeats of the exact `steps`-step region, max over ranks",
                      "ms_per_step_min_max": [min(samples_ms) / steps, max(samples_ms) / steps]},
            "repeats": repeats,
            "frac_of_hbm_peak": value / world / hbm_peak,
            "roofline": {"kernel": "norm_bwd_tma + norm_dparam_stage2 (dx + dscale/dshift, one pass over dy and x)", "bound": "hbm",
                         "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "traffic": traffic, "traffic_record": traffic_rec, "peak_source": peak_src,
                         "algorithmic_bytes": BWD_BYTES, "avg_launch_ms": bwd_ms,
                         "timing": {"method": "a loop of backward + stage-2 launches over the rotation, right after "
                                              "the timed region", "step_ms": ms_per_step,
                                    "forward_only_loop_ms": fwd_ms, "backward_only_loop_ms": bwd_ms}},
            "roofline_fc1": None if not fc1 else {
                "kernel": "fc1_pair_kernel (tcgen05, gated GELU-tanh epilogue), config 4 bf16", "bound": "tensor",
                "achieved": fc1["TFLOP/s"], "peak": tf_peak, "unit": "TFLOP/s", "frac": fc1["TFLOP/s"] / tf_peak,
                "flops": 2.0 * 8192 * 1152 * 4608, "avg_launch_ms": fc1["ms"], "peak_source": peak_src + " (burst)"},
            "e2e": e2e_line, "gpu_launches": 3 * steps, "clocks": clocks,
            "cpu_baseline": cpu_line, "extras": extras,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_profile_case(op: str, variant: int = -1) -> None:
    """A handful of direct launches (no graphs, no rotation) of one operator at its benchmark size: the
    command ncu captures. `op`: norm (config 2 AdaLN fwd + bwd), rms, gate (2048 rows of config 3), fc1, fc1_bwd,
    residual."""
    from novadit_b200 import capi, synth

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if variant >= 0:
        capi.lib().nd_tune_norm_variant(variant)
    if op in ("norm", "rms"):
        work = NormWorkload("layer" if op == "norm" else "rms", dev)
        for i in range(6):
            work.step(work.sets[i % NSETS])
    elif op == "gate":
        x, dy = synth.gate_act_inputs(1, 4096, 4608, torch.bfloat16, seed=3)  # 151 MB in + out
        xg, dyg = x.to(dev), dy.to(dev)
        for _ in range(3):
            for act in ("silu", "gelu"):
                capi.gate_act_fwd(xg, act)
                capi.gate_act_bwd(dyg, xg, act)
    elif op == "fc1":
        xf, wf, bf = (t.to(dev) for t in synth.fc1_inputs(8192, 1152, 4608, torch.bfloat16, seed=0))
        qx, sx = capi.quantize_e4m3(xf)
        qw, sw = capi.quantize_e4m3(wf)
        for _ in range(3):
            capi.fc1_fwd(xf, wf, bf, "gelu", 1)
            capi.fc1_fwd(qx, qw, bf, "gelu", 1, alpha_dev=torch.cat([sx, sw]), out_dtype=torch.bfloat16)
    elif op == "fc1_bwd":
        # the FC1 backward at the DiT-XL/2 MLP shape: dz with recomputation, dx and dW (CTA-pair tiles), dbias
        mt, hh, n2 = 8192, 1152, 9216
        xb, wb, bb = (t.to(dev) for t in synth.fc1_inputs(mt, hh, n2, torch.bfloat16, seed=1))
        dyb = torch.randn(mt, n2 // 2, device=dev).to(torch.bfloat16)
        for _ in range(2):
            dzb = capi.fc1_bwd_dz(xb, wb, bb, dyb, "gelu")
            capi.fc1_bwd_gemm(dzb, wb, "dx")
            capi.fc1_bwd_gemm(dzb, xb, "dw")
            capi.colsum(dzb)
    elif op == "residual":
        # config 2 with the gated residual in front of the norm, and its backward partner
        work = NormWorkload("layer", dev)
        st = work.sets[0]
        x, dy = st["x"], st["dy"]
        gate = torch.randn(x.shape[0], x.shape[-1], device=dev).to(x.dtype)
        for _ in range(3):
            capi.norm_fwd_residual("layer", x, dy, gate, st["scale"], st["shift"], EPS)
            capi.gated_residual_bwd_add(dy, x, dy, gate)
    else:
        raise SystemExit(f"unknown profile case {op}")
    torch.cuda.synchronize()
    print("profile case done:", op)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="novadit_b200", choices=["novadit_b200", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the other operators (AdaRMSNorm, gate-act, FC1)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--profile-variant", type=int, default=-1, help="norm kernel variant for --profile")
    ap.add_argument("--profile", default=None, help="run a few direct launches of one operator (for ncu) and exit")
    args = ap.parse_args()
    if args.profile:
        run_profile_case(args.profile, args.profile_variant)
        return
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
