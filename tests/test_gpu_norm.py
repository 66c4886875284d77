"""AdaLN / AdaRMSNorm CUDA kernels against the CPU oracle and the reference's golden vectors.

Every call goes through the C ABI (`novadit_b200.capi`). Bars: bf16/fp16 outputs max_abs <= 2e-2
and relative L2 <= 1e-2; fp32 dscale/dshift relative L2 <= 1e-4 (see tests/helpers.py).
"""
from __future__ import annotations

import pytest
import torch

from novadit_b200 import capi, synth
from oracle import novadit_oracle as oracle
from tests import golden_io
from tests.helpers import assert_f32_parity, assert_half_parity, assert_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"
NORM = golden_io.load("norm_golden")


def run_fwd_bwd(kind, x, scale, shift, dy, eps, mode="fused", **kw):
    """Forward then backward through the C ABI; returns (y, stats..., dx, dscale, dshift) on the device."""
    xd, sd, hd, gd = (t.to(DEV).contiguous() for t in (x, scale, shift, dy))
    sd2, hd2 = sd.reshape(sd.shape[0], -1), hd.reshape(hd.shape[0], -1)
    if kind == "layer":
        y, mean, invstd = capi.norm_fwd(kind, xd, sd2, hd2, eps)
    else:
        y, invstd = capi.norm_fwd(kind, xd, sd2, hd2, eps)
        mean = None
    dx, dscale, dshift = capi.norm_bwd(kind, gd, xd, sd2, mean, invstd, mode=mode, **kw)
    torch.cuda.synchronize()
    return y, mean, invstd, dx, dscale, dshift


def oracle_fwd_bwd(kind, x, scale, shift, dy, eps, compute=torch.float64):
    """(y, mean, invstd, dx, dscale, dshift, y_exact, dx_exact): fp64 oracle, rounded once, plus the
    unrounded fp64 values used to recognise rounding near-ties."""
    if kind == "layer":
        ye, mean, invstd = oracle.adaln_fwd(x, scale, shift, eps, compute=compute, round_out=False)
        dxe, ds, dh = oracle.adaln_bwd(dy, x, scale, eps, compute=compute, round_out=False)
    else:
        ye, invstd = oracle.adarms_fwd(x, scale, shift, eps, compute=compute, round_out=False)
        mean = None
        dxe, ds, dh = oracle.adarms_bwd(dy, x, scale, eps, compute=compute, round_out=False)
    return ye.to(x.dtype), mean, invstd, dxe.to(x.dtype), ds, dh, ye, dxe


def compare_all(kind, got, want, what):
    y, mean, invstd, dx, ds, dh = got
    wy, wmean, winvstd, wdx, wds, wdh, ye, dxe = want
    if wy.dtype == torch.float32:
        assert_parity(y, wy, what + " y")
        assert_parity(dx, wdx, what + " dx")
    else:
        assert_half_parity(y, wy, what + " y", exact=ye)
        assert_half_parity(dx, wdx, what + " dx", exact=dxe)
    if kind == "layer":
        assert_f32_parity(mean.reshape(wmean.shape), wmean, what + " mean", tol=1e-4 + 0.0)
    assert_f32_parity(invstd.reshape(winvstd.shape), winvstd, what + " invstd", tol=1e-5)
    assert_f32_parity(ds, wds, what + " dscale")
    assert_f32_parity(dh, wdh, what + " dshift")


@pytest.mark.parametrize("case", sorted(NORM))
def test_matches_reference_golden_vectors(case):
    """The committed outputs of the reference's own functions, on the same seeded inputs."""
    g = NORM[case]
    dtype = golden_io.DTYPES[g["dtype"]]
    b, s, h = (int(v) for v in g["shape"])
    x, scale, shift, dy = synth.norm_inputs(b, s, h, dtype, int(g["seed"]))
    y, mean, invstd, dx, ds, dh = run_fwd_bwd(g["kind"], x, scale, shift, dy, float(g["eps"]))
    want_y, want_dx = golden_io.unpack(g["y"], dtype), golden_io.unpack(g["dx"], dtype)
    y, dx = y.cpu().reshape(-1, h), dx.cpu().reshape(-1, h)
    if "rows" in g:
        rows = torch.from_numpy(g["rows"])
        y, dx = y[rows], dx[rows]
    assert_parity(y, want_y.reshape(y.shape), case + " y")
    assert_parity(dx, want_dx.reshape(dx.shape), case + " dx")
    assert_f32_parity(ds, torch.from_numpy(g["dscale"]).reshape(b, h), case + " dscale")
    assert_f32_parity(dh, torch.from_numpy(g["dshift"]).reshape(b, h), case + " dshift")


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("dtype,shape", [
    (torch.float16, (2, 3, 768)), (torch.bfloat16, (2, 3, 768)),      # the reference's aligned cases
    (torch.float16, (2, 3, 770)), (torch.bfloat16, (2, 3, 770)),      # rows not 16-byte aligned: scalar path
    (torch.bfloat16, (2, 257, 768)), (torch.float16, (2, 257, 770)),  # S = 257: ragged row tiles (dparam case)
    (torch.float32, (2, 256, 768)),                                   # workload config 1 (fp32)
    (torch.bfloat16, (3, 5, 8)), (torch.bfloat16, (1, 1, 1152)),      # tiny H; a single row
    (torch.bfloat16, (2, 9, 4096)), (torch.bfloat16, (2, 5, 8192)),   # 512 / 1024 threads per row
    (torch.bfloat16, (1, 3, 16384)), (torch.float32, (2, 3, 2500)),   # several vectors per thread; fp32 scalar path
])
def test_matches_oracle_small_shapes(kind, dtype, shape):
    b, s, h = shape
    x, scale, shift, dy = synth.norm_inputs(b, s, h, dtype, seed=100 + h % 97)
    eps = 1e-6 if dtype == torch.float32 else 1e-5
    got = run_fwd_bwd(kind, x, scale, shift, dy, eps)
    compare_all(kind, got, oracle_fwd_bwd(kind, x, scale, shift, dy, eps), f"{kind} {dtype} {shape}")


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_config2_dit_xl_shape_bf16(kind, seed):
    """Workload config 2: B=32, S=256, H=1152 bf16, eps 1e-6, over several seeds."""
    x, scale, shift, dy = synth.norm_inputs(32, 256, 1152, torch.bfloat16, seed)
    got = run_fwd_bwd(kind, x, scale, shift, dy, 1e-6)
    compare_all(kind, got, oracle_fwd_bwd(kind, x, scale, shift, dy, 1e-6), f"config2 {kind} seed {seed}")


@pytest.mark.parametrize("kind", ["layer", "rms"])
def test_separate_backward_entry_points_equal_fused(kind):
    x, scale, shift, dy = synth.norm_inputs(4, 100, 1152, torch.bfloat16, 3)
    y, mean, invstd, dx, ds, dh = run_fwd_bwd(kind, x, scale, shift, dy, 1e-5, mode="fused")
    _, _, _, dx2, _, _ = run_fwd_bwd(kind, x, scale, shift, dy, 1e-5, mode="dx")
    _, _, _, _, ds2, dh2 = run_fwd_bwd(kind, x, scale, shift, dy, 1e-5, mode="dparam")
    assert torch.equal(dx, dx2) and torch.equal(ds, ds2) and torch.equal(dh, dh2)


@pytest.mark.parametrize("kind", ["layer", "rms"])
def test_inference_equals_training_output_bitwise(kind):
    x, scale, shift, _ = synth.norm_inputs(2, 33, 1152, torch.bfloat16, 4)
    xd, sd, hd = x.to(DEV), scale.to(DEV), shift.to(DEV)
    y_train = capi.norm_fwd(kind, xd, sd, hd, 1e-5)[0]
    y_inf = capi.norm_fwd(kind, xd, sd, hd, 1e-5, stats=False)[0]
    assert torch.equal(y_train, y_inf)


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("variant", [0, 1, 3, 4, 5, 6])
def test_every_kernel_variant_meets_the_bars(kind, variant):
    """The tuning knob selects among instantiations of the hot kernels; each must be correct."""
    x, scale, shift, dy = synth.norm_inputs(5, 77, 1152, torch.bfloat16, 8)
    want = oracle_fwd_bwd(kind, x, scale, shift, dy, 1e-6)
    L = capi.lib()
    try:
        L.nd_tune_norm_variant(variant)
        for mode in ("fused", "dx", "dparam"):
            got = run_fwd_bwd(kind, x, scale, shift, dy, 1e-6, mode=mode)
            if mode == "fused":
                compare_all(kind, got, want, f"variant {variant}")
            elif mode == "dx":
                assert_half_parity(got[3], want[3], f"variant {variant} dx only", exact=want[7])
            else:
                assert_f32_parity(got[4], want[4], f"variant {variant} dscale only")
                assert_f32_parity(got[5], want[5], f"variant {variant} dshift only")
        assert L.nd_device_error(0) == 0, "a bounded device-side wait expired"
    finally:
        L.nd_tune_norm_variant(0)


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("dtype,shape", [
    (torch.bfloat16, (3, 77, 1152)),    # 4.5 passes per lane, ragged groups at every sample end
    (torch.float16, (2, 130, 768)),     # 3 full passes
    (torch.bfloat16, (5, 9, 128)),      # half a pass, samples shorter than three groups
    (torch.bfloat16, (2, 40, 1536)),    # 6 passes, the widest row of this kernel
    (torch.bfloat16, (1, 1, 64)),       # a single row
    (torch.float32, (2, 33, 768)),      # fp32 rows: 4 elements per vector, 6 passes
])
def test_warp_per_row_forward_kernel(kind, dtype, shape):
    """The forward kernel the launcher picks for large tensors, forced on small ones: full result, statistics
    off (inference), and a shard that starts and ends inside samples."""
    b, s_len, h = shape
    x, scale, shift, dy = synth.norm_inputs(b, s_len, h, dtype, 17)
    want = oracle_fwd_bwd(kind, x, scale, shift, dy, 1e-6)
    xd, sd, hd = x.to(DEV), scale.to(DEV), shift.to(DEV)
    L = capi.lib()
    try:
        L.nd_tune_norm_variant(4)
        out = capi.norm_fwd(kind, xd, sd, hd, 1e-6)
        y_inf = capi.norm_fwd(kind, xd, sd, hd, 1e-6, stats=False)[0]
        rows = b * s_len
        lo, hi = rows // 3, rows - rows // 4
        part = capi.norm_fwd(kind, xd.reshape(-1, h)[lo:hi].contiguous(), sd, hd, 1e-6, row_start=lo, seq_len=s_len)
        torch.cuda.synchronize()
    finally:
        L.nd_tune_norm_variant(0)
    y, stats = out[0], out[1:]
    if dtype == torch.float32:
        assert_parity(y, want[0], "y")
    else:
        assert_half_parity(y, want[0], "y", exact=want[6])
    if kind == "layer":
        assert_f32_parity(stats[0].reshape(want[1].shape), want[1], "mean", tol=1e-4)
    assert_f32_parity(stats[-1].reshape(want[2].shape), want[2], "invstd", tol=1e-5)
    assert torch.equal(y_inf, y)
    assert torch.equal(part[0], y.reshape(-1, h)[lo:hi])
    assert torch.equal(part[-1].reshape(-1), stats[-1].reshape(-1)[lo:hi])
    assert L.nd_device_error(0) == 0


@pytest.mark.parametrize("tile_rows", [1, 8, 24, 64, 1000])
def test_row_tile_height_does_not_change_results_beyond_rounding(tile_rows):
    x, scale, shift, dy = synth.norm_inputs(3, 130, 768, torch.bfloat16, 5)
    want = oracle_fwd_bwd("layer", x, scale, shift, dy, 1e-5)
    L = capi.lib()
    try:
        L.nd_tune_norm_tile_rows(tile_rows)
        got = run_fwd_bwd("layer", x, scale, shift, dy, 1e-5, ws=capi.Workspace())
    finally:
        L.nd_tune_norm_tile_rows(0)
    compare_all("layer", got, want, f"tile_rows {tile_rows}")


class _DirtyWorkspace(capi.Workspace):
    """Scratch that starts out full of ones in every bit: the library must not rely on its contents."""

    def get(self, nbytes, device, stream=0):
        fresh = (torch.device(device), stream) not in self.bufs
        buf = super().get(nbytes, device, stream)
        if fresh and buf is not None:
            buf.fill_(0xFF)
        return buf


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("mode", ["fused", "dparam"])
@pytest.mark.parametrize("shape,row_lo,row_hi", [
    ((32, 256, 1152), 0, None),      # the benchmark shape: one or two samples per chunk of rows
    ((6, 300, 768), 0, None),
    ((5, 640, 1152), 700, 2900),     # a shard that starts and ends inside samples
    ((2, 4096, 128), 0, None),       # long samples: many partial slots per sample
])
def test_dparam_does_not_depend_on_scratch_contents_or_replay(kind, mode, shape, row_lo, row_hi):
    """dscale/dshift are bit-identical from scratch memory that was never cleared, launch after launch on the
    same scratch, and under CUDA-graph replay."""
    b, s_len, h = shape
    x, scale, shift, dy = synth.norm_inputs(b, s_len, h, torch.bfloat16, 31)
    xd, sd, hd, gd = (t.to(DEV) for t in (x, scale, shift, dy))
    if kind == "layer":
        _, mean, invstd = capi.norm_fwd(kind, xd, sd, hd, 1e-6)
    else:
        _, invstd = capi.norm_fwd(kind, xd, sd, hd, 1e-6)
        mean = None
    row_hi = b * s_len if row_hi is None else row_hi
    rows = slice(row_lo, row_hi)
    xs, gs = xd.reshape(-1, h)[rows].contiguous(), gd.reshape(-1, h)[rows].contiguous()
    ms = None if mean is None else mean.reshape(-1)[rows].contiguous()
    vs = invstd.reshape(-1)[rows].contiguous()

    def bwd(ws, **kw):
        return capi.norm_bwd(kind, gs, xs, sd, ms, vs, mode=mode, row_start=row_lo, seq_len=s_len, batch=b, ws=ws, **kw)

    _, want_ds, want_dh = bwd(capi.Workspace())
    torch.cuda.synchronize()
    ws = _DirtyWorkspace()
    for attempt in range(3):
        _, ds, dh = bwd(ws)
        torch.cuda.synchronize()
        assert torch.equal(ds, want_ds) and torch.equal(dh, want_dh), f"launch {attempt} on the same scratch"
    ds, dh = torch.zeros_like(want_ds), torch.zeros_like(want_dh)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        bwd(ws, dscale=ds, dshift=dh)  # sizes this stream's scratch before the capture
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            bwd(ws, dscale=ds, dshift=dh)
    for replay in range(3):
        ds.fill_(7.0)
        dh.fill_(7.0)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        touched = ds.ne(7.0).any(dim=1)  # samples of the shard
        assert touched.any()
        assert torch.equal(ds[touched], want_ds[touched]) and torch.equal(dh[touched], want_dh[touched]), \
            f"graph replay {replay}"
    assert capi.lib().nd_device_error(0) == 0


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(32, 256, 1152), (3, 250, 768), (5, 77, 1536)])
def test_the_flat_walk_agrees_with_the_general_kernels_bit_for_bit(kind, dtype, shape):
    """Sample-aligned plans run the flat kernels (one sample per chunk, no row predicates in full groups); variant 6
    keeps the general bulk-copy kernels. Same arithmetic in the same order: every output of the forward, of the
    forward with the residual in front and of the three backward modes is bit-identical (ragged last groups and
    chunk sizes that differ by one row included: 250 and 77 rows per sample)."""
    x, scale, shift, dy = (t.to(DEV) for t in synth.norm_inputs(*shape, dtype, seed=5))
    gate = (torch.arange(scale.numel(), device=DEV).reshape(scale.shape) % 7 * 0.125).to(dtype)
    L = capi.lib()
    outs = {}
    try:
        for variant in (6, 0):
            L.nd_tune_norm_variant(variant)
            f = capi.norm_fwd(kind, x, scale, shift, 1e-6)
            mean, inv = (f[1], f[2]) if kind == "layer" else (None, f[1])
            got = list(f) + list(capi.norm_fwd_residual(kind, x, dy, gate, scale, shift, 1e-6))
            for mode in ("dx", "dparam", "fused"):
                got += [t for t in capi.norm_bwd(kind, dy, x, scale, mean, inv, mode=mode) if t is not None]
            outs[variant] = got
    finally:
        L.nd_tune_norm_variant(0)
    torch.cuda.synchronize()
    assert len(outs[0]) == len(outs[6])
    for a, b in zip(outs[0], outs[6]):
        assert torch.equal(a, b)
    assert L.nd_device_error(0) == 0


def test_dparam_is_deterministic_run_to_run():
    x, scale, shift, dy = synth.norm_inputs(8, 256, 1152, torch.bfloat16, 6)
    first = run_fwd_bwd("layer", x, scale, shift, dy, 1e-6)
    for _ in range(3):
        again = run_fwd_bwd("layer", x, scale, shift, dy, 1e-6)
        assert torch.equal(first[4], again[4]) and torch.equal(first[5], again[5]) and torch.equal(first[3], again[3])


@pytest.mark.parametrize("kind", ["layer", "rms"])
@pytest.mark.parametrize("n_shards", [2, 3, 8])
def test_row_shards_reproduce_the_unsharded_result(kind, n_shards):
    """Shard the B*S rows (shards cut through samples); partial dscale/dshift sum to the full result."""
    b, s, h = 3, 50, 768
    x, scale, shift, dy = synth.norm_inputs(b, s, h, torch.bfloat16, 7)
    want = oracle_fwd_bwd(kind, x, scale, shift, dy, 1e-5)
    xd, gd = x.to(DEV).reshape(-1, h), dy.to(DEV).reshape(-1, h)
    sd, hd = scale.to(DEV), shift.to(DEV)
    rows = b * s
    bounds = [rows * i // n_shards for i in range(n_shards + 1)]
    ys, dxs = [], []
    ds_sum = torch.zeros(b, h, dtype=torch.float32, device=DEV)
    dh_sum = torch.zeros_like(ds_sum)
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        xs, gs = xd[lo:hi].contiguous(), gd[lo:hi].contiguous()
        if kind == "layer":
            y, mean, invstd = capi.norm_fwd(kind, xs, sd, hd, 1e-5, row_start=lo, seq_len=s)
        else:
            y, invstd = capi.norm_fwd(kind, xs, sd, hd, 1e-5, row_start=lo, seq_len=s)
            mean = None
        dx, ds, dh = capi.norm_bwd(kind, gs, xs, sd, mean, invstd, row_start=lo, seq_len=s, batch=b)
        ys.append(y)
        dxs.append(dx)
        ds_sum += ds
        dh_sum += dh
    assert_half_parity(torch.cat(ys).reshape(b, s, h), want[0], "sharded y")
    assert_half_parity(torch.cat(dxs).reshape(b, s, h), want[3], "sharded dx")
    assert_f32_parity(ds_sum, want[4], "sharded dscale")
    assert_f32_parity(dh_sum, want[5], "sharded dshift")


def test_empty_shard_and_bad_arguments():
    L = capi.lib()
    x = torch.zeros(4, 8, dtype=torch.bfloat16, device=DEV)
    s = torch.zeros(1, 8, dtype=torch.bfloat16, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    assert L.nd_adaln_fwd(capi.ND_BF16, x.data_ptr(), s.data_ptr(), s.data_ptr(), x.data_ptr(), None, None,
                          0, 0, 4, 8, 1e-5, st) == 0
    assert L.nd_adaln_fwd(capi.ND_BF16, None, s.data_ptr(), s.data_ptr(), x.data_ptr(), None, None,
                          4, 0, 4, 8, 1e-5, st) == -1
    assert L.nd_adaln_fwd(capi.ND_E4M3, x.data_ptr(), s.data_ptr(), s.data_ptr(), x.data_ptr(), None, None,
                          4, 0, 4, 8, 1e-5, st) == -2
    # a mean without an invstd is inconsistent
    m = torch.zeros(4, dtype=torch.float32, device=DEV)
    assert L.nd_adaln_fwd(capi.ND_BF16, x.data_ptr(), s.data_ptr(), s.data_ptr(), x.data_ptr(), m.data_ptr(), None,
                          4, 0, 4, 8, 1e-5, st) == -1
    # dparam without the workspace it needs
    big = torch.zeros(64, 8, dtype=torch.bfloat16, device=DEV)
    stat = torch.zeros(64, dtype=torch.float32, device=DEV)
    out = torch.zeros(1, 8, dtype=torch.float32, device=DEV)
    assert L.nd_norm_dparam_ws_bytes(64, 0, 64, 8) > 0 and L.nd_norm_dparam_ws_bytes(0, 0, 64, 8) == 0
    assert L.nd_adaln_bwd_dparam(capi.ND_BF16, big.data_ptr(), big.data_ptr(), stat.data_ptr(), stat.data_ptr(),
                                 out.data_ptr(), out.data_ptr(), 64, 0, 64, 8, None, 0, st) == -4
    torch.cuda.synchronize()


def test_constant_rows_and_large_offsets_stay_finite():
    """var = 0 rows (constant input) and a large common offset (where E[x^2]-mean^2 would cancel)."""
    b, s, h = 2, 4, 1152
    x = torch.full((b, s, h), 3.0, dtype=torch.bfloat16)
    x[1] = (torch.randn(s, h) * 0.01 + 100.0).to(torch.bfloat16)
    scale = torch.zeros(b, h, dtype=torch.bfloat16)
    shift = torch.zeros(b, h, dtype=torch.bfloat16)
    dy = torch.ones(b, s, h, dtype=torch.bfloat16)
    got = run_fwd_bwd("layer", x, scale, shift, dy, 1e-5)
    want = oracle_fwd_bwd("layer", x, scale, shift, dy, 1e-5)
    assert torch.isfinite(got[0].float()).all() and torch.isfinite(got[3].float()).all()
    assert_half_parity(got[0], want[0], "offset rows y")
    assert float(got[0][0].float().abs().max()) == 0.0  # constant row normalises to exactly 0


@pytest.mark.parametrize("kind", ["layer", "rms"])
def test_full_size_properties(kind):
    """Size-independent properties at a size the CPU oracle is not asked to handle (256k rows):
    rows are independent (a permutation of rows within a sample permutes y bit for bit) and dshift
    equals the plain column sum of dy; 64 sampled rows are also checked against the oracle."""
    b, s, h = 64, 4096, 1152
    g = torch.Generator(device=DEV).manual_seed(9)
    x = torch.randn(b, s, h, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    dy = torch.randn(b, s, h, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    scale = (torch.randn(b, h, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    shift = (torch.randn(b, h, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    out = capi.norm_fwd(kind, x, scale, shift, 1e-6)
    y, invstd = out[0], out[-1]
    mean = out[1] if kind == "layer" else None
    perm = torch.randperm(s, generator=g, device=DEV)
    y_perm = capi.norm_fwd(kind, x[:, perm].contiguous(), scale, shift, 1e-6)[0]
    assert torch.equal(y_perm, y[:, perm])
    dx, ds, dh = capi.norm_bwd(kind, dy, x, scale, mean, invstd)
    want_dh = dy.float().sum(dim=1)
    assert_f32_parity(dh, want_dh, "dshift vs column sum")
    # spot-check 64 random rows of y and dx against the oracle
    rows = torch.randint(0, b * s, (64,), generator=g, device=DEV)
    bs = rows // s
    xs = x.reshape(-1, h)[rows].cpu().unsqueeze(1)
    sc, sh = scale[bs].cpu(), shift[bs].cpu()
    dys = dy.reshape(-1, h)[rows].cpu().unsqueeze(1)
    if kind == "layer":
        wy = oracle.adaln_fwd(xs, sc, sh, 1e-6, compute=torch.float64)[0]
        wdx = oracle.adaln_bwd(dys, xs, sc, 1e-6, compute=torch.float64)[0]
    else:
        wy = oracle.adarms_fwd(xs, sc, sh, 1e-6, compute=torch.float64)[0]
        wdx = oracle.adarms_bwd(dys, xs, sc, 1e-6, compute=torch.float64)[0]
    assert_half_parity(y.reshape(-1, h)[rows].cpu().unsqueeze(1), wy, "sampled rows y")
    assert_half_parity(dx.reshape(-1, h)[rows].cpu().unsqueeze(1), wdx, "sampled rows dx")


def test_an_expired_wait_sets_the_error_word_and_the_launch_returns():
    """The abort path of the bulk-copy norm kernels, exercised without faulting or hanging anything: the wait limit
    is shortened to 2 ms and CTA 0 is told not to send its first copy (nothing is in flight for that stage), so its
    first wait runs out. The kernel must record the expiry in the device error word, leave through the abort path
    and complete; afterwards the context is usable and an ordinary launch gives the ordinary result."""
    L = capi.lib()
    x, scale, shift, dy = (t.to(DEV) for t in synth.norm_inputs(4, 64, 1152, torch.bfloat16, seed=5))
    want_y, mean, invstd = capi.norm_fwd("layer", x, scale, shift, 1e-6)
    want_dx, want_ds, want_dh = capi.norm_bwd("layer", dy, x, scale, mean, invstd)
    torch.cuda.synchronize()
    assert L.nd_device_error(1) == 0
    try:
        L.nd_tune_norm_wait_test(2_000_000, 1)
        capi.norm_fwd("layer", x, scale, shift, 1e-6)
        torch.cuda.synchronize()                      # the launch completes: no hang, no fault
        assert L.nd_device_error(1) == 1              # forward wait expired (and the word is cleared again)
        capi.norm_bwd("layer", dy, x, scale, mean, invstd)
        torch.cuda.synchronize()
        assert L.nd_device_error(1) == 2              # backward wait expired
    finally:
        L.nd_tune_norm_wait_test(0, 0)
    y, _, _ = capi.norm_fwd("layer", x, scale, shift, 1e-6)
    dx, ds, dh = capi.norm_bwd("layer", dy, x, scale, mean, invstd)
    torch.cuda.synchronize()
    assert L.nd_device_error(0) == 0
    assert torch.equal(y, want_y) and torch.equal(dx, want_dx) and torch.equal(ds, want_ds) and torch.equal(dh, want_dh)
