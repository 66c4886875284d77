"""Fused FC1 (tcgen05) against the CPU oracle and the reference's golden vectors, through the C ABI."""
from __future__ import annotations

import pytest
import torch

import novadit_b200.ops as ops
from novadit_b200 import capi, synth
from oracle import novadit_oracle as oracle
from tests import golden_io
from tests.helpers import FP8_REL_L2, assert_half_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"
FC1 = golden_io.load("fc1_golden")


def new_status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def run(x, w, b, act, layout, **kw):
    """layout: 1 = stacked [gate | value] rows, 2 = interleaved rows, 0 = no gating."""
    status = new_status()
    wd = w.to(DEV)
    bd = None if b is None else b.to(DEV)
    if layout == 2:
        wd = ops.interleave_weight(wd)
        bd = None if bd is None else ops.interleave_bias(bd)
    y = capi.fc1_fwd(x.to(DEV), wd, bd, act, layout, status=status, **kw)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"device-side wait expired, code {int(status.item())}"
    return y


@pytest.mark.parametrize("case", sorted(FC1))
def test_matches_reference_golden_vectors(case):
    g = FC1[case]
    dtype = golden_io.DTYPES[g["dtype"]]
    m, k, n = (int(v) for v in g["shape"])
    x, w, b = synth.fc1_inputs(m, k, n, dtype, int(g["seed"]))
    y = run(x, w, b if g["with_bias"] else None, g["act"], 1)
    assert_half_parity(y, golden_io.unpack(g["y"], dtype).reshape(m, n // 2), case)


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("layout", [0, 1, 2])
@pytest.mark.parametrize("dtype,mkn,bias", [
    (torch.bfloat16, (64, 128, 128), True),      # the reference's JIT numeric test shape (M=64, H=128, I=64)
    (torch.float16, (64, 128, 128), False),
    (torch.bfloat16, (256, 768, 1536), True),    # DiT-S like, several k-blocks and n-tiles
    (torch.bfloat16, (300, 200, 272), True),     # ragged M, K and N tiles (zero-filled tails)
    (torch.float16, (129, 1152, 528), True),
    (torch.bfloat16, (1, 64, 16), True),         # a single row
])
def test_matches_oracle(act, layout, dtype, mkn, bias):
    m, k, n = mkn
    x, w, b = synth.fc1_inputs(m, k, n, dtype, seed=50 + m % 7)
    y = run(x, w, b if bias else None, act, layout)
    exact = oracle.fc1_fwd(x, w, b if bias else None, act, gated=layout != 0, compute=torch.float64,
                           out_dtype=torch.float64)
    assert_half_parity(y, exact.to(dtype), f"fc1 {act} layout {layout} {dtype} {mkn}", exact=exact)


@pytest.mark.parametrize("dtype,mkn,bias", [
    (torch.bfloat16, (8192, 9216, 1152), False),  # the backward-dx GEMM of the DiT-XL/2 MLP: dz [M, 2I] @ W [2I, H]
    (torch.float16, (300, 200, 272), True),
    (torch.bfloat16, (64, 128, 128), True),
])
def test_identity_epilogue_is_a_plain_gemm(dtype, mkn, bias):
    m, k, n = mkn
    x, w, b = synth.fc1_inputs(m, k, n, dtype, seed=61)
    y = run(x, w, b if bias else None, "none", 0)
    want = x.double() @ w.double().T + (b.double() if bias else 0.0)
    assert_half_parity(y, want.to(dtype), f"plain gemm {dtype} {mkn}", exact=want)


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("dtype,mkn,bias", [
    (torch.bfloat16, (300, 200, 272), True),      # ragged tiles in every dimension
    (torch.float16, (129, 1152, 528), False),
    (torch.bfloat16, (1, 64, 16), True),
    (torch.bfloat16, (2048, 1152, 9216), True),   # DiT-XL/2 MLP width, several tiles per CTA
])
@pytest.mark.parametrize("pair", [0, 1])
def test_backward_dz_kernel_matches_oracle(tile_mode, pair, act, dtype, mkn, bias):
    """dz = d(value * act(gate)) / dz with z recomputed inside the kernel, against the fp64 closed form; on single-CTA
    tiles and on CTA-pair tiles."""
    tile_mode(pair)
    m, k, n = mkn
    x, w, b = synth.fc1_inputs(m, k, n, dtype, seed=71)
    dy = torch.randn(m, n // 2, generator=torch.Generator().manual_seed(72)).to(dtype)
    status = new_status()
    dz = capi.fc1_bwd_dz(x.to(DEV), w.to(DEV), b.to(DEV) if bias else None, dy.to(DEV), act, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    z = (x.double() @ w.double().T + (b.double() if bias else 0.0)).requires_grad_(True)
    zg, zv = z.chunk(2, dim=-1)
    a = torch.nn.functional.silu(zg) if act == "silu" else torch.nn.functional.gelu(zg, approximate="tanh")
    (want,) = torch.autograd.grad(a * zv, (z,), dy.double())
    assert_half_parity(dz.cpu(), want.to(dtype), f"dz {act} {dtype} {mkn}", exact=want)


@pytest.mark.parametrize("act", ["silu", "gelu"])
@pytest.mark.parametrize("dtype,mkn", [
    (torch.bfloat16, (300, 200, 272)),     # ragged row tile, ragged column chunk (136 outputs: 4 full chunks + 8)
    (torch.float16, (129, 1152, 528)),
    (torch.bfloat16, (1, 64, 16)),
    (torch.bfloat16, (2048, 1152, 9216)),  # DiT-XL/2 MLP width: 16 row tiles x 4 quarters of partial sums
])
@pytest.mark.parametrize("pair", [0, 1])
def test_backward_dz_with_dbias_in_the_epilogue(tile_mode, pair, act, dtype, mkn):
    """nd_fc1_bwd_dz_dbias: the same dz bit for bit, and dbias = the fp32 sum over the tokens of the STORED dz; on
    single-CTA tiles and on CTA-pair tiles (whose second CTA may lie wholly past the last row)."""
    tile_mode(pair)
    m, k, n = mkn
    x, w, b = synth.fc1_inputs(m, k, n, dtype, seed=73)
    dy = torch.randn(m, n // 2, generator=torch.Generator().manual_seed(74)).to(dtype)
    status = new_status()
    args = (x.to(DEV), w.to(DEV), b.to(DEV), dy.to(DEV), act)
    dz_only = capi.fc1_bwd_dz(*args, status=status)
    dz, dbias = capi.fc1_bwd_dz_dbias(*args, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(dz, dz_only)
    want = dz.double().sum(dim=0)
    # fp32 accumulation of up to m terms, then one rounding to the element type
    scale = dz.double().abs().sum(dim=0).clamp_min(1e-30)
    err = (dbias.double() - want).abs()
    assert bool((err <= 1e-6 * scale + torch.finfo(dtype).eps * want.abs() + 1e-30).all()), float((err / scale).max())
    again = capi.fc1_bwd_dz_dbias(*args, status=status)[1]
    assert torch.equal(dbias, again)


def test_backward_dx_binding_matches_matmul():
    gen = torch.Generator().manual_seed(8)
    dz = torch.randn(2, 150, 512, generator=gen).to(DEV, torch.bfloat16)
    w = (torch.randn(512, 264, generator=gen) * 0.05).to(DEV, torch.bfloat16)
    dx = ops.novadit_cuda.fused_fc1_bias_act_backward_dx(dz, w)
    want = dz.double() @ w.double()
    assert dx.shape == (2, 150, 264)
    assert_half_parity(dx.cpu(), want.cpu().to(torch.bfloat16), "backward dx", exact=want.cpu())


@pytest.fixture
def tile_mode():
    """Forces single-CTA (0) or two-CTA (1) tiles for one test and restores the per-problem choice."""
    lib = capi.lib()

    def force(mode):
        lib.nd_tune_fc1_pair(mode)

    yield force
    lib.nd_tune_fc1_pair(-1)


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("layout", [0, 1, 2])
@pytest.mark.parametrize("dtype,mkn", [
    (torch.bfloat16, (300, 200, 272)),     # ragged in M (also against the 256-row pair tile), K and N
    (torch.float16, (129, 1152, 528)),     # one row into the second CTA of a pair
    (torch.bfloat16, (1, 64, 16)),
    (torch.bfloat16, (1024, 1152, 4608)),  # more tiles than CTAs: every CTA walks several tiles and ring wraps
])
def test_both_tile_modes_match_oracle(tile_mode, pair, layout, dtype, mkn):
    m, k, n = mkn
    tile_mode(pair)
    x, w, b = synth.fc1_inputs(m, k, n, dtype, seed=77 + m % 5)
    y = run(x, w, b, "gelu", layout)
    exact = oracle.fc1_fwd(x, w, b, "gelu", gated=layout != 0, compute=torch.float64, out_dtype=torch.float64)
    assert_half_parity(y, exact.to(dtype), f"fc1 pair={pair} layout {layout} {dtype} {mkn}", exact=exact)


@pytest.mark.parametrize("pair", [0, 1])
def test_both_tile_modes_fp8(tile_mode, pair):
    m, k, n = 512, 1152, 4608
    tile_mode(pair)
    x, w, b = synth.fc1_inputs(m, k, n, torch.bfloat16, seed=5)
    qx, sx = capi.quantize_e4m3(x.to(DEV))
    qw, sw = capi.quantize_e4m3(w.to(DEV))
    status = new_status()
    y = capi.fc1_fwd(qx, qw, b.to(DEV), "silu", 1, alpha_dev=torch.cat([sx, sw]), out_dtype=torch.bfloat16,
                     status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    oqx, osx = oracle.quant_e4m3(x)
    oqw, osw = oracle.quant_e4m3(w)
    want = oracle.fc1_fwd_fp8(oqx, osx, oqw, osw, b, "silu", gated=True)
    assert oracle.rel_l2(y.cpu(), want) < FP8_REL_L2


@pytest.mark.parametrize("layout", [0, 1])
def test_config4_bf16(layout):
    """Workload config 4: M=8192, K=1152, N=4608, bias, GELU-tanh, bf16 (gated as in the reference, and plain)."""
    x, w, b = synth.fc1_inputs(8192, 1152, 4608, torch.bfloat16, seed=0)
    y = run(x, w, b, "gelu", layout)
    exact = oracle.fc1_fwd(x, w, b, "gelu", gated=layout != 0, compute=torch.float64, out_dtype=torch.float64)
    assert_half_parity(y, exact.to(torch.bfloat16), f"config4 layout {layout}", exact=exact)


@pytest.mark.parametrize("layout", [0, 1])
def test_config4_fp8_e4m3(layout):
    """FP8 e4m3 operands with per-tensor amax scales; bar: relative L2 <= 3e-2 against the fp32 GEMM of the
    de-quantised operands. The quantisation itself must match the oracle's bit for bit."""
    x, w, b = synth.fc1_inputs(8192, 1152, 4608, torch.bfloat16, seed=0)
    qx, sx = capi.quantize_e4m3(x.to(DEV))
    qw, sw = capi.quantize_e4m3(w.to(DEV))
    oqx, osx = oracle.quant_e4m3(x)
    oqw, osw = oracle.quant_e4m3(w)
    assert abs(float(sx) - osx) <= 1e-6 * osx and abs(float(sw) - osw) <= 1e-6 * osw
    assert torch.equal(qx.cpu().view(torch.uint8), oqx.view(torch.uint8))
    assert torch.equal(qw.cpu().view(torch.uint8), oqw.view(torch.uint8))
    status = new_status()
    y = capi.fc1_fwd(qx, qw, b.to(DEV), "gelu", layout, alpha_dev=torch.cat([sx, sw]), out_dtype=torch.bfloat16,
                     status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = oracle.fc1_fwd_fp8(oqx, osx, oqw, osw, b, "gelu", gated=layout != 0)
    rl = oracle.rel_l2(y.cpu(), want)
    assert rl <= FP8_REL_L2, f"fp8 rel_l2 {rl:.3e}"
    assert rl <= 5e-3, f"fp8 kernel error vs de-quantised fp32 GEMM unexpectedly large: {rl:.3e}"
    # information: distance to the un-quantised product (dominated by quantisation, not by the kernel)
    print("fp8 vs unquantised fp32:", oracle.rel_l2(y.cpu(), oracle.fc1_fwd(x, w, b, "gelu", gated=layout != 0)))


def test_large_case_properties():
    """M=32768, K=3072, N=12288: sampled rows against an fp32 GEMM and row independence."""
    m, k, n = 32768, 3072, 12288
    g = torch.Generator(device=DEV).manual_seed(21)
    x = torch.randn(m, k, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    b = (torch.randn(n, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    status = new_status()
    y = capi.fc1_fwd(x, w, b, "gelu", 1, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    rows = torch.randint(0, m, (256,), generator=g, device=DEV)
    xs = x[rows].contiguous()
    exact = oracle.fc1_fwd(xs.cpu(), w.cpu(), b.cpu(), "gelu", gated=True, compute=torch.float64,
                           out_dtype=torch.float64)
    assert_half_parity(y[rows].cpu(), exact.to(torch.bfloat16), "large case sampled rows", exact=exact)
    # the same rows computed as their own small problem give the same bits
    assert torch.equal(capi.fc1_fwd(xs, w, b, "gelu", 1), y[rows])


def test_unsupported_shapes_are_rejected_not_mangled():
    L = capi.lib()
    x = torch.zeros(8, 20, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(16, 20, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(8, 8, dtype=torch.bfloat16, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    # K = 20 bf16 is a 40-byte row pitch: not a multiple of 16 bytes, TMA cannot address it
    assert L.nd_fc1_fwd(capi.ND_BF16, capi.ND_BF16, 0, 1, x.data_ptr(), w.data_ptr(), None, 1.0, None,
                        y.data_ptr(), 8, 20, 16, None, st) == -2
    # n_out = 4 is not a multiple of 8
    assert L.nd_fc1_fwd(capi.ND_BF16, capi.ND_BF16, 0, 1, x.data_ptr(), w.data_ptr(), None, 1.0, None,
                        y.data_ptr(), 8, 16, 8, None, st) == -2


@pytest.fixture
def pair_tiles():
    """Forces whole single-CTA tiles (0) or evenly cut CTA-pair tiles (1) in nd_fc1_bwd_gemm for one test."""
    lib = capi.lib()

    def force(mode):
        lib.nd_tune_fc1_bwd_pair(mode)

    yield force
    lib.nd_tune_fc1_bwd_pair(-1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [
    (256, 192, 128),      # exactly one row of tiles, two k-blocks
    (304, 264, 520),      # ragged in all three dimensions (row tile, column tile and k-block hang over)
    (1024, 1152, 2304),   # H = 1152: six column tiles, reduction over 2I = 2304
    (128, 64, 64),        # a single tile narrower than one box row
    (6000, 1152, 520),    # 24 row blocks of five column tiles (the fifth a half tile): 120 tiles of 9 k-blocks cut
                          # into 74 ranges of 14 / 15 k-blocks, most tiles shared by two CTA pairs
    (520, 392, 72),       # a third, mostly empty row block; two column tiles, the second ragged
    (8, 8, 8),            # smallest legal problem
])
@pytest.mark.parametrize("workspace", [False, True])
def test_backward_gemms_read_their_operands_in_place(dtype, m, n, k, workspace, pair_tiles):
    """nd_fc1_bwd_gemm: op "dx" = a [m, k] @ b [k, n] (b MN-major), op "dw" = a [k, m]^T @ b [k, n] (both MN-major),
    against the fp64 products of the same 16-bit inputs; on whole 128 x 192 single-CTA tiles (no workspace) and on
    the 256 x 256 tiles of CTA pairs with the reduction cut evenly over the pairs (workspace)."""
    gen = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=gen) * 0.5).to(dtype)
    at = (torch.randn(k, m, generator=gen) * 0.5).to(dtype)
    b = (torch.randn(k, n, generator=gen) * 0.5).to(dtype)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pair_tiles(1 if workspace else 0)  # with a workspace the library would otherwise choose per problem
    got = capi.fc1_bwd_gemm(a.to(DEV), b.to(DEV), "dx", status=status, workspace=workspace)
    want = a.double() @ b.double()
    assert_half_parity_scaled(got.cpu(), want, f"dx gemm {dtype} {(m, n, k)}")
    again = capi.fc1_bwd_gemm(a.to(DEV), b.to(DEV), "dx", status=status, workspace=workspace)
    assert torch.equal(got, again), "the result must not depend on which CTA pair finishes a shared tile"
    got = capi.fc1_bwd_gemm(at.to(DEV), b.to(DEV), "dw", status=status, workspace=workspace)
    want = at.double().T @ b.double()
    assert_half_parity_scaled(got.cpu(), want, f"dw gemm {dtype} {(m, n, k)}")
    assert int(status.item()) == 0
    assert capi.lib().nd_device_error(0) == 0


def assert_half_parity_scaled(got, want64, what):
    """A GEMM output has no O(1) scale: compare relative to the result's rms (rel-L2 <= 1e-2 of the bar set, and no
    element further than 2e-2 rms-units + one rounding step from the fp64 value)."""
    rms = float(want64.pow(2).mean().sqrt())
    assert oracle.rel_l2(got.double(), want64) <= 1e-2, what
    step = torch.finfo(got.dtype).eps * want64.abs().clamp_min(rms)
    assert bool(((got.double() - want64).abs() <= 2e-2 * rms + step).all()), what


def test_backward_dw_and_dbias_bindings_and_the_autograd_function():
    gen = torch.Generator().manual_seed(21)
    b, s, h, inter = 2, 200, 264, 256
    x = torch.randn(b, s, h, generator=gen).to(DEV, torch.bfloat16)
    w = (torch.randn(2 * inter, h, generator=gen) * 0.05).to(DEV, torch.bfloat16)
    bias = (torch.randn(2 * inter, generator=gen) * 0.05).to(DEV, torch.bfloat16)
    dz = torch.randn(b, s, 2 * inter, generator=gen).to(DEV, torch.bfloat16)
    ext = ops.novadit_cuda
    dw = ext.fused_fc1_bias_act_backward_dw(dz, x)
    want = dz.double().reshape(-1, 2 * inter).T @ x.double().reshape(-1, h)
    assert dw.shape == (2 * inter, h)
    assert_half_parity_scaled(dw.cpu(), want.cpu(), "backward dW")
    db = ext.fused_fc1_bias_act_backward_dbias(dz)
    assert_half_parity_scaled(db.cpu(), dz.double().sum(dim=(0, 1)).cpu(), "backward dbias")
    # the whole Function: gradients of <y, dy> against the fp32 PyTorch definition on the same bf16 values
    dy = torch.randn(b, s, inter, generator=gen).to(DEV, torch.bfloat16)
    leaves = [t.clone().requires_grad_(True) for t in (x, w, bias)]
    y = ops.fused_fc1_bias_act(*leaves, "gelu")
    grads = torch.autograd.grad(y, leaves, dy)
    ref_leaves = [t.float().requires_grad_(True) for t in (x, w, bias)]
    yr = ops.fc1_bias_act_ref(*ref_leaves, "gelu")
    ref_grads = torch.autograd.grad(yr, ref_leaves, dy.float())
    for g, r, name in zip(grads, ref_grads, ("dx", "dW", "dbias")):
        assert oracle.rel_l2(g.float().cpu(), r.cpu()) < 1e-2, name


def test_fc1_launches_leave_the_device_error_word_clear():
    """The FC1 kernels record an expired wait in the device error word (codes 101..) as well as in the caller's
    status word, so that launches through the torch extension, which passes no status word, are covered by
    nd_device_error() too. Nothing expires in a healthy run: after forward, FP8 forward and backward-dz launches
    with NO status word the error word must still read zero."""
    L = capi.lib()
    assert L.nd_device_error(1) >= 0  # clear whatever an earlier test may have left
    x, w, b = (t.to(DEV) for t in synth.fc1_inputs(512, 256, 512, torch.bfloat16, seed=4))
    dy = torch.randn(512, 256, device=DEV).to(torch.bfloat16)
    capi.fc1_fwd(x, w, b, "gelu", 1)            # status=None
    capi.fc1_bwd_dz(x, w, b, dy, "gelu")        # status=None
    qx, sx = capi.quantize_e4m3(x)
    qw, sw = capi.quantize_e4m3(w)
    capi.fc1_fwd(qx, qw, b, "silu", 0, alpha_dev=torch.cat([sx, sw]), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert L.nd_device_error(0) == 0
