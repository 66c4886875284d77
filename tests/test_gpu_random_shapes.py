"""Seeded random shapes for every operator family against the CPU oracle: widths that are and are not multiples
of the vector width, rows that do not fill tiles or groups, samples of one row, shards that cut samples."""
from __future__ import annotations

import random

import pytest
import torch

from novadit_b200 import capi, synth
from oracle import novadit_oracle as oracle
from tests.helpers import FP8_REL_L2, assert_f32_parity, assert_half_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"


def norm_cases():
    rnd = random.Random(1234)
    cases = []
    for i in range(36):
        h = rnd.choice([8, 24, 64, 72, 128, 200, 256, 520, 768, 770, 1000, 1152, 1536, 2048, 4096, 4104])
        b = rnd.randint(1, 5)
        s = rnd.choice([1, 2, 3, 5, 7, 16, 33, 100, 257])
        dtype = rnd.choice([torch.bfloat16, torch.float16])
        kind = rnd.choice(["layer", "rms"])
        cases.append(pytest.param(kind, dtype, b, s, h, 500 + i, id=f"{kind}-{str(dtype)[6:]}-{b}x{s}x{h}"))
    return cases


@pytest.mark.parametrize("kind,dtype,b,s,h,seed", norm_cases())
def test_norm_random_shapes(kind, dtype, b, s, h, seed):
    x, scale, shift, dy = synth.norm_inputs(b, s, h, dtype, seed)
    xd, sd, hd, gd = (t.to(DEV) for t in (x, scale, shift, dy))
    rows = b * s
    rnd = random.Random(seed)
    lo = rnd.randint(0, rows - 1)
    hi = rnd.randint(lo + 1, rows)
    if kind == "layer":
        y, mean, inv = capi.norm_fwd(kind, xd, sd, hd, 1e-6)
        wy, _, _ = oracle.adaln_fwd(x, scale, shift, 1e-6, compute=torch.float64, round_out=False)
        wdx, wds, wdh = oracle.adaln_bwd(dy, x, scale, 1e-6, compute=torch.float64, round_out=False)
    else:
        y, inv = capi.norm_fwd(kind, xd, sd, hd, 1e-6)
        mean = None
        wy, _ = oracle.adarms_fwd(x, scale, shift, 1e-6, compute=torch.float64, round_out=False)
        wdx, wds, wdh = oracle.adarms_bwd(dy, x, scale, 1e-6, compute=torch.float64, round_out=False)
    dx, ds, dh = capi.norm_bwd(kind, gd, xd, sd, mean, inv)
    # a shard [lo, hi) of the rows: forward rows equal the full result bit for bit, partial dscale/dshift only
    # touch the shard's samples
    xs = xd.reshape(-1, h)[lo:hi].contiguous()
    part = capi.norm_fwd(kind, xs, sd, hd, 1e-6, row_start=lo, seq_len=s)
    torch.cuda.synchronize()
    assert_half_parity(y, wy.to(dtype), "y", exact=wy)
    assert_half_parity(dx, wdx.to(dtype), "dx", exact=wdx)
    assert_f32_parity(ds, wds.float(), "dscale")
    assert_f32_parity(dh, wdh.float(), "dshift")
    assert torch.equal(part[0], y.reshape(-1, h)[lo:hi])
    assert capi.lib().nd_device_error(0) == 0


def gate_cases():
    rnd = random.Random(99)
    cases = []
    for i in range(16):
        inter = rnd.choice([1, 7, 8, 33, 64, 200, 1000, 2048, 2049, 4608, 6144])
        rows = rnd.choice([1, 2, 3, 5, 31, 64, 257])
        dtype = rnd.choice([torch.bfloat16, torch.float16, torch.float32])
        act = rnd.choice(["silu", "gelu"])
        cases.append(pytest.param(act, dtype, rows, inter, 700 + i, id=f"{act}-{str(dtype)[6:]}-{rows}x{inter}"))
    return cases


@pytest.mark.parametrize("act,dtype,rows,inter,seed", gate_cases())
def test_gate_act_random_shapes(act, dtype, rows, inter, seed):
    x, dy = synth.gate_act_inputs(1, rows, inter, dtype, seed)
    y = capi.gate_act_fwd(x.to(DEV), act)
    dz = capi.gate_act_bwd(dy.to(DEV), x.to(DEV), act)
    torch.cuda.synchronize()
    wy = oracle.gate_act_fwd(x, act, compute=torch.float64, round_out=False)
    wdz = oracle.gate_act_bwd(dy, x, act, compute=torch.float64, round_out=False)
    if dtype == torch.float32:
        assert oracle.rel_l2(y.cpu(), wy.float()) < 1e-5 and oracle.rel_l2(dz.cpu(), wdz.float()) < 1e-5
    else:
        assert_half_parity(y, wy.to(dtype), "y", exact=wy)
        assert_half_parity(dz, wdz.to(dtype), "dz", exact=wdz)


def fc1_cases():
    rnd = random.Random(7)
    cases = []
    for i in range(20):
        m = rnd.choice([1, 5, 64, 127, 128, 129, 255, 257, 700, 1500])
        k = rnd.choice([8, 64, 72, 200, 512, 1152, 2048])
        n = rnd.choice([16, 48, 256, 272, 528, 1040, 2304])
        dtype = rnd.choice([torch.bfloat16, torch.float16])
        layout = rnd.choice([0, 1, 2])
        pair = rnd.choice([0, 1])
        act = rnd.choice(["silu", "gelu"])
        cases.append(pytest.param(act, dtype, m, k, n, layout, pair, 900 + i,
                                  id=f"{act}-{str(dtype)[6:]}-{m}x{k}x{n}-layout{layout}-pair{pair}"))
    return cases


@pytest.mark.parametrize("act,dtype,m,k,n,layout,pair,seed", fc1_cases())
def test_fc1_random_shapes(act, dtype, m, k, n, layout, pair, seed):
    import novadit_b200.ops as ops

    x, w, b = synth.fc1_inputs(m, k, n, dtype, seed)
    wd, bd = w.to(DEV), b.to(DEV)
    if layout == 2:
        wd, bd = ops.interleave_weight(wd), ops.interleave_bias(bd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    lib = capi.lib()
    try:
        lib.nd_tune_fc1_pair(pair)
        y = capi.fc1_fwd(x.to(DEV), wd, bd, act, layout, status=status)
        dz = None
        if layout == 1:
            dy = torch.randn(m, n // 2, generator=torch.Generator().manual_seed(seed)).to(dtype)
            dz = capi.fc1_bwd_dz(x.to(DEV), wd, bd, dy.to(DEV), act, status=status)
        torch.cuda.synchronize()
    finally:
        lib.nd_tune_fc1_pair(-1)
    assert int(status.item()) == 0
    want = oracle.fc1_fwd(x, w, b, act, gated=layout != 0, compute=torch.float64, out_dtype=torch.float64)
    assert_half_parity(y, want.to(dtype), "y", exact=want)
    if dz is not None:
        z = (x.double() @ w.double().T + b.double()).requires_grad_(True)
        zg, zv = z.chunk(2, dim=-1)
        a = torch.nn.functional.silu(zg) if act == "silu" else torch.nn.functional.gelu(zg, approximate="tanh")
        (wdz,) = torch.autograd.grad(a * zv, (z,), dy.double())
        assert_half_parity(dz.cpu(), wdz.to(dtype), "dz", exact=wdz)


@pytest.mark.parametrize("m,k,n,seed", [(130, 256, 272, 1), (1000, 1152, 528, 2), (64, 128, 48, 3)])
def test_fc1_fp8_random_shapes(m, k, n, seed):
    x, w, b = synth.fc1_inputs(m, k, n, torch.bfloat16, seed)
    qx, sx = capi.quantize_e4m3(x.to(DEV))
    qw, sw = capi.quantize_e4m3(w.to(DEV))
    y = capi.fc1_fwd(qx, qw, b.to(DEV), "gelu", 1, alpha_dev=torch.cat([sx, sw]), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    oqx, osx = oracle.quant_e4m3(x)
    oqw, osw = oracle.quant_e4m3(w)
    assert oracle.rel_l2(y.cpu(), oracle.fc1_fwd_fp8(oqx, osx, oqw, osw, b, "gelu", gated=True)) < FP8_REL_L2
