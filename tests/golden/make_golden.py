"""Generate golden vectors from the reference's own PyTorch implementation.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py /path/to/novadit-checkout

It imports `novadit.ops` from that checkout (its CPU functions `adaln_ref`,
`adarmsnorm_ref`, `gate_act_ref`, `geglu_ref`, `fc1_bias_act_ref`), evaluates
them and their autograd backward on seeded inputs, and writes small `.npz`
fixtures beside this script. The reference checkout is needed only here; the
tests read the committed fixtures.

Half-precision tensors are stored as their raw 16-bit patterns (`*_bits`
arrays) so that no rounding happens on the way through numpy.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from novadit_b200 import synth  # noqa: E402


def pack(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy()
    return t.numpy()


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(pack(t).tobytes()).hexdigest()


def norm_case(ops, kind, batch, seq, hidden, dtype, eps, seed, mod3d=False, rows_kept=None):
    x, scale, shift, dy = synth.norm_inputs(batch, seq, hidden, dtype, seed)
    if mod3d:
        scale, shift = scale.unsqueeze(1), shift.unsqueeze(1)
    ref = ops.adaln_ref if kind == "layer" else ops.adarmsnorm_ref
    y = ref(x, scale, shift, eps)  # forward exactly as the reference evaluates it (fp32 inside, one rounding)
    # Backward: autograd of the same function on upcast copies of the identical bits, rounded once.
    # (Autograd on half-precision leaves would add the three x.float() branches in bf16/fp16 and
    # round dx three times; the reference's own CUDA tests compare with an fp32 formula instead.)
    xr = x.float().requires_grad_(True)
    sr = scale.float().requires_grad_(True)
    hr = shift.float().requires_grad_(True)
    dx, dscale, dshift = torch.autograd.grad(ref(xr, sr, hr, eps), (xr, sr, hr), dy.float())
    dx = dx.to(dtype)
    dscale, dshift = dscale.reshape(batch, hidden), dshift.reshape(batch, hidden)
    out = {
        "kind": kind, "shape": np.array([batch, seq, hidden]), "dtype": str(dtype).split(".")[-1],
        "eps": eps, "seed": seed, "mod3d": int(mod3d),
        "x_sha": sha(x), "dy_sha": sha(dy),
        "dscale": pack(dscale.float()), "dshift": pack(dshift.float()),
    }
    if rows_kept is None:
        out.update(y=pack(y), dx=pack(dx))
    else:
        rows = torch.arange(0, batch * seq, rows_kept)
        out.update(rows=rows.numpy(),
                   y=pack(y.reshape(-1, hidden)[rows]), dx=pack(dx.reshape(-1, hidden)[rows]))
    return out


def gate_case(ops, act, batch, seq, inter, dtype, seed):
    x, dy = synth.gate_act_inputs(batch, seq, inter, dtype, seed)
    # evaluated on upcast copies of the same bits and rounded once, the way the
    # reference's own backward test builds its expectation
    xf = x.float().requires_grad_(True)
    y = ops.gate_act_ref(xf, act)
    (dz,) = torch.autograd.grad(y, (xf,), dy.float())
    chain = ops.gate_act_ref(x, act)  # the input-dtype chain, for information
    return {
        "act": act, "shape": np.array([batch, seq, inter]), "dtype": str(dtype).split(".")[-1],
        "seed": seed, "x_sha": sha(x),
        "y": pack(y.detach().to(dtype)), "dz": pack(dz.to(dtype)), "y_chain": pack(chain),
    }


def fc1_case(ops, act, m, k, n, dtype, seed, with_bias):
    x, w, b = synth.fc1_inputs(m, k, n, dtype, seed)
    bias = b if with_bias else None
    y = ops.fc1_bias_act_ref(x.float(), w.float(), None if bias is None else bias.float(), act)
    return {
        "act": act, "shape": np.array([m, k, n]), "dtype": str(dtype).split(".")[-1], "seed": seed,
        "with_bias": int(with_bias), "x_sha": sha(x), "y": pack(y.to(dtype)),
    }


def main() -> None:
    ref_root = sys.argv[1]
    sys.path.insert(0, ref_root)
    import novadit.ops as ops  # the reference package

    torch.manual_seed(0)
    torch.set_num_threads(1)  # fixed summation order inside the reference's reductions
    bf16, f16, f32 = torch.bfloat16, torch.float16, torch.float32

    norm = {}
    for kind in ("layer", "rms"):
        norm[f"{kind}_bf16_aligned"] = norm_case(ops, kind, 2, 5, 768, bf16, 1e-5, 11)
        norm[f"{kind}_f16_ragged"] = norm_case(ops, kind, 2, 3, 770, f16, 1e-5, 12)
        norm[f"{kind}_bf16_mod3d"] = norm_case(ops, kind, 3, 7, 1152, bf16, 1e-6, 13, mod3d=True)
        norm[f"{kind}_bf16_s257"] = norm_case(ops, kind, 2, 257, 136, bf16, 1e-5, 14)
        # workload config 1: fp32, B=2 S=256 H=768, eps 1e-6, seed 0; y/dx kept for every 32nd row
        norm[f"{kind}_f32_config1"] = norm_case(ops, kind, 2, 256, 768, f32, 1e-6, 0, rows_kept=32)
    flat = {f"{c}/{k}": v for c, d in norm.items() for k, v in d.items()}
    np.savez_compressed(os.path.join(HERE, "norm_golden.npz"), **flat)

    gate = {}
    for act in ("silu", "gelu"):
        gate[f"{act}_f32_ragged"] = gate_case(ops, act, 2, 4, 385, f32, 21)
        gate[f"{act}_bf16_aligned"] = gate_case(ops, act, 2, 4, 768, bf16, 22)
        gate[f"{act}_f16_aligned"] = gate_case(ops, act, 1, 3, 4608, f16, 23)
    flat = {f"{c}/{k}": v for c, d in gate.items() for k, v in d.items()}
    np.savez_compressed(os.path.join(HERE, "gate_act_golden.npz"), **flat)

    fc1 = {}
    for act in ("silu", "gelu"):
        fc1[f"{act}_bf16_bias"] = fc1_case(ops, act, 64, 128, 128, bf16, 31, True)
        fc1[f"{act}_bf16_nobias"] = fc1_case(ops, act, 64, 128, 128, bf16, 32, False)
        fc1[f"{act}_f16_bias_ragged"] = fc1_case(ops, act, 48, 192, 96, f16, 33, True)
    flat = {f"{c}/{k}": v for c, d in fc1.items() for k, v in d.items()}
    np.savez_compressed(os.path.join(HERE, "fc1_golden.npz"), **flat)

    # exact known answers for the weight (de)interleave helpers
    w = torch.arange(24, dtype=torch.float32).reshape(6, 4)
    b = torch.arange(6, dtype=torch.float32)
    wi = ops.interleave_weight(w)
    np.savez_compressed(
        os.path.join(HERE, "interleave_golden.npz"),
        w=w.numpy(), b=b.numpy(), w_inter=wi.numpy(), b_inter=ops.interleave_bias(b).numpy(),
        w_round=ops.un_interleave_weight(wi).numpy(),
        split_gate=ops.split_gated_weight(wi)[0].numpy(), split_value=ops.split_gated_weight(wi)[1].numpy(),
    )
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
