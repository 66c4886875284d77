"""Drop-in under the reference's own Python: `novadit.ops` / `novadit.modules`, unchanged, on this library's kernels.

The reference imports its native extension as the top-level module `novadit_cuda` inside a try/except
(`novadit/ops/__init__.py:10-18`) and silently falls back to PyTorch when the import fails. Integration route A puts
this package's directory, which holds `novadit_cuda.<abi>.so`, on `sys.path`; nothing else changes. The test does
exactly that in a fresh interpreter (so that nothing of `novadit_b200` is imported by accident), checks that the
reference picked the extension up, and runs the reference's `NovaDiTBlock` at the DiT-XL/2 shape with its
`use_fused_*` switches on against the same block with them off (the reference's PyTorch path), forward and
backward. Needs the reference's Python package: an install under `baseline/_ref` (skipped when absent).
"""
from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "novadit_b200")
REF_DIR = os.path.join(ROOT, "baseline", "_ref")

SCRIPT = r"""
import json, os, sys
import torch
import novadit.ops as ops
import novadit_cuda
from novadit.modules import NovaDiTBlock, NovaDiTMLP

out = {"has_ext": bool(ops.HAS_NOVADIT_CUDA), "ext_file": novadit_cuda.__file__,
       "same_module": ops.novadit_cuda is novadit_cuda, "novadit_b200_imported": "novadit_b200" in sys.modules}
dev, dt = "cuda", torch.bfloat16

def rel(a, b):
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))

torch.manual_seed(0)
B, S, H, heads = 32, 256, 1152, 16
fused = NovaDiTBlock(H, heads, attention_backend="sdpa", device=dev, dtype=dt)           # every use_fused_* on
plain = NovaDiTBlock(H, heads, attention_backend="sdpa", use_fused_adaln=False, use_fused_qkv_pack=False,
                     use_fused_out_residual=False, use_fused_gate_act=False, device=dev, dtype=dt)
plain.load_state_dict(fused.state_dict())
x = torch.randn(B, S, H, device=dev).to(dt)
mods = [(torch.randn(B, H, device=dev) * 0.1).to(dt) for _ in range(4)]
dy = torch.randn(B, S, H, device=dev).to(dt)
res = []
for blk in (fused, plain):
    xi = x.clone().requires_grad_(True)
    mi = [m.clone().requires_grad_(True) for m in mods]
    y = blk(xi, *mi)
    grads = torch.autograd.grad(y, (xi, *mi, *blk.parameters()), dy)
    res.append((y, grads))
(yf, gf), (yp, gp) = res
out["block_y_rel_l2"] = rel(yf, yp)
out["block_dx_rel_l2"] = rel(gf[0], gp[0])
out["block_dmod_rel_l2"] = max(rel(a, b) for a, b in zip(gf[1:5], gp[1:5]))
out["block_dparam_rel_l2"] = rel(torch.cat([g.flatten() for g in gf[5:]]), torch.cat([g.flatten() for g in gp[5:]]))

# The MLP with the fused FC1 switched on (the block never passes that flag: dit_block.py:40-48) against the
# reference's own PyTorch definition of the same function. Forward only: the reference's Function re-enters
# autograd in its backward with grad mode off (ops/fc1_bias_act.py:248-268) and raises under a plain backward
# pass whatever extension is loaded.
mlp = NovaDiTMLP(H, 4 * H, activation="gelu", use_fused_fc1_bias_act=True, device=dev, dtype=dt)
xm = torch.randn(4, 256, H, device=dev).to(dt)
with torch.no_grad():
    ym = mlp(xm)
    yr = mlp.fc2(ops.fc1_bias_act_ref(xm, mlp.fc1.weight, mlp.fc1.bias, "gelu"))
out["mlp_y_rel_l2"] = rel(ym, yr)
torch.cuda.synchronize()
print("RESULT " + json.dumps(out))
"""


def test_reference_python_runs_on_this_extension():
    if not os.path.isdir(os.path.join(REF_DIR, "novadit")):
        pytest.skip("no install of the reference's Python package under baseline/_ref")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([PKG_DIR, REF_DIR])  # route A: the extension's directory first
    proc = subprocess.run([sys.executable, "-c", SCRIPT], capture_output=True, text=True, env=env, cwd="/", timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    line = [ln for ln in proc.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    out = json.loads(line[len("RESULT "):])
    assert out["has_ext"] and out["same_module"], out
    assert os.path.dirname(out["ext_file"]) == PKG_DIR, out["ext_file"]  # this library's .so, nobody else's
    assert not out["novadit_b200_imported"]
    # two bf16 pipelines that round at different points (the fused operators round once, the PyTorch path after
    # every operation): a few bf16 steps, not more
    assert out["block_y_rel_l2"] < 1e-2, out
    assert out["block_dx_rel_l2"] < 2e-2 and out["block_dmod_rel_l2"] < 2e-2 and out["block_dparam_rel_l2"] < 2e-2, out
    assert out["mlp_y_rel_l2"] < 1e-2, out
