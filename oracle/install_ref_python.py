"""Install the reference's pure-Python package (`novadit`) into baseline/_ref - test infrastructure.

    python -m oracle.install_ref_python [path to a checkout of the reference]

What it is for: the drop-in test (tests/test_gpu_dropin_reference.py) and the block-stack harness run the
reference's OWN `novadit.ops` / `novadit.modules`, unchanged, on top of this library's `novadit_cuda` extension.
Only the reference's Python is installed; its CUDA extension is not (this library replaces it).

How: `pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <copy of the checkout>`. The
checkout may be read-only and pip writes build files into the source tree, hence the copy. The reference's
setup.py adds its CUDA extension whenever torch finds a CUDA toolkit, and hands setuptools absolute source paths,
which setuptools rejects ("setup script specifies an absolute path"); its own fallback - an empty extension list
when `import torch` fails (setup.py:23-28) - is taken by putting a stub `torch` module that raises ImportError on
the build's PYTHONPATH. Nothing of the reference is modified, and nothing is copied into the tracked tree:
baseline/_ref is git-ignored.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TARGET = os.path.join(ROOT, "baseline", "_ref")


def installed() -> bool:
    return os.path.isfile(os.path.join(TARGET, "novadit", "ops", "__init__.py"))


def install(ref_root: str) -> None:
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "reference")
        shutil.copytree(ref_root, src, ignore=shutil.ignore_patterns(".git", "*.ncu-rep", "build", "*.egg-info"))
        stub = os.path.join(tmp, "stub")
        os.makedirs(stub)
        with open(os.path.join(stub, "torch.py"), "w") as f:
            f.write('raise ImportError("not needed to install the pure-Python package")\n')
        env = dict(os.environ, PYTHONPATH=stub)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", TARGET, "--upgrade", src]
        proc = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=tmp)
        if proc.returncode != 0:
            raise RuntimeError("pip install of the reference failed:\n" + proc.stdout[-2000:] + proc.stderr[-2000:])
    print("installed the reference's Python package into", TARGET)


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NOVADIT_REFERENCE_ROOT", "")
    if not os.path.isdir(os.path.join(root, "novadit")):
        raise SystemExit("usage: python -m oracle.install_ref_python <checkout of the reference>")
    install(root)
