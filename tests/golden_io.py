"""Load the committed golden fixtures (outputs of the reference's own functions)."""
from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def load(name: str) -> dict[str, dict]:
    """Return {case: {field: value}} for `tests/golden/<name>.npz`."""
    raw = np.load(os.path.join(GOLDEN_DIR, name + ".npz"), allow_pickle=False)
    cases: dict[str, dict] = {}
    for key in raw.files:
        case, field = key.split("/", 1)
        v = raw[key]
        cases.setdefault(case, {})[field] = v.item() if v.ndim == 0 else v
    return cases


def unpack(arr: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    """Inverse of the generator's `pack`: int16 bit patterns back to fp16/bf16."""
    t = torch.from_numpy(np.ascontiguousarray(arr))
    if dtype in (torch.bfloat16, torch.float16):
        return t.view(dtype)
    return t


def bits_sha(t: torch.Tensor) -> str:
    import hashlib

    t = t.detach().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.view(torch.int16)
    return hashlib.sha256(t.numpy().tobytes()).hexdigest()
