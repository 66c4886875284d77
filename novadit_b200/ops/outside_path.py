"""Names the reference's `novadit.ops` exports that lie OUTSIDE the accelerated operator path.

They exist so that code written against the reference's package imports unchanged: the two `torch.compile`
comparison baselines of novadit/ops/norm_compile.py are not provided.
"""
from __future__ import annotations


def adaln_compile(*args, **kwargs):
    raise NotImplementedError("the torch.compile comparison baseline is not part of this library; use fused_adaln")


def adarmsnorm_compile(*args, **kwargs):
    raise NotImplementedError("the torch.compile comparison baseline is not part of this library; use fused_adarmsnorm")
