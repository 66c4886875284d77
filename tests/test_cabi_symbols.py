"""The C-ABI library loads and exports every symbol the headers under `include/` declare (no GPU needed)."""
from __future__ import annotations

import ctypes
import os
import re

import pytest

from novadit_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADERS = [os.path.join(ROOT, "include", name) for name in ("novadit_b200.h", "novadit_b200_tuning.h")]


def declared_symbols(headers=HEADERS) -> list[str]:
    names = set()
    for header in headers:
        text = re.sub(r"/\*.*?\*/", "", open(header).read(), flags=re.S)
        names.update(re.findall(r"\b(nd_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_operator_header_holds_no_tuning_hook():
    assert not [n for n in declared_symbols(HEADERS[:1]) if n.startswith("nd_tune_")]
    assert all(n.startswith("nd_tune_") for n in declared_symbols(HEADERS[1:]))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("nd_adaln_fwd", "nd_adaln_bwd_dx", "nd_adaln_bwd_dparam", "nd_adaln_bwd", "nd_adarms_fwd",
                 "nd_adarms_bwd_dx", "nd_adarms_bwd_dparam", "nd_adarms_bwd", "nd_gate_act_fwd", "nd_gate_act_bwd",
                 "nd_fc1_fwd", "nd_amax", "nd_quant_e4m3", "nd_norm_dparam_ws_bytes"):
        assert must in names


def test_library_exports_every_declared_symbol():
    if not os.path.exists(capi.LIB_PATH):
        pytest.fail(f"{capi.LIB_PATH} not built: run `python -m novadit_b200.build`")
    handle = ctypes.CDLL(capi.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} declared in the header but not exported"


def test_ctypes_signatures_cover_the_header():
    assert sorted(capi.SIGNATURES) == declared_symbols()


def test_status_strings_and_pure_host_queries():
    L = capi.lib()
    assert L.nd_status_string(0) == b"ok"
    for code in (-1, -2, -3, -4, -5):
        assert L.nd_status_string(code) not in (b"ok", b"unknown status")
    assert L.nd_version() >= 100
    assert L.nd_amax_ws_bytes() >= 1024
    # argument validation happens before any CUDA call
    assert L.nd_adaln_fwd(1, None, None, None, None, None, None, 4, 0, 2, 8, 1e-5, None) == -1
    assert L.nd_adaln_fwd(1, None, None, None, None, None, None, 0, 0, 2, 8, 1e-5, None) == 0  # empty shard
    assert L.nd_adaln_fwd(1, None, None, None, None, None, None, 4, 0, 0, 8, 1e-5, None) == -1  # seq_len 0
    assert L.nd_gate_act_fwd(1, 7, None, None, 4, 8, None) == -2  # unknown activation
    assert L.nd_gate_act_fwd(1, 0, None, None, 0, 8, None) == 0
    assert L.nd_fc1_fwd(1, 1, 0, 1, None, None, None, 1.0, None, None, 4, 8, 7, None, None) == -1  # odd n, gated
    assert L.nd_fc1_fwd(1, 2, 0, 1, None, None, None, 1.0, None, None, 4, 8, 8, None, None) == -2  # fp32 output
    assert L.nd_fc1_fwd(1, 1, 0, 1, None, None, None, 1.0, None, None, 0, 8, 8, None, None) == 0
    assert L.nd_amax(1, None, 0, None, None, 0, None) == -1
