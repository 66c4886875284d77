"""ctypes binding of the C ABI (`include/novadit_b200.h`) plus tensor-level helpers.

This is the route the parity tests and the benchmark take: torch tensors are
used only as device buffers (`data_ptr()`), every call goes through the
`extern "C"` entry points of ``libnovadit_b200.so``. There is no fallback: if the
library is missing, importing this module's `lib()` raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_size_t, c_void_p

import torch

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libnovadit_b200.so")

ND_F16, ND_BF16, ND_F32, ND_E4M3 = 0, 1, 2, 3
ACT_SILU, ACT_GELU = 0, 1
ACT_IDS = {"silu": ACT_SILU, "gelu": ACT_GELU, "none": 2}
DTYPE_IDS = {torch.float16: ND_F16, torch.bfloat16: ND_BF16, torch.float32: ND_F32,
             torch.float8_e4m3fn: ND_E4M3}

_SHAPE4 = [c_int64, c_int64, c_int64, c_int64]  # rows, row_start, seq_len, hidden

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "nd_status_string": (ctypes.c_char_p, [c_int]),
    "nd_last_cuda_error": (c_int, []),
    "nd_version": (c_int, []),
    "nd_device_error": (c_int, [c_int]),
    "nd_tune_norm_tile_rows": (None, [c_int]),
    "nd_tune_norm_variant": (None, [c_int]),
    "nd_tune_norm_stages": (None, [c_int]),
    "nd_tune_norm_pdl": (None, [c_int]),
    "nd_tune_norm_chunks_per_sm": (None, [c_int]),
    "nd_tune_norm_wait_test": (None, [ctypes.c_uint64, c_int]),
    "nd_adaln_fwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             *_SHAPE4, c_float, c_void_p]),
    "nd_adaln_bwd_dx": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                *_SHAPE4, c_void_p]),
    "nd_norm_dparam_ws_bytes": (c_size_t, _SHAPE4),
    "nd_adaln_bwd_dparam": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, *_SHAPE4, c_void_p, c_size_t, c_void_p]),
    "nd_adaln_bwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, *_SHAPE4, c_void_p, c_size_t, c_void_p]),
    "nd_noalloc_scratch_bytes": (c_size_t, []),
    "nd_adaln_bwd_noalloc": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, *_SHAPE4, c_void_p]),
    "nd_adarms_fwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, *_SHAPE4,
                              c_float, c_void_p]),
    "nd_adarms_bwd_dx": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, *_SHAPE4,
                                 c_void_p]),
    "nd_adarms_bwd_dparam": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     *_SHAPE4, c_void_p, c_size_t, c_void_p]),
    "nd_adarms_bwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, *_SHAPE4, c_void_p, c_size_t, c_void_p]),
    "nd_adaln_fwd_e4m3": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, *_SHAPE4, c_float, c_void_p]),
    "nd_adarms_fwd_e4m3": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   *_SHAPE4, c_float, c_void_p]),
    "nd_gate_act_fwd": (c_int, [c_int, c_int, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "nd_gate_act_bwd": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                c_void_p]),
    "nd_gate_act_bwd_gate_first": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                           c_void_p]),
    "nd_out_residual_fwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "nd_qkv_pack_fwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "nd_qkv_pack_bwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "nd_gated_residual_fwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, *_SHAPE4, c_void_p]),
    "nd_gated_residual_ws_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64, c_int64]),
    "nd_adaln_fwd_residual": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, *_SHAPE4, c_float, c_void_p]),
    "nd_adarms_fwd_residual": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, *_SHAPE4, c_float, c_void_p]),
    "nd_gated_residual_bwd_add": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          *_SHAPE4, c_int64, c_void_p]),
    "nd_gated_residual_bwd": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, *_SHAPE4, c_int64,
                                      c_void_p]),
    "nd_fc1_fwd": (c_int, [c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_float,
                           c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "nd_fc1_bwd_dz": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                              c_int64, c_void_p, c_void_p]),
    "nd_fc1_bwd_dbias_ws_bytes": (c_size_t, [c_int64, c_int64]),
    "nd_fc1_bwd_dz_dbias": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_size_t, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "nd_fc1_bwd_gemm_ws_bytes": (c_size_t, []),
    "nd_fc1_bwd_gemm": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_size_t,
                                c_void_p, c_void_p]),
    "nd_colsum_ws_bytes": (c_size_t, [c_int64]),
    "nd_colsum": (c_int, [c_int, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_size_t, c_void_p]),
    "nd_tune_gate_act": (None, [c_int, c_int]),
    "nd_tune_fc1_pair": (None, [c_int]),
    "nd_tune_fc1_bwd_pair": (None, [c_int]),
    "nd_tune_fc1_pdl": (None, [c_int]),
    "nd_tune_fc1_trace": (None, [c_void_p]),
    "nd_amax_ws_bytes": (c_size_t, []),
    "nd_amax": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_size_t, c_void_p]),
    "nd_quant_e4m3": (c_int, [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
}

_lib = None


class NovaditError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded C-ABI library. Raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NovaditError(
                f"{LIB_PATH} is missing: build it with `python -m novadit_b200.build` "
                "(the operators have no CPU or PyTorch fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().nd_status_string(status).decode()
        extra = ""
        if status == -3:
            extra = f" (cudaError {lib().nd_last_cuda_error()})"
        raise NovaditError(f"{what}: {msg}{extra}")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts: torch.Tensor) -> None:
    """Every tensor contiguous, on CUDA, on ONE device, and that device current: the C ABI launches on the current
    device's stream, so pointers of another device would be handed to the wrong GPU (the torch extension sets
    the device itself; this ctypes layer asks the caller to)."""
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda or not t.is_contiguous():
            raise NovaditError("tensors must be contiguous CUDA tensors")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise NovaditError(f"tensors on different devices: {dev} and {t.device}")
    if dev is not None and dev.index != torch.cuda.current_device():
        raise NovaditError(f"tensors live on {dev} but the current device is cuda:{torch.cuda.current_device()}: "
                           f"wrap the call in `with torch.cuda.device({dev.index})`")


class Workspace:
    """Cached, 256-byte aligned device scratch buffers (grown on demand, never initialised), one per device
    and stream: launches on different streams may run concurrently and must not share scratch."""

    def __init__(self) -> None:
        self.bufs: dict[tuple, torch.Tensor] = {}

    def get(self, nbytes: int, device, stream: int = 0) -> torch.Tensor | None:
        if nbytes == 0:
            return None
        key = (torch.device(device), stream)
        buf = self.bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            self.bufs[key] = buf
        return buf


_WS = Workspace()


# ---------------------------------------------------------------- norm operators
def norm_fwd(kind, x, scale, shift, eps, *, stats=True, row_start=0, seq_len=None, y=None,
             mean=None, invstd=None):
    """AdaLN (`kind="layer"`) / AdaRMSNorm (`kind="rms"`) forward on rows `x` [rows, H] (or [B,S,H]).

    Returns (y, mean, invstd) for "layer" and (y, inv_rms) for "rms"; statistics are None when
    `stats` is False. `scale`/`shift` are the FULL [B, H] modulation arrays; `row_start` is the
    global index of x's first row.
    """
    _need_cuda(x, scale, shift)
    hidden = x.shape[-1]
    if seq_len is None:
        seq_len = x.shape[1] if x.dim() == 3 else 1
    rows = x.numel() // hidden
    y = torch.empty_like(x) if y is None else y
    lead = x.shape[:-1]
    dt = DTYPE_IDS[x.dtype]
    if kind == "layer":
        if stats:
            mean = torch.empty(lead, dtype=torch.float32, device=x.device) if mean is None else mean
            invstd = torch.empty(lead, dtype=torch.float32, device=x.device) if invstd is None else invstd
        check(lib().nd_adaln_fwd(dt, _ptr(x), _ptr(scale), _ptr(shift), _ptr(y), _ptr(mean), _ptr(invstd),
                                 rows, row_start, seq_len, hidden, eps, _stream()), "nd_adaln_fwd")
        return y, mean, invstd
    if stats:
        invstd = torch.empty(lead, dtype=torch.float32, device=x.device) if invstd is None else invstd
    check(lib().nd_adarms_fwd(dt, _ptr(x), _ptr(scale), _ptr(shift), _ptr(y), _ptr(invstd),
                              rows, row_start, seq_len, hidden, eps, _stream()), "nd_adarms_fwd")
    return y, invstd


def norm_fwd_e4m3(kind, x, scale, shift, eps, q_scale, amax=None, *, stats=True, row_start=0, seq_len=None):
    """Forward with FP8 e4m3 output: returns (q, mean, invstd) / (q, inv_rms). `q_scale` is a device float (the
    de-quantisation scale), `amax` an optional device float that receives max(amax, max |y|)."""
    _need_cuda(x, scale, shift, q_scale, amax)
    hidden = x.shape[-1]
    if seq_len is None:
        seq_len = x.shape[1] if x.dim() == 3 else 1
    rows = x.numel() // hidden
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    lead = x.shape[:-1]
    dt = DTYPE_IDS[x.dtype]
    invstd = torch.empty(lead, dtype=torch.float32, device=x.device) if stats else None
    if kind == "layer":
        mean = torch.empty(lead, dtype=torch.float32, device=x.device) if stats else None
        check(lib().nd_adaln_fwd_e4m3(dt, _ptr(x), _ptr(scale), _ptr(shift), _ptr(q), _ptr(mean), _ptr(invstd),
                                      _ptr(q_scale), _ptr(amax), rows, row_start, seq_len, hidden, eps, _stream()),
              "nd_adaln_fwd_e4m3")
        return q, mean, invstd
    check(lib().nd_adarms_fwd_e4m3(dt, _ptr(x), _ptr(scale), _ptr(shift), _ptr(q), _ptr(invstd), _ptr(q_scale),
                                   _ptr(amax), rows, row_start, seq_len, hidden, eps, _stream()),
          "nd_adarms_fwd_e4m3")
    return q, invstd


def norm_bwd(kind, dy, x, scale, mean, invstd, *, mode="fused", row_start=0, seq_len=None, batch=None,
             dx=None, dscale=None, dshift=None, ws=None):
    """Backward. mode: "dx", "dparam" or "fused". Returns (dx, dscale, dshift) with None for parts
    not computed. dscale/dshift are [batch, H] fp32 over the FULL batch; rows of samples the shard
    does not touch are left as they were (zero when allocated here)."""
    _need_cuda(dy, x, scale, mean, invstd)
    hidden = x.shape[-1]
    if seq_len is None:
        seq_len = x.shape[1] if x.dim() == 3 else 1
    rows = x.numel() // hidden
    if batch is None:
        batch = x.shape[0] if x.dim() == 3 else (row_start + rows + seq_len - 1) // seq_len
    dt = DTYPE_IDS[x.dtype]
    L = lib()
    want_dx, want_dp = mode in ("dx", "fused"), mode in ("dparam", "fused")
    if want_dx and dx is None:
        dx = torch.empty_like(x)
    ws_t, ws_bytes = None, 0
    if want_dp:
        if dscale is None:
            dscale = torch.zeros(batch, hidden, dtype=torch.float32, device=x.device)
        if dshift is None:
            dshift = torch.zeros(batch, hidden, dtype=torch.float32, device=x.device)
        ws_bytes = L.nd_norm_dparam_ws_bytes(rows, row_start, seq_len, hidden)
    st = _stream()
    if want_dp:
        ws_t = (ws or _WS).get(ws_bytes, x.device, st or 0)
    shape = (rows, row_start, seq_len, hidden)
    if kind == "layer":
        if mode == "dx":
            check(L.nd_adaln_bwd_dx(dt, _ptr(dy), _ptr(x), _ptr(scale), _ptr(mean), _ptr(invstd), _ptr(dx),
                                    *shape, st), "nd_adaln_bwd_dx")
        elif mode == "dparam":
            check(L.nd_adaln_bwd_dparam(dt, _ptr(dy), _ptr(x), _ptr(mean), _ptr(invstd), _ptr(dscale),
                                        _ptr(dshift), *shape, _ptr(ws_t), ws_bytes, st), "nd_adaln_bwd_dparam")
        else:
            check(L.nd_adaln_bwd(dt, _ptr(dy), _ptr(x), _ptr(scale), _ptr(mean), _ptr(invstd), _ptr(dx),
                                 _ptr(dscale), _ptr(dshift), *shape, _ptr(ws_t), ws_bytes, st), "nd_adaln_bwd")
    else:
        if mode == "dx":
            check(L.nd_adarms_bwd_dx(dt, _ptr(dy), _ptr(x), _ptr(scale), _ptr(invstd), _ptr(dx), *shape, st),
                  "nd_adarms_bwd_dx")
        elif mode == "dparam":
            check(L.nd_adarms_bwd_dparam(dt, _ptr(dy), _ptr(x), _ptr(invstd), _ptr(dscale), _ptr(dshift),
                                         *shape, _ptr(ws_t), ws_bytes, st), "nd_adarms_bwd_dparam")
        else:
            check(L.nd_adarms_bwd(dt, _ptr(dy), _ptr(x), _ptr(scale), _ptr(invstd), _ptr(dx), _ptr(dscale),
                                  _ptr(dshift), *shape, _ptr(ws_t), ws_bytes, st), "nd_adarms_bwd")
    return dx, dscale, dshift


# ---------------------------------------------------------------- gate-act
def gate_act_fwd(x, act="silu", y=None):
    _need_cuda(x)
    inter = x.shape[-1] // 2
    rows = x.numel() // (2 * inter)
    y = torch.empty(*x.shape[:-1], inter, dtype=x.dtype, device=x.device) if y is None else y
    check(lib().nd_gate_act_fwd(DTYPE_IDS[x.dtype], ACT_IDS[act], _ptr(x), _ptr(y), rows, inter, _stream()),
          "nd_gate_act_fwd")
    return y


def gate_act_bwd(dy, x, act="silu", dz=None, gate_first=False):
    """dz for rows [up | gate] (default) or [gate | up] (`gate_first`: FC1's pre-activation layout)."""
    _need_cuda(dy, x)
    inter = x.shape[-1] // 2
    rows = x.numel() // (2 * inter)
    dz = torch.empty_like(x) if dz is None else dz
    fn = lib().nd_gate_act_bwd_gate_first if gate_first else lib().nd_gate_act_bwd
    check(fn(DTYPE_IDS[x.dtype], ACT_IDS[act], _ptr(dy), _ptr(x), _ptr(dz), rows, inter, _stream()),
          "nd_gate_act_bwd_gate_first" if gate_first else "nd_gate_act_bwd")
    return dz


# ---------------------------------------------------------------- gated residual
GATED_TILE_ROWS = 8


def gated_residual_fwd(x, branch, gate, *, row_start=0, seq_len=None):
    """y = x + gate[b] * branch; x, branch [B,S,H] (or a row shard [rows,H] with row_start / seq_len), gate [B,H]."""
    _need_cuda(x, branch, gate)
    hidden = x.shape[-1]
    if seq_len is None:
        seq_len = x.shape[1] if x.dim() == 3 else 1
    rows = x.numel() // hidden
    y = torch.empty_like(x)
    check(lib().nd_gated_residual_fwd(DTYPE_IDS[x.dtype], _ptr(x), _ptr(branch), _ptr(gate), _ptr(y), rows, row_start,
                                      seq_len, hidden, _stream()), "nd_gated_residual_fwd")
    return y


def gated_residual_bwd(dy, branch, gate, *, row_start=0, seq_len=None):
    """(dbranch, dgate_partials [samples, tiles, H] fp32); dgate = partials.sum(1)."""
    _need_cuda(dy, branch, gate)
    hidden = dy.shape[-1]
    if seq_len is None:
        seq_len = dy.shape[1] if dy.dim() == 3 else 1
    rows = dy.numel() // hidden
    L = lib()
    nbytes = L.nd_gated_residual_ws_bytes(rows, row_start, seq_len, hidden, GATED_TILE_ROWS)
    tiles = (seq_len + GATED_TILE_ROWS - 1) // GATED_TILE_ROWS
    part = torch.empty(nbytes // (4 * hidden * tiles), tiles, hidden, dtype=torch.float32, device=dy.device)
    dbranch = torch.empty_like(dy)
    check(L.nd_gated_residual_bwd(DTYPE_IDS[dy.dtype], _ptr(dy), _ptr(branch), _ptr(gate), _ptr(dbranch), _ptr(part),
                                  rows, row_start, seq_len, hidden, GATED_TILE_ROWS, _stream()), "nd_gated_residual_bwd")
    return dbranch, part


def gated_residual_bwd_add(dy, dres, branch, gate, *, row_start=0, seq_len=None):
    """(dsum = dy + dres, dbranch = gate * dsum, dgate_partials of dsum * branch)."""
    _need_cuda(dy, dres, branch, gate)
    hidden = dy.shape[-1]
    if seq_len is None:
        seq_len = dy.shape[1] if dy.dim() == 3 else 1
    rows = dy.numel() // hidden
    L = lib()
    nbytes = L.nd_gated_residual_ws_bytes(rows, row_start, seq_len, hidden, GATED_TILE_ROWS)
    tiles = (seq_len + GATED_TILE_ROWS - 1) // GATED_TILE_ROWS
    part = torch.empty(nbytes // (4 * hidden * tiles), tiles, hidden, dtype=torch.float32, device=dy.device)
    dsum, dbranch = torch.empty_like(dy), torch.empty_like(dy)
    check(L.nd_gated_residual_bwd_add(DTYPE_IDS[dy.dtype], _ptr(dy), _ptr(dres), _ptr(branch), _ptr(gate), _ptr(dsum),
                                      _ptr(dbranch), _ptr(part), rows, row_start, seq_len, hidden, GATED_TILE_ROWS,
                                      _stream()), "nd_gated_residual_bwd_add")
    return dsum, dbranch, part


def norm_fwd_residual(kind, x, branch, gate, scale, shift, eps, *, stats=True, row_start=0, seq_len=None):
    """x_new = x + gate[b] * branch (gate None: x + branch) and its AdaLN ("layer") / AdaRMSNorm ("rms") in one
    pass. Returns (x_new, y, mean, invstd) / (x_new, y, inv_rms)."""
    _need_cuda(x, branch, gate, scale, shift)
    hidden = x.shape[-1]
    if seq_len is None:
        seq_len = x.shape[1] if x.dim() == 3 else 1
    rows = x.numel() // hidden
    x_new, y = torch.empty_like(x), torch.empty_like(x)
    lead = x.shape[:-1]
    dt = DTYPE_IDS[x.dtype]
    invstd = torch.empty(lead, dtype=torch.float32, device=x.device) if stats else None
    if kind == "layer":
        mean = torch.empty(lead, dtype=torch.float32, device=x.device) if stats else None
        check(lib().nd_adaln_fwd_residual(dt, _ptr(x), _ptr(branch), _ptr(gate), _ptr(scale), _ptr(shift), _ptr(x_new),
                                          _ptr(y), _ptr(mean), _ptr(invstd), rows, row_start, seq_len, hidden, eps,
                                          _stream()), "nd_adaln_fwd_residual")
        return x_new, y, mean, invstd
    check(lib().nd_adarms_fwd_residual(dt, _ptr(x), _ptr(branch), _ptr(gate), _ptr(scale), _ptr(shift), _ptr(x_new),
                                       _ptr(y), _ptr(invstd), rows, row_start, seq_len, hidden, eps, _stream()),
          "nd_adarms_fwd_residual")
    return x_new, y, invstd


# ---------------------------------------------------------------- FC1
def fc1_fwd(x, w, bias=None, act="silu", gated=True, *, alpha=1.0, alpha_dev=None, out_dtype=None, y=None,
            status=None):
    """x [..., K], w [N, K] -> y [..., N/2] (gated) or [..., N]. Operands bf16/fp16/e4m3."""
    _need_cuda(x, w, bias)
    k = x.shape[-1]
    m = x.numel() // k
    n = w.shape[0]
    if out_dtype is None:
        out_dtype = torch.bfloat16 if x.dtype == torch.float8_e4m3fn else x.dtype
    n_out = n // 2 if gated else n
    if y is None:
        y = torch.empty(*x.shape[:-1], n_out, dtype=out_dtype, device=x.device)
    check(lib().nd_fc1_fwd(DTYPE_IDS[x.dtype], DTYPE_IDS[out_dtype], ACT_IDS[act], int(gated), _ptr(x), _ptr(w),
                           _ptr(bias), float(alpha), _ptr(alpha_dev), _ptr(y), m, k, n, _ptr(status), _stream()),
          "nd_fc1_fwd")
    return y


def fc1_bwd_dz(x, w, bias, dy, act="silu", status=None):
    """dz [..., N] of the gated FC1 (w rows [gate | value]) from x, w, bias and dy [..., N/2], z recomputed inside."""
    _need_cuda(x, w, bias, dy)
    k = x.shape[-1]
    m = x.numel() // k
    n = w.shape[0]
    dz = torch.empty(*x.shape[:-1], n, dtype=x.dtype, device=x.device)
    check(lib().nd_fc1_bwd_dz(DTYPE_IDS[x.dtype], ACT_IDS[act], _ptr(x), _ptr(w), _ptr(bias), _ptr(dy), _ptr(dz),
                              m, k, n, _ptr(status), _stream()), "nd_fc1_bwd_dz")
    return dz


def fc1_bwd_dz_dbias(x, w, bias, dy, act="silu", status=None):
    """(dz, dbias) of the gated FC1: dz as fc1_bwd_dz, dbias [N] = dz summed over the tokens inside the same launch."""
    _need_cuda(x, w, bias, dy)
    k = x.shape[-1]
    m = x.numel() // k
    n = w.shape[0]
    L = lib()
    dz = torch.empty(*x.shape[:-1], n, dtype=x.dtype, device=x.device)
    dbias = torch.empty(n, dtype=x.dtype, device=x.device)
    ws = torch.empty(max(L.nd_fc1_bwd_dbias_ws_bytes(m, n), 16), dtype=torch.uint8, device=x.device)
    check(L.nd_fc1_bwd_dz_dbias(DTYPE_IDS[x.dtype], ACT_IDS[act], _ptr(x), _ptr(w), _ptr(bias), _ptr(dy), _ptr(dz),
                                _ptr(dbias), _ptr(ws), ws.numel(), m, k, n, _ptr(status), _stream()),
          "nd_fc1_bwd_dz_dbias")
    return dz, dbias


_GEMM_WS: dict = {}


def fc1_bwd_gemm(a, b, op: str, status=None, workspace=True):
    """op "dx": a [m, k] @ b [k, n]; op "dw": a [k, m]^T @ b [k, n]. Returns c [m, n] in a's dtype.
    `workspace=False` passes no workspace (whole single-CTA tiles instead of evenly cut CTA-pair tiles)."""
    _need_cuda(a, b, status)
    if op == "dx":
        m, k = a.shape
    else:
        k, m = a.shape
    n = b.shape[1]
    c = torch.empty(m, n, dtype=a.dtype, device=a.device)
    L = lib()
    st = _stream()
    ws = None
    if workspace:
        key = (a.device, st or 0)  # per device AND stream: launches on two streams must not share partial tiles
        ws = _GEMM_WS.get(key)
        if ws is None:
            ws = _GEMM_WS[key] = torch.empty(L.nd_fc1_bwd_gemm_ws_bytes(), dtype=torch.uint8, device=a.device)
    check(L.nd_fc1_bwd_gemm(DTYPE_IDS[a.dtype], 0 if op == "dx" else 1, _ptr(a), _ptr(b), _ptr(c), m, n, k,
                            _ptr(ws), ws.numel() if ws is not None else 0, _ptr(status), st), "nd_fc1_bwd_gemm")
    return c


def colsum(x):
    """Column sums of a [rows, cols] fp16 / bf16 matrix (fp32 accumulation, fixed order), in x's dtype."""
    _need_cuda(x)
    rows, cols = x.shape
    L = lib()
    ws = torch.empty(L.nd_colsum_ws_bytes(cols), dtype=torch.uint8, device=x.device)
    out = torch.empty(cols, dtype=x.dtype, device=x.device)
    check(L.nd_colsum(DTYPE_IDS[x.dtype], _ptr(x), rows, cols, _ptr(out), _ptr(ws), ws.numel(), _stream()), "nd_colsum")
    return out


_AMAX_WS: dict = {}


def quantize_e4m3(x):
    """Per-tensor amax scaling to e4m3 on the device. Returns (q, scale[1] fp32 device tensor)."""
    _need_cuda(x)
    L = lib()
    dev = x.device
    st = _stream()
    key = (dev, st or 0)  # per device AND stream: two streams must not share the per-CTA maxima
    ws = _AMAX_WS.get(key)
    if ws is None:
        ws = _AMAX_WS[key] = torch.empty(L.nd_amax_ws_bytes(), dtype=torch.uint8, device=dev)
    amax = torch.empty(1, dtype=torch.float32, device=dev)
    scale = torch.empty(1, dtype=torch.float32, device=dev)
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=dev)
    check(L.nd_amax(DTYPE_IDS[x.dtype], _ptr(x), x.numel(), _ptr(amax), _ptr(ws), ws.numel(), st), "nd_amax")
    check(L.nd_quant_e4m3(DTYPE_IDS[x.dtype], _ptr(x), x.numel(), _ptr(amax), _ptr(q), _ptr(scale), st),
          "nd_quant_e4m3")
    return q, scale
