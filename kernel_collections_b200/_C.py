"""ctypes binding of libxkv.so (the C ABI declared in include/xkv.h).

There is no CPU fallback: if the library cannot be loaded (and cannot be built because
nvcc is absent) importing this module raises, and every op raises on a non-CUDA tensor.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

from . import build as _build

XKV_F32, XKV_BF16, XKV_F16 = 0, 1, 2
SCORE_DENSE, SCORE_LATENT, SCORE_RECON_ROPE, SCORE_RECON = 0, 1, 2, 3
VALUE_DENSE, VALUE_LATENT = 0, 1
FLAG_LOGITS_ONLY, FLAG_FORCE_GENERIC, FLAG_RECON_SINGLE_CTA, FLAG_PV_MMA_SYNC, FLAG_RECON_PAIR = 1, 2, 4, 8, 16
FLAG_LATENT_MMA_SYNC = 32

_DTYPES = {torch.float32: XKV_F32, torch.bfloat16: XKV_BF16, torch.float16: XKV_F16}

EXPORTS = [
    "xkv_version", "xkv_decode_params_size", "xkv_strerror", "xkv_decode_plan", "xkv_decode_workspace_bytes", "xkv_decode",
    "xkv_workspace_status", "xkv_decode_builtin_scratch",
    "xkv_dense_decode", "xkv_absorbed_decode", "xkv_recon_rope_decode", "xkv_qab_logits",
    "xkv_mla_decode", "xkv_group_decode_workspace_bytes", "xkv_group_decode", "xkv_merge",
    "xkv_rope_table", "xkv_rope_query", "xkv_latent_append", "xkv_peer_allgather",
]


class DecodeParams(C.Structure):
    """Mirror of struct xkv_decode_params (include/xkv.h); field order and types must match."""
    _fields_ = [
        ("dtype", C.c_int32), ("score_mode", C.c_int32), ("value_mode", C.c_int32), ("flags", C.c_uint32),
        ("batch", C.c_int32), ("num_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("kv_len", C.c_int32),
        ("head_dim", C.c_int32), ("value_dim", C.c_int32), ("k_rank", C.c_int32), ("v_rank", C.c_int32),
        ("tail_dim", C.c_int32),
        ("k_proj_heads", C.c_int32), ("v_proj_heads", C.c_int32),
        ("num_splits", C.c_int32), ("pos_offset", C.c_int32),
        ("sm_scale", C.c_float), ("theta", C.c_float), ("logit_cap", C.c_float),
        ("inv_freq", C.c_void_p), ("rope_table", C.c_void_p),
        ("q", C.c_void_p), ("q_sb", C.c_int64), ("q_sh", C.c_int64),
        ("q_tail", C.c_void_p), ("qt_sb", C.c_int64), ("qt_sh", C.c_int64),
        ("k", C.c_void_p), ("k_sb", C.c_int64), ("k_sl", C.c_int64), ("k_sh", C.c_int64),
        ("k_tail", C.c_void_p), ("kt_sb", C.c_int64), ("kt_sl", C.c_int64),
        ("k_proj", C.c_void_p), ("kp_sb", C.c_int64), ("kp_sh", C.c_int64), ("kp_sr", C.c_int64),
        ("kp_sd", C.c_int64),
        ("v", C.c_void_p), ("v_sb", C.c_int64), ("v_sl", C.c_int64), ("v_sh", C.c_int64),
        ("v_proj", C.c_void_p), ("vp_sb", C.c_int64), ("vp_sh", C.c_int64), ("vp_sr", C.c_int64),
        ("vp_sd", C.c_int64),
        ("out", C.c_void_p), ("o_sb", C.c_int64), ("o_sh", C.c_int64),
        ("logits", C.c_void_p), ("lg_sb", C.c_int64), ("lg_sh", C.c_int64),
        ("kv_lens", C.c_void_p),
        ("lse_out", C.c_void_p), ("lse_sb", C.c_int64),
        ("mask", C.c_void_p), ("mask_sb", C.c_int64), ("mask_sh", C.c_int64),
    ]


_lib = None
_lib_lock = threading.Lock()


def lib_path() -> str:
    return _build.LIB_PATH


def load():
    """Load (building first if the in-tree library is absent or stale and nvcc exists)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        try:
            if _build.needs_build():
                _build.build()
        except Exception as e:  # stale-but-present library is still usable; absent is fatal
            if not os.path.exists(path):
                raise RuntimeError(f"libxkv.so is missing and could not be built: {e}") from e
        lib = C.CDLL(path)
        lib.xkv_version.restype = C.c_int
        lib.xkv_strerror.restype = C.c_char_p
        lib.xkv_strerror.argtypes = [C.c_int]
        lib.xkv_decode_plan.restype = C.c_char_p
        lib.xkv_decode_plan.argtypes = [C.POINTER(DecodeParams)]
        lib.xkv_decode_workspace_bytes.restype = C.c_size_t
        lib.xkv_decode_workspace_bytes.argtypes = [C.POINTER(DecodeParams)]
        for name in ("xkv_decode", "xkv_dense_decode", "xkv_absorbed_decode", "xkv_recon_rope_decode",
                     "xkv_qab_logits", "xkv_mla_decode"):
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(DecodeParams), C.c_void_p, C.c_size_t, C.c_void_p]
        lib.xkv_group_decode_workspace_bytes.restype = C.c_size_t
        lib.xkv_group_decode_workspace_bytes.argtypes = [C.POINTER(DecodeParams), C.c_int]
        lib.xkv_group_decode.restype = C.c_int
        lib.xkv_group_decode.argtypes = [C.POINTER(DecodeParams), C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
        lib.xkv_merge.restype = C.c_int
        lib.xkv_merge.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                  C.c_int, C.c_int64, C.c_int64, C.c_void_p]
        lib.xkv_rope_table.restype = C.c_int
        lib.xkv_rope_table.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
        lib.xkv_rope_query.restype = C.c_int
        lib.xkv_rope_query.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int64,
                                       C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p]
        lib.xkv_latent_append.restype = C.c_int
        lib.xkv_latent_append.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64,
                                          C.c_int64, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_void_p]
        lib.xkv_peer_allgather.restype = C.c_int
        lib.xkv_peer_allgather.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_size_t, C.c_int, C.c_int,
                                           C.c_uint32, C.c_void_p, C.c_void_p]
        lib.xkv_decode_params_size.restype = C.c_size_t
        lib.xkv_decode_builtin_scratch.restype = C.c_int
        lib.xkv_decode_builtin_scratch.argtypes = [C.POINTER(DecodeParams), C.c_void_p]
        lib.xkv_workspace_status.restype = C.c_int
        lib.xkv_workspace_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
        if lib.xkv_version() != 1:
            raise RuntimeError("libxkv.so version mismatch")
        if lib.xkv_decode_params_size() != C.sizeof(DecodeParams):
            raise RuntimeError("xkv_decode_params layout differs between libxkv.so and its ctypes mirror")
        _lib = lib
        return lib


def strerror(rc: int) -> str:
    return load().xkv_strerror(rc).decode()


def check(rc: int, what: str):
    if rc == 0:
        return
    msg = f"{what}: {strerror(rc)} (status {rc})"
    if rc in (-1, -2, -3, -8):
        raise ValueError(msg)
    raise RuntimeError(msg)


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {t.dtype}; expected float32, bfloat16 or float16") from None


def require_cuda(*tensors):
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("kernel_collections_b200 runs on CUDA tensors only (no CPU fallback)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"all tensors of one call must live on one device; got {dev} and {t.device}")


# ---- workspace: one grow-only byte buffer per (device, stream) ------------------------------
_workspaces: dict = {}


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (_device_of(device), torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


_inv_freq_cache: dict = {}


def inv_freq(dim: int, theta: float, device: torch.device) -> torch.Tensor:
    """fp32 theta^(-2j/dim), computed with the same torch expression the reference's rotary
    helper uses (flash_recontruction/rope/rope_ref.py:4) so the angles agree bit for bit."""
    key = (dim, float(theta), str(device))
    t = _inv_freq_cache.get(key)
    if t is None:
        t = (1.0 / (float(theta) ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))).to(device)
        _inv_freq_cache[key] = t
    return t


class DeviceTimeout(RuntimeError):
    """A bounded device-side wait of a tensor-core kernel expired; the output of that call is not valid."""


_check_status = os.environ.get("XKV_CHECK_STATUS", "0") not in ("", "0")


def set_check_status(on: bool) -> bool:
    """Turn the post-call status check on or off (default: the XKV_CHECK_STATUS environment variable
    as it was when this module was imported, else off).  With it on, every decode call synchronises
    its stream, reads the status words its kernels left in the workspace and raises DeviceTimeout
    when a bounded wait gave up.  Returns the previous setting."""
    global _check_status
    prev, _check_status = _check_status, bool(on)
    return prev


def _device_of(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def raise_on_status(ws_ptr: int, stream: int, what: str):
    """Read the status words at `ws_ptr` (synchronises `stream`) and raise if the call failed."""
    detail = (C.c_int32 * 8)()
    rc = load().xkv_workspace_status(ws_ptr, stream, detail)
    if rc == -6:
        d = list(detail)
        raise DeviceTimeout(f"{what}: {strerror(rc)} (role {d[1]}, tile {d[2]}, chunk {d[3]}, step {d[4]}); "
                            "the output of this call is not valid")
    check(rc, what)


def run_decode(params: DecodeParams, device: torch.device, entry: str = "xkv_decode", check_status=None):
    lib = load()
    with torch.cuda.device(_device_of(device)):
        nbytes = lib.xkv_decode_workspace_bytes(C.byref(params))
        if nbytes == 0:
            # let the entry point produce the precise status
            rc = getattr(lib, entry)(C.byref(params), None, 0, None)
            check(rc if rc != 0 else -2, entry)
        ws = workspace(device, nbytes)
        stream = torch.cuda.current_stream(device).cuda_stream
        rc = getattr(lib, entry)(C.byref(params), ws.data_ptr(), ws.numel(), stream)
        check(rc, entry)
        if _check_status if check_status is None else check_status:
            raise_on_status(ws.data_ptr(), stream, entry)


def last_status(device: torch.device):
    """Synchronise the current stream and return (status, detail[8]) of the last call that used
    this (device, stream) workspace."""
    key = (_device_of(device), torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None:
        return 0, [0] * 8
    detail = (C.c_int32 * 8)()
    with torch.cuda.device(key[0]):
        rc = load().xkv_workspace_status(buf.data_ptr(), key[1], detail)
    return rc, list(detail)


BUILTIN_SCRATCH_BYTES = 8 << 20


def run_decode_builtin_scratch(params: DecodeParams, device: torch.device):
    """Launch through xkv_decode_builtin_scratch: no workspace tensor, no allocation."""
    with torch.cuda.device(_device_of(device)):
        rc = load().xkv_decode_builtin_scratch(C.byref(params), torch.cuda.current_stream(device).cuda_stream)
    check(rc, "xkv_decode_builtin_scratch")


def plan_name(params: DecodeParams, device=None):
    if device is not None and device.type == "cuda":
        with torch.cuda.device(_device_of(device)):
            r = load().xkv_decode_plan(C.byref(params))
    else:
        r = load().xkv_decode_plan(C.byref(params))
    return r.decode() if r else None
