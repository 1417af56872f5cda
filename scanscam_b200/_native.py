"""ctypes binding of the C-ABI library (``include/scanscam_b200.h``).

This is the same boundary any other FFI client would bind; the test-suite and the benchmark
call the kernels through it with raw device pointers taken from torch tensors.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# SCANSCAM_B200_LIB selects another build of the same library (e.g. the checked build, see build.py).
LIB_PATH = os.environ.get("SCANSCAM_B200_LIB") or os.path.join(_HERE, "libscanscam_b200.so")

OK, ERR_BAD_ARG, ERR_ALIGNMENT, ERR_LAUNCH, ERR_DEVICE_WAIT, ERR_WORKSPACE, ERR_UNSUPPORTED, ERR_DEVICE_CHECK = range(8)
VARIANT_AUTO, VARIANT_WARP, VARIANT_TMA, VARIANT_LOOKBACK, VARIANT_FLAT, VARIANT_FLAT_ANY = range(6)
CL_AUTO, CL_PLAIN, CL_LOOKBACK, CL_LOOKBACK_TMA, CL_STREAM, CL_CHUNKED, CL_NARROW = range(7)  # ssb_cl_variant_t

_p, _i64, _int, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t

# name -> (restype, argtypes); one entry per declaration in include/scanscam_b200.h
SIGNATURES = {
    "ssb_version": (_int, []),
    "ssb_status_string": (ctypes.c_char_p, [_int]),
    "ssb_last_error": (ctypes.c_char_p, []),
    "ssb_scan_fwd_f32": (_int, [_p, _p, _p, _i64, _i64, _p, _p]),
    "ssb_scan_fwd_f64": (_int, [_p, _p, _p, _i64, _i64, _p, _p]),
    "ssb_scan_fwd_f32_ex": (_int, [_p, _p, _p, _i64, _i64, _p, _int, _p, _sz, _p]),
    "ssb_scan_f64_workspace_bytes": (_sz, [_i64, _i64]),
    "ssb_scan_fwd_f64_ex": (_int, [_p, _p, _p, _i64, _i64, _p, _p, _sz, _p]),
    "ssb_scan_bwd_f64_ex": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _p, _sz, _p]),
    "ssb_scan_fwd_f32_static": (_int, [_p, _p, _p, _i64, _i64, _p, _p]),
    "ssb_scan_bwd_f32": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _p]),
    "ssb_scan_bwd_f64": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _p]),
    "ssb_scan_bwd_f32_ex": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _int, _p, _sz, _p]),
    "ssb_scan_sigmoid_fwd_f32": (_int, [_p, _p, _p, _i64, _i64, _p, _p]),
    "ssb_scan_sigmoid_bwd_f32": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _p]),
    "ssb_scan_fwd_bf16": (_int, [_p, _p, _p, _i64, _i64, _p, _p]),
    "ssb_scan_bwd_bf16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _p]),
    "ssb_scan_fwd_f16": (_int, [_p, _p, _p, _i64, _i64, _p, _p]),
    "ssb_scan_bwd_f16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _p]),
    "ssb_scan_sigmoid_fwd_bf16": (_int, [_p, _p, _p, _i64, _i64, _p, _p]),
    "ssb_scan_sigmoid_bwd_bf16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _p]),
    "ssb_scan_sigmoid_fwd_f16": (_int, [_p, _p, _p, _i64, _i64, _p, _p]),
    "ssb_scan_sigmoid_bwd_f16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _p]),
    "ssb_scan_bwd_recompute_bf16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _p]),
    "ssb_scan_bwd_recompute_f16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _p]),
    "ssb_scan_bwd_recompute_workspace_bytes": (_sz, [_i64, _i64]),
    "ssb_scan_bwd_recompute_f32": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _p, _p, _p, _sz, _p]),
    "ssb_scan_workspace_bytes": (_sz, [_i64, _i64, _int]),
    "ssb_scan_cl_fwd_f32": (_int, [_p, _p, _p, _i64, _i64, _i64, _p]),
    "ssb_scan_cl_fwd_f64": (_int, [_p, _p, _p, _i64, _i64, _i64, _p]),
    "ssb_scan_cl_bwd_f32": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p]),
    "ssb_scan_cl_bwd_f64": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p]),
    "ssb_scan_recommend": (_int, [_i64, _i64, _int, _int, _int]),
    "ssb_scan_cl_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "ssb_scan_cl_h16_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "ssb_scan_cl_sigmoid_fwd_f32": (_int, [_p, _p, _p, _i64, _i64, _i64, _p, _sz, _p]),
    "ssb_scan_cl_sigmoid_bwd_f32": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _sz, _p]),
    "ssb_scan_cl_sigmoid_fwd_bf16": (_int, [_p, _p, _p, _i64, _i64, _i64, _p, _sz, _p]),
    "ssb_scan_cl_sigmoid_bwd_bf16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _sz, _p]),
    "ssb_scan_cl_sigmoid_fwd_f16": (_int, [_p, _p, _p, _i64, _i64, _i64, _p, _sz, _p]),
    "ssb_scan_cl_sigmoid_bwd_f16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _sz, _p]),
    "ssb_scan_cl_fwd_bf16": (_int, [_p, _p, _p, _i64, _i64, _i64, _p, _sz, _p]),
    "ssb_scan_cl_bwd_bf16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _sz, _p]),
    "ssb_scan_cl_fwd_f16": (_int, [_p, _p, _p, _i64, _i64, _i64, _p, _sz, _p]),
    "ssb_scan_cl_bwd_f16": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _sz, _p]),
    "ssb_scan_cl_recommend": (_int, [_i64, _i64, _i64, _int, _int, _int]),
    "ssb_scan_cl_variant_workspace_bytes": (_sz, [_i64, _i64, _i64, _int, _int]),
    "ssb_scan_cl_sigmoid_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "ssb_scan_cl_fwd_f32_ex": (_int, [_p, _p, _p, _i64, _i64, _i64, _int, _p, _sz, _p]),
    "ssb_scan_cl_bwd_f32_ex": (_int, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _int, _p, _sz, _p]),
    "ssb_shard_reduce_fwd_f32": (_int, [_p, _p, _p, _i64, _i64, _p, _sz, _p]),
    "ssb_shard_reduce_bwd_f32": (_int, [_p, _p, _p, _i64, _i64, _p, _sz, _p]),
    "ssb_shard_reduce_workspace_bytes": (_sz, [_i64, _i64]),
    "ssb_shard_carry_f32": (_int, [_p, _int, _int, _int, _i64, _p, _p]),
    "ssb_shard_map_fwd_f32": (_int, [_p, _p, _p, _i64, _i64, ctypes.c_float, _p, _p]),
    "ssb_shard_map_bwd_f32": (_int, [_p, _p, _p, _i64, _i64, ctypes.c_float, _p, _p]),
    "ssb_peer_exchange_bytes": (_sz, [_int, _i64]),
    "ssb_peer_buffer_create": (_int, [_sz, ctypes.POINTER(_p), ctypes.c_char_p]),
    "ssb_peer_buffer_open": (_int, [ctypes.c_char_p, ctypes.POINTER(_p)]),
    "ssb_peer_buffer_close": (_int, [_p]),
    "ssb_peer_buffer_destroy": (_int, [_p]),
    "ssb_shard_map_publish_f32": (_int, [_p, _p, _i64, _i64, ctypes.c_float, _int, _p, ctypes.c_uint, _p, _p]),
    "ssb_shard_carry_peer_f32": (_int, [_p, ctypes.c_uint, _int, _p, _p]),
    "ssb_selftest_wait_timeout": (_int, [_p, _sz, _p]),
    "ssb_checked_build": (_int, []),
    "ssb_selftest_index_check": (_int, [_p]),
    "ssb_device_status": (_int, [ctypes.POINTER(_int)]),
}

class PeerExchangeStruct(ctypes.Structure):
    """``ssb_peer_exchange_t``."""

    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("rows", ctypes.c_int64), ("buffers", ctypes.c_void_p * 8)]


_lib = None


def load() -> ctypes.CDLL:
    """Loads the library (raises ``OSError`` when it has not been built) and types every symbol."""
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class NativeError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"scanscam_b200 status {status}: {message}")
        self.status = status


def check(status: int) -> None:
    """Raises :class:`NativeError` for a non-zero status, with the library's message."""
    if status != OK:
        lib = load()
        raise NativeError(status, f"{lib.ssb_status_string(status).decode()}: {lib.ssb_last_error().decode()}")


def ptr(t) -> int | None:
    """Device pointer of a torch tensor (None passes through as NULL)."""
    return None if t is None else t.data_ptr()


def stream_of(t) -> int:
    """The raw handle of torch's current stream on the tensor's device."""
    import torch

    return torch.cuda.current_stream(t.device).cuda_stream
