"""ctypes binding of ``libtq_b200.so`` (the C ABI declared in ``include/tq_b200.h``).

There is no CPU or PyTorch fallback: if the library has not been built
(``python -m tq_local_b200.build``) importing a symbol raises, and every call
with a non-zero status raises :class:`TQError`.
"""

from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# TQ_B200_LIBRARY selects another build of the same library (the bounds-checked one, see build.py)
LIB_PATH = os.environ.get("TQ_B200_LIBRARY") or os.path.join(_PKG, "libtq_b200.so")

TQ_DTYPE_F32, TQ_DTYPE_F16, TQ_DTYPE_BF16 = 0, 1, 2
TQ_MAX_GROUPS = 8

EXPORTS = (
    "tq_abi_version", "tq_last_cuda_error", "tq_ctx_create", "tq_ctx_destroy", "tq_pack",
    "tq_decode_workspace_bytes", "tq_decode_suggest_splits", "tq_decode_attn", "tq_dequant",
    "tq_key_norm_sum", "tq_profile_enable", "tq_profile_read", "tq_device_status", "tq_static_scratch_bytes",
    "tq_decode_attn_static", "tq_decode_step_workspace_bytes", "tq_decode_step_host", "tq_decode_step_dev",
    "tq_peer_buffer_create", "tq_peer_buffer_open", "tq_peer_buffer_close", "tq_peer_buffer_destroy",
    "tq_decode_attn_gather", "tq_gather_wait", "tq_decode_step_host_gather", "tq_set_wait_limit_ms", "tq_decode_attn_f32out",
    "tq_parts_exchange_bytes", "tq_decode_attn_parts", "tq_decode_parts_finish",
)

_ERRORS = {-1: "bad argument", -2: "unsupported shape or mode", -3: "CUDA error", -4: "workspace too small"}


class TQError(RuntimeError):
    pass


class CodecDesc(C.Structure):
    _fields_ = [
        ("head_dim", C.c_int32), ("bits", C.c_int32), ("use_qjl", C.c_int32),
        ("rot_k", C.c_void_p), ("rot_v", C.c_void_p), ("qjl", C.c_void_p),
        ("centers_k", C.c_void_p), ("bounds_k", C.c_void_p),
        ("centers_v", C.c_void_p), ("bounds_v", C.c_void_p),
    ]


class CacheDesc(C.Structure):
    _fields_ = [
        ("k_codes", C.c_void_p), ("k_norms", C.c_void_p), ("k_signs", C.c_void_p),
        ("k_rnorms", C.c_void_p), ("v_codes", C.c_void_p), ("v_norms", C.c_void_p),
        ("batch", C.c_int32), ("kv_heads", C.c_int32), ("capacity", C.c_int32),
        ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("seq_start", C.c_void_p),
    ]


class DenseDesc(C.Structure):
    _fields_ = [
        ("data", C.c_void_p), ("dtype", C.c_int32),
        ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_t", C.c_int64),
    ]


TQ_MAX_PEERS = 8


class GatherDesc(C.Structure):
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32), ("q_heads_total", C.c_int32), ("seq", C.c_uint32),
        ("out", C.c_void_p * TQ_MAX_PEERS), ("out_stride", C.c_int64), ("flags", C.c_void_p * TQ_MAX_PEERS),
        ("counter", C.c_void_p), ("seq_dev", C.c_void_p), ("out_local_only", C.c_int32),
    ]


_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise TQError(
            f"{LIB_PATH} is missing: build the sm_100a library with `python -m tq_local_b200.build` "
            "(there is no fallback path)."
        )
    L = C.CDLL(LIB_PATH)
    L.tq_abi_version.restype = C.c_int32
    L.tq_last_cuda_error.restype = C.c_char_p
    L.tq_ctx_create.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.POINTER(CodecDesc)]
    L.tq_ctx_create.restype = C.c_int32
    L.tq_ctx_destroy.argtypes = [C.c_void_p]
    L.tq_ctx_destroy.restype = C.c_int32
    L.tq_pack.argtypes = [C.c_void_p, C.POINTER(DenseDesc), C.POINTER(DenseDesc), C.c_int32,
                          C.POINTER(CacheDesc), C.c_int32, C.c_void_p]
    L.tq_pack.restype = C.c_int32
    L.tq_decode_workspace_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32]
    L.tq_decode_workspace_bytes.restype = C.c_size_t
    L.tq_decode_suggest_splits.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32]
    L.tq_decode_suggest_splits.restype = C.c_int32
    L.tq_decode_attn.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.POINTER(CacheDesc), C.c_int32,
                                 C.POINTER(DenseDesc), C.POINTER(DenseDesc), C.c_int32, C.c_int32,
                                 C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    L.tq_decode_attn.restype = C.c_int32
    L.tq_dequant.argtypes = [C.c_void_p, C.POINTER(CacheDesc), C.c_int32, C.c_int32, C.c_int32,
                             C.POINTER(DenseDesc), C.c_void_p]
    L.tq_dequant.restype = C.c_int32
    L.tq_key_norm_sum.argtypes = [C.POINTER(DenseDesc), C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    L.tq_key_norm_sum.restype = C.c_int32
    L.tq_profile_enable.argtypes = [C.c_void_p, C.c_int32]
    L.tq_profile_enable.restype = C.c_int32
    L.tq_profile_read.argtypes = [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    L.tq_profile_read.restype = C.c_int32
    L.tq_device_status.argtypes = [C.c_void_p, C.POINTER(C.c_int32)]
    L.tq_device_status.restype = C.c_int32
    L.tq_static_scratch_bytes.restype = C.c_size_t
    L.tq_decode_attn_static.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.POINTER(CacheDesc), C.c_int32,
                                        C.c_int32, C.c_void_p, C.c_void_p]
    L.tq_decode_attn_static.restype = C.c_int32
    L.tq_decode_step_workspace_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32]
    L.tq_decode_step_workspace_bytes.restype = C.c_size_t
    L.tq_decode_step_host.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                      C.POINTER(CacheDesc), C.c_int32, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p,
                                      C.c_void_p]
    L.tq_decode_step_host.restype = C.c_int32
    L.tq_decode_step_dev.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                     C.POINTER(CacheDesc), C.c_void_p, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p,
                                     C.POINTER(GatherDesc), C.c_void_p]
    L.tq_decode_step_dev.restype = C.c_int32
    L.tq_peer_buffer_create.argtypes = [C.c_size_t, C.POINTER(C.c_void_p), C.c_void_p]
    L.tq_peer_buffer_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    L.tq_peer_buffer_close.argtypes = [C.c_void_p]
    L.tq_peer_buffer_destroy.argtypes = [C.c_void_p]
    L.tq_decode_attn_gather.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.POINTER(CacheDesc), C.c_int32,
                                        C.c_int32, C.c_void_p, C.c_size_t, C.POINTER(GatherDesc), C.c_void_p]
    L.tq_gather_wait.argtypes = [C.c_void_p, C.POINTER(GatherDesc), C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
    L.tq_decode_step_host_gather.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                             C.POINTER(CacheDesc), C.c_int32, C.c_int32, C.c_void_p, C.c_size_t,
                                             C.POINTER(GatherDesc), C.c_void_p, C.c_void_p]
    L.tq_decode_step_host_gather.restype = C.c_int32
    L.tq_decode_attn_f32out.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.POINTER(CacheDesc), C.c_int32,
                                        C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    L.tq_decode_attn_f32out.restype = C.c_int32
    L.tq_parts_exchange_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32]
    L.tq_parts_exchange_bytes.restype = C.c_size_t
    L.tq_decode_attn_parts.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.POINTER(CacheDesc), C.c_int32,
                                       C.c_int32, C.c_void_p, C.c_size_t, C.POINTER(GatherDesc), C.c_int32, C.c_void_p]
    L.tq_decode_attn_parts.restype = C.c_int32
    L.tq_decode_parts_finish.argtypes = [C.c_void_p, C.POINTER(GatherDesc), C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                         C.c_void_p, C.c_void_p]
    L.tq_decode_parts_finish.restype = C.c_int32
    L.tq_set_wait_limit_ms.argtypes = [C.c_void_p, C.c_int32]
    L.tq_set_wait_limit_ms.restype = C.c_int32
    for name in ("tq_peer_buffer_create", "tq_peer_buffer_open", "tq_peer_buffer_close", "tq_peer_buffer_destroy",
                 "tq_decode_attn_gather", "tq_gather_wait"):
        getattr(L, name).restype = C.c_int32
    _lib = L
    return L


def check(status: int, what: str) -> None:
    if status == 0:
        return
    msg = _ERRORS.get(status, f"status {status}")
    if status == -3:
        msg += ": " + (lib().tq_last_cuda_error() or b"").decode()
    raise TQError(f"{what} failed: {msg}")
