"""Device codec context: the rotation / QJL / codebook tables of one setting,
uploaded once per (device, bits, mode, seed) and shared by every layer and head.

Mirrors the state ``PackedMSELayer.lazy_initialization`` builds in the reference
(``src/turboquant/runtime/packed_qmse_cache.py:226-283``): values use
``rotation(seed)`` and the ``bits`` codebook; Q_prod keys use ``rotation(seed+1)``,
the ``bits-1`` codebook and a Gaussian QJL matrix seeded with ``seed + 31337``.
"""

from __future__ import annotations

import ctypes as C
import threading

import numpy as np
import torch

from tq_local_b200.quantization.turboquant_mse import build_scalar_codebook, random_rotation_matrix
from tq_local_b200.runtime import ffi

QJL_SEED_OFFSET = 31337

_TORCH_TO_TQ = {torch.float32: ffi.TQ_DTYPE_F32, torch.float16: ffi.TQ_DTYPE_F16, torch.bfloat16: ffi.TQ_DTYPE_BF16}


def tq_dtype(dtype: torch.dtype) -> int:
    try:
        return _TORCH_TO_TQ[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}; expected float32, float16 or bfloat16") from None


def generate_qjl_matrix(dimension: int, seed: int) -> torch.Tensor:
    """Seeded Gaussian projection (packed_qmse_cache.py:143-145), CPU float32."""
    return torch.randn(dimension, dimension, generator=torch.Generator().manual_seed(seed), dtype=torch.float32)


def dense_desc(t: torch.Tensor) -> ffi.DenseDesc:
    """Describe a [B, H, T, 128] tensor (any outer strides, last axis contiguous)."""
    if t.dim() != 4 or t.shape[-1] != 128 or t.stride(-1) != 1:
        raise ValueError(f"expected [B, H, T, 128] with a contiguous last axis, got {tuple(t.shape)} / {t.stride()}")
    return ffi.DenseDesc(t.data_ptr(), tq_dtype(t.dtype), t.stride(0), t.stride(1), t.stride(2))


class Codec:
    """Owns one ``tq_ctx`` on one CUDA device."""

    _cache: dict[tuple, "Codec"] = {}
    _lock = threading.Lock()

    def __init__(self, device: torch.device, bits: int, use_qjl: bool, seed: int = 0, grid_size: int = 32769,
                 head_dim: int = 128, rot_v: np.ndarray | None = None, rot_k: np.ndarray | None = None):
        if head_dim != 128:
            raise NotImplementedError("the sm_100a kernels are specialised for head_dim == 128")
        if bits not in (2, 3, 4):
            raise NotImplementedError(f"bits={bits}: the packed kernels cover 2, 3 and 4 bits")
        if device.type != "cuda":
            raise ffi.TQError("TurboQuant-B200 runs on CUDA devices only; there is no CPU path")
        self.device = device
        self.bits = bits
        self.use_qjl = bool(use_qjl)
        self.key_bits = bits - 1 if use_qjl else bits
        self.seed = seed
        self.head_dim = head_dim

        val_cb = build_scalar_codebook(head_dim, bits, grid_size)
        self.rot_v = np.ascontiguousarray(rot_v if rot_v is not None else random_rotation_matrix(head_dim, seed),
                                          dtype=np.float32)
        self.cen_v = val_cb.centers.astype(np.float32)
        self.bnd_v = val_cb.boundaries.astype(np.float32)
        if use_qjl:
            key_cb = build_scalar_codebook(head_dim, bits - 1, grid_size)
            self.rot_k = np.ascontiguousarray(
                rot_k if rot_k is not None else random_rotation_matrix(head_dim, seed + 1), dtype=np.float32)
            self.cen_k = key_cb.centers.astype(np.float32)
            self.bnd_k = key_cb.boundaries.astype(np.float32)
            self.qjl = generate_qjl_matrix(head_dim, seed + QJL_SEED_OFFSET).numpy()
        else:
            self.rot_k, self.cen_k, self.bnd_k, self.qjl = self.rot_v, self.cen_v, self.bnd_v, None

        ptr = lambda a: a.ctypes.data_as(C.c_void_p) if a is not None else None
        desc = ffi.CodecDesc(head_dim, bits, int(self.use_qjl), ptr(self.rot_k), ptr(self.rot_v), ptr(self.qjl),
                             ptr(self.cen_k), ptr(self.bnd_k), ptr(self.cen_v), ptr(self.bnd_v))
        handle = C.c_void_p()
        index = device.index if device.index is not None else torch.cuda.current_device()
        with torch.cuda.device(index):
            ffi.check(ffi.lib().tq_ctx_create(C.byref(handle), index, C.byref(desc)), "tq_ctx_create")
        self.handle = handle
        self._torch_tables: dict[str, torch.Tensor] = {}

    def table(self, name: str) -> torch.Tensor:
        """Device copy of a host table (``rot_k``, ``rot_v``, ``qjl``, ``cen_k`` ...), for
        callers that want the reference's ``layer.rotation`` / ``layer.centers`` tensors."""
        if name not in self._torch_tables:
            self._torch_tables[name] = torch.from_numpy(np.asarray(getattr(self, name))).to(self.device)
        return self._torch_tables[name]

    @classmethod
    def get(cls, device: torch.device, bits: int, use_qjl: bool, seed: int = 0, grid_size: int = 32769,
            head_dim: int = 128) -> "Codec":
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        key = (str(device), bits, bool(use_qjl), seed, grid_size, head_dim)
        with cls._lock:
            if key not in cls._cache:
                cls._cache[key] = cls(device, bits, use_qjl, seed, grid_size, head_dim)
            return cls._cache[key]

    def profile(self, on: bool) -> None:
        """Switch the library's measurement hooks on or off (see ``tq_profile_enable``)."""
        ffi.check(ffi.lib().tq_profile_enable(self.handle, int(on)), "tq_profile_enable")

    def profile_read(self) -> tuple[float, int, int]:
        """(summed main-kernel ms, main-kernel launches, all launches) since the last read."""
        ms, n_main, n_all = C.c_double(), C.c_int64(), C.c_int64()
        ffi.check(ffi.lib().tq_profile_read(self.handle, C.byref(ms), C.byref(n_main), C.byref(n_all)),
                  "tq_profile_read")
        return ms.value, n_main.value, n_all.value

    def device_status(self) -> int:
        """0 unless a kernel's bounded wait ever ran out (synchronises with the device)."""
        v = C.c_int32()
        ffi.check(ffi.lib().tq_device_status(self.handle, C.byref(v)), "tq_device_status")
        return v.value

    _STATUS_TEXT = {
        1: "a decode kernel's wait for its bulk copies ran out",
        2: "a decode kernel's shared-memory layout did not fit and it did not run",
        3: "the encoder's wait ran out",
        4: "an append addressed a token past the cache's capacity and was dropped",
        5: "the wait for a peer's attention outputs ran out (tq_gather_wait)",
        6: "the bounds-checked build stopped a kernel from reading or writing outside a buffer",
    }

    def raise_on_device_status(self, where: str) -> None:
        """Raise :class:`TQError` when a kernel of this context has reported a problem.  The
        bounded waits only set the status word; results computed after that are not to be
        trusted, so the generation loops call this wherever they synchronise anyway."""
        status = self.device_status()
        if status:
            raise ffi.TQError(f"{where}: device status {status} ({self._STATUS_TEXT.get(status, 'unknown')}); "
                              "the outputs of this context are not valid")

    def set_wait_limit_ms(self, limit_ms: int) -> None:
        """How long ``tq_gather_wait`` polls for its peers before giving up (default 2000 ms)."""
        ffi.check(ffi.lib().tq_set_wait_limit_ms(self.handle, int(limit_ms)), "tq_set_wait_limit_ms")

    def close(self) -> None:
        if getattr(self, "handle", None):
            ffi.lib().tq_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):  # best effort; contexts are tiny and usually live for the process
        try:
            self.close()
        except Exception:
            pass
