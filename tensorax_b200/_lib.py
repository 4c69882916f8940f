"""ctypes binding of the C-ABI library (``include/tensorax_b200.h``).

The shared object is built in-tree by ``tensorax_b200/build.py`` (nvcc, sm_100a).
There is no fallback of any kind: if the library is missing, or if it loads on a
machine without a CUDA device, every compute call raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int32, c_int64, c_size_t, c_void_p, c_char_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libtensorax_b200.so")

TX_OK = 0
TX_DTYPE_F32 = 0
TX_DTYPE_F16 = 1
TX_SDPA_FORCE_SIMT = 1
TX_SDPA_P_IN_SMEM = 2
TX_SDPA_OUT_F16 = 4
TX_SDPA_F32_VIA_F16 = 8

# every symbol include/tensorax_b200.h declares
EXPORTED_SYMBOLS = (
    "tx_last_error", "tx_version",
    "tx_cuda_is_available", "tx_cuda_device_count", "tx_cuda_set_device", "tx_cuda_malloc", "tx_cuda_free", "tx_cuda_free_on", "tx_cuda_pool_trim", "tx_cuda_memcpy_h2d",
    "tx_cuda_memcpy_d2h", "tx_cuda_memcpy_d2d", "tx_cuda_synchronize",
    "tx_host_alloc_pinned", "tx_host_free_pinned",
    "tx_sdpa_naive_cuda", "tx_sdpa_tiled_cuda", "tx_sdpa_flash_cuda",
    "tx_sdpa_optimized_flash_cuda", "tx_sdpa_mma_cuda", "tx_sdpa_mma_fp16_cuda",
    "tx_cast_f32_to_f16_cuda", "tx_repeat_interleave_cuda", "tx_linear_f32_cuda", "tx_linear_set_cuda_cores_only",
    "tx_sdpa_forward", "tx_sdpa_finish", "tx_sdpa_uses_tensor_cores",
    "tx_kernel_launch_count", "tx_profile_sections_sdpa", "tx_sdpa_forward_host", "tx_sdpa_fp16_static_scratch",
    "tx_sdpa_backward",
    "tx_sdpa_naive_profile_sections_cuda", "tx_sdpa_tiled_profile_sections_cuda", "tx_sdpa_flash_profile_sections_cuda",
    "tx_sdpa_mma_profile_sections_cuda", "tx_sdpa_optimized_flash_profile_sections_cuda",
    "tx_selftest_wait_timeout", "tx_sdpa_forward_host_copies_only", "tx_sdpa_set_group_l2_bytes",
)


class SdpaDesc(ctypes.Structure):
    """Mirror of ``tx_sdpa_desc``."""
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p),
        ("mask", c_void_p), ("kv_lens", c_void_p), ("out", c_void_p),
        ("batch", c_int64), ("q_heads", c_int64), ("kv_heads", c_int64),
        ("seq_q", c_int64), ("seq_k", c_int64), ("d_k", c_int64), ("d_v", c_int64),
        ("dtype", c_int32), ("causal", c_int32), ("flags", c_int32), ("reserved", c_int32),
        ("stream", c_void_p), ("lse", c_void_p),
    ]


class SdpaBwdDesc(ctypes.Structure):
    """Mirror of ``tx_sdpa_bwd_desc``."""
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("out", c_void_p), ("dout", c_void_p),
        ("lse", c_void_p), ("kv_lens", c_void_p), ("dq", c_void_p), ("dk", c_void_p), ("dv", c_void_p),
        ("batch", c_int64), ("q_heads", c_int64), ("kv_heads", c_int64),
        ("seq_q", c_int64), ("seq_k", c_int64), ("d", c_int64),
        ("causal", c_int32), ("flags", c_int32), ("stream", c_void_p),
    ]


class BackendError(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference raises RuntimeError
    from its dispatchers, csrc/tensor_ops.cpp:855-898)."""


_lib = None


def load():
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.isfile(LIB_PATH):
        raise RuntimeError(
            f"C++ backend not available. Please build the package first "
            f"(python -m tensorax_b200.build); expected {LIB_PATH}")
    lib = ctypes.CDLL(LIB_PATH)
    lib.tx_last_error.restype = c_char_p
    lib.tx_last_error.argtypes = []
    lib.tx_version.restype = c_int
    lib.tx_cuda_is_available.restype = c_int
    lib.tx_cuda_set_device.argtypes = [c_int]
    lib.tx_cuda_malloc.restype = c_void_p
    lib.tx_cuda_malloc.argtypes = [c_size_t]
    lib.tx_cuda_free.argtypes = [c_void_p]
    lib.tx_cuda_free_on.argtypes = [c_void_p, c_void_p]
    for name in ("tx_cuda_memcpy_h2d", "tx_cuda_memcpy_d2h", "tx_cuda_memcpy_d2d"):
        getattr(lib, name).argtypes = [c_void_p, c_void_p, c_size_t]
    lib.tx_host_alloc_pinned.restype = c_void_p
    lib.tx_host_alloc_pinned.argtypes = [c_size_t]
    lib.tx_host_free_pinned.argtypes = [c_void_p]
    f32_sig = [c_void_p] * 5 + [c_int64] * 6
    for name in ("tx_sdpa_naive_cuda", "tx_sdpa_tiled_cuda", "tx_sdpa_flash_cuda",
                 "tx_sdpa_optimized_flash_cuda", "tx_sdpa_mma_cuda"):
        getattr(lib, name).argtypes = f32_sig
    for name in ("naive", "tiled", "flash", "mma", "optimized_flash"):
        getattr(lib, f"tx_sdpa_{name}_profile_sections_cuda").argtypes = f32_sig + [ctypes.POINTER(ctypes.c_longlong)]
    lib.tx_sdpa_mma_fp16_cuda.argtypes = [c_void_p] * 4 + [c_int64] * 6
    lib.tx_cast_f32_to_f16_cuda.argtypes = [c_void_p, c_void_p, c_int64]
    lib.tx_repeat_interleave_cuda.argtypes = [c_void_p, c_void_p] + [c_int64] * 4 + [c_int32]
    lib.tx_linear_f32_cuda.argtypes = [c_void_p] * 4 + [c_int64] * 4 + [c_int32] * 2
    lib.tx_linear_set_cuda_cores_only.argtypes = [c_int]
    lib.tx_sdpa_set_group_l2_bytes.argtypes = [c_int64]
    lib.tx_sdpa_forward.argtypes = [ctypes.POINTER(SdpaDesc)]
    lib.tx_profile_sections_sdpa.argtypes = [ctypes.POINTER(SdpaDesc), ctypes.POINTER(ctypes.c_longlong)]
    lib.tx_selftest_wait_timeout.argtypes = [ctypes.POINTER(SdpaDesc), c_int32]
    lib.tx_sdpa_forward_host.argtypes = [ctypes.POINTER(SdpaDesc)]
    lib.tx_sdpa_forward_host_copies_only.argtypes = [ctypes.POINTER(SdpaDesc)]
    lib.tx_sdpa_backward.argtypes = [ctypes.POINTER(SdpaBwdDesc)]
    lib.tx_sdpa_uses_tensor_cores.argtypes = [ctypes.POINTER(SdpaDesc)]
    lib.tx_sdpa_finish.argtypes = [c_void_p]
    lib.tx_sdpa_fp16_static_scratch.argtypes = [c_void_p] * 4 + [c_int64] * 6 + [c_int32, c_void_p, c_void_p]
    lib.tx_kernel_launch_count.restype = c_int64
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != TX_OK:
        msg = load().tx_last_error().decode("utf-8", "replace")
        raise BackendError(msg or f"tensorax_b200 backend error {rc}")


def cuda_is_available() -> bool:
    return bool(load().tx_cuda_is_available())


class DeviceBuffer:
    """Owning handle of one cudaMalloc'ed buffer (freed with the object), the
    ownership rule of the reference's TensorImpl (csrc/tensor_ops.cpp:64-76)."""

    def __init__(self, nbytes: int):
        lib = load()
        if not lib.tx_cuda_is_available():
            raise BackendError("CUDA device not available: tensorax_b200 has no CPU fallback")
        self.nbytes = int(nbytes)
        self.ptr = lib.tx_cuda_malloc(self.nbytes)
        if not self.ptr:
            check(3)

    def __del__(self):
        ptr, self.ptr = getattr(self, "ptr", None), None
        if ptr and _lib is not None:
            _lib.tx_cuda_free(ptr)

    def upload(self, array) -> None:
        import numpy as np
        a = np.ascontiguousarray(array)
        assert a.nbytes <= self.nbytes
        check(load().tx_cuda_memcpy_h2d(self.ptr, a.ctypes.data_as(c_void_p), a.nbytes))

    def download(self, shape, dtype):
        import numpy as np
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= self.nbytes
        check(load().tx_cuda_memcpy_d2h(out.ctypes.data_as(c_void_p), self.ptr, out.nbytes))
        return out


def to_device(array) -> DeviceBuffer:
    import numpy as np
    a = np.ascontiguousarray(array)
    buf = DeviceBuffer(max(a.nbytes, 1))
    buf.upload(a)
    return buf
