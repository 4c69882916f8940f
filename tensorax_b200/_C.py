"""Python-level mirror of the reference's pybind11 module ``tensorax._C`` for the
SDPA forward path (tensorax csrc/tensor_ops.cpp:1513-1641), implemented over the
C ABI in ``include/tensorax_b200.h``.

Same function names, argument names, defaults, result shapes/dtypes and error
types (``RuntimeError`` with the reference's messages) as the reference's
dispatchers (csrc/tensor_ops.cpp:830-1181).  What is different, on purpose:

* CUDA only.  Host ("cpu") tensors exist for ingress/egress, but every SDPA call
  on them raises: this package ships no CPU compute path.
* Additive relaxations the reference lacks: fp16 inputs on the generic entry
  points (output float32), K/V with fewer heads than Q (grouped heads, mapped
  in-kernel), ``scaled_dot_product_attention_ex`` with implicit causal /
  key-length masks, and numpy buffer ingress/egress (``from_numpy``/``to_numpy``).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np

from . import _lib

_NP = {"float32": np.float32, "float16": np.float16, "half": np.float16}


class TensorImpl:
    """Mirror of ``tensorax::TensorImpl`` (csrc/tensor_ops.h:14-30): read-only
    ``shape``, ``size``, ``dtype``, ``device``; owns its buffer."""

    __slots__ = ("_shape", "_size", "_dtype", "_device", "_buf", "_host")

    def __init__(self, shape: Sequence[int], dtype: str, device: str, host=None, buf=None):
        if dtype not in _NP:
            raise RuntimeError(f"tensorax_b200 tensors hold float32 or float16, not {dtype!r}")
        if device not in ("cpu", "cuda"):
            raise RuntimeError(f"Unknown device: {device}")
        self._shape = [int(s) for s in shape]
        self._size = int(np.prod(self._shape, dtype=np.int64)) if len(self._shape) else 1
        self._dtype = dtype
        self._device = device
        self._host = host
        self._buf = buf
        if device == "cuda" and buf is None:
            self._buf = _lib.DeviceBuffer(max(self._size * self.itemsize, 1))
        if device == "cpu" and host is None:
            self._host = np.zeros(self._size, dtype=_NP[dtype])

    shape = property(lambda self: list(self._shape))
    size = property(lambda self: self._size)
    dtype = property(lambda self: self._dtype)
    device = property(lambda self: self._device)

    @property
    def itemsize(self) -> int:
        return 2 if self._dtype in ("float16", "half") else 4

    @property
    def data_ptr(self) -> int:
        if self._device != "cuda":
            raise RuntimeError("data_ptr: host tensor")
        return self._buf.ptr


# ------------------------------------------------------------------ creation / movement
def cuda_is_available() -> bool:
    return _lib.cuda_is_available()


def from_numpy(array, device: str = "cuda", dtype: Optional[str] = None) -> TensorImpl:
    """Buffer ingress (no Python lists): numpy fp32/fp16 array -> tensor."""
    a = np.asarray(array)
    if dtype is None:
        dtype = "float16" if a.dtype == np.float16 else "float32"
    a = np.ascontiguousarray(a, dtype=_NP[dtype])
    if device == "cpu":
        return TensorImpl(a.shape, dtype, "cpu", host=a.reshape(-1).copy())
    t = TensorImpl(a.shape, dtype, "cuda")
    if a.size:
        t._buf.upload(a)
    return t


def to_numpy(t: TensorImpl):
    """Buffer egress: tensor -> numpy array of the tensor's own dtype and shape."""
    if t.device == "cpu":
        return t._host.reshape(t._shape).copy()
    return t._buf.download(tuple(t._shape), _NP[t.dtype])


def create_tensor_cpu(data: List[float], shape: List[int], dtype: str) -> TensorImpl:
    return from_numpy(np.asarray(data, dtype=np.float32).reshape(shape), "cpu", dtype)


def create_tensor_cuda(data: List[float], shape: List[int], dtype: str) -> TensorImpl:
    return from_numpy(np.asarray(data, dtype=np.float32).reshape(shape), "cuda", dtype)


def tensor_cpu_to_cuda(t: TensorImpl) -> TensorImpl:
    return from_numpy(t._host.reshape(t._shape), "cuda", t.dtype)


def tensor_cuda_to_cpu(t: TensorImpl) -> TensorImpl:
    return from_numpy(to_numpy(t), "cpu", t.dtype)


def tensor_to_list(t: TensorImpl) -> List[float]:
    return to_numpy(t).astype(np.float64).reshape(-1).tolist()


def copy_tensor(t: TensorImpl) -> TensorImpl:
    if t.device == "cpu":
        return TensorImpl(t._shape, t.dtype, "cpu", host=t._host.copy())
    out = TensorImpl(t._shape, t.dtype, "cuda")
    _lib.check(_lib.load().tx_cuda_memcpy_d2d(out.data_ptr, t.data_ptr, t.size * t.itemsize))
    return out


def reshape(t: TensorImpl, shape: List[int]) -> TensorImpl:
    if int(np.prod(shape, dtype=np.int64)) != t.size:
        raise RuntimeError("reshape: size mismatch")
    out = copy_tensor(t)
    out._shape = [int(s) for s in shape]
    return out


def repeat_interleave(x: TensorImpl, repeats: int, dim: int) -> TensorImpl:
    """csrc/tensor_ops.cpp:121-162: out index j*repeats+r along ``dim`` <- in index j."""
    ndim = len(x._shape)
    if dim < 0:
        dim += ndim
    if dim < 0 or dim >= ndim:
        raise RuntimeError("Dimension out of range")
    out_shape = list(x._shape)
    out_shape[dim] *= int(repeats)
    if x.device == "cpu":
        arr = np.repeat(x._host.reshape(x._shape), int(repeats), axis=dim)
        return TensorImpl(out_shape, x.dtype, "cpu", host=np.ascontiguousarray(arr).reshape(-1))
    inner = int(np.prod(x._shape[dim + 1:], dtype=np.int64)) if dim + 1 < ndim else 1
    dim_size = x._shape[dim]
    outer = x.size // (dim_size * inner)
    out = TensorImpl(out_shape, x.dtype, "cuda")
    lib = _lib.load()
    _lib.check(lib.tx_repeat_interleave_cuda(x.data_ptr, out.data_ptr, outer, dim_size, inner,
                                             int(repeats), x.itemsize))
    _lib.check(lib.tx_cuda_synchronize())
    return out


def cast_to_fp16(src: TensorImpl) -> TensorImpl:
    """csrc/tensor_ops.cpp:1033-1045."""
    if src.dtype == "float16":
        return src
    if src.device != "cuda":
        raise RuntimeError("cast_to_fp16: only CUDA tensors supported")
    dst = TensorImpl(src._shape, "float16", "cuda")
    _lib.check(_lib.load().tx_cast_f32_to_f16_cuda(src.data_ptr, dst.data_ptr, src.size))
    return dst


def linear(x: TensorImpl, weight: TensorImpl, bias: Optional[TensorImpl] = None, heads_in: int = 0,
           heads_out: int = 0) -> TensorImpl:
    """x @ weight.T + bias on CUDA, exact fp32 (reference: F.linear -> matmul,
    tensorax/functional.py:105-110, csrc/tensor_ops.cpp:295-329).  No reference counterpart for
    `heads_in` / `heads_out`: they fold MultiHeadAttention's reshape + transpose(1, 2)
    (tensorax/nn/attention/layers.py:117-125) into the projection -- x read as
    [B, heads_in, S, K/heads_in], result written as [B, heads_out, S, N/heads_out]."""
    if x.device != "cuda" or weight.device != "cuda" or (bias is not None and bias.device != "cuda"):
        raise RuntimeError("linear: tensorax_b200 implements the CUDA path only")
    if x.dtype != "float32" or weight.dtype != "float32":
        raise RuntimeError("linear: float32 tensors expected")
    if len(weight._shape) != 2:
        raise RuntimeError("linear: weight must be [out_features, in_features]")
    N, K = weight._shape
    if heads_in:
        if len(x._shape) != 4 or x._shape[1] != heads_in or x._shape[1] * x._shape[3] != K:
            raise RuntimeError("linear: head-split input must be [B, heads, S, in_features/heads]")
        B, S = x._shape[0], x._shape[2]
    else:
        if x._shape[-1] != K or len(x._shape) not in (2, 3):
            raise RuntimeError("linear: input must be [S, in_features] or [B, S, in_features]")
        B, S = (1, x._shape[0]) if len(x._shape) == 2 else (x._shape[0], x._shape[1])
    if bias is not None and list(bias._shape) != [N]:
        raise RuntimeError("linear: bias must be [out_features]")
    if heads_out:
        if N % heads_out:
            raise RuntimeError("linear: out_features must be a multiple of heads_out")
        out_shape = [B, heads_out, S, N // heads_out]
    else:
        out_shape = [S, N] if (len(x._shape) == 2 and not heads_in) else [B, S, N]
    out = TensorImpl(out_shape, "float32", "cuda")
    lib = _lib.load()
    _lib.check(lib.tx_linear_f32_cuda(x.data_ptr, weight.data_ptr, bias.data_ptr if bias is not None else None,
                                      out.data_ptr, B, S, K, N, int(heads_in), int(heads_out)))
    _lib.check(lib.tx_sdpa_finish(None))      # waits, and reports a kernel-side failure if there was one
    return out


# ------------------------------------------------------------------ SDPA dispatchers
def _validate(query, key, value, mask, who="SDPA"):
    """Validation order and messages of csrc/tensor_ops.cpp:855-898."""
    if len(query._shape) != 4 or len(key._shape) != 4 or len(value._shape) != 4:
        raise RuntimeError(f"{who}: Query, Key, Value must be 4D tensors [batch, num_heads, seq_len, d]")
    if query.device != key.device or query.device != value.device:
        raise RuntimeError(f"{who}: All tensors must be on the same device")
    if mask is not None and mask.device != query.device:
        raise RuntimeError(f"{who}: Mask must be on the same device as Q, K, V")
    B, H, Sq, dk = query._shape
    Sk, dv = key._shape[2], value._shape[3]
    Hkv = key._shape[1]
    # reference: key heads == query heads; relaxed to "divides" for grouped K/V heads
    if key._shape[0] != B or Hkv <= 0 or H % Hkv != 0 or key._shape[3] != dk:
        raise RuntimeError(f"{who}: Key dimensions don't match Query")
    if value._shape[0] != B or value._shape[1] != Hkv or value._shape[2] != Sk:
        raise RuntimeError(f"{who}: Value dimensions don't match Key")
    if mask is not None and list(mask._shape) != [B, H, Sq, Sk]:
        raise RuntimeError(f"{who}: Mask shape must be [batch, num_heads, seq_len_q, seq_len_k]")
    return B, H, Hkv, Sq, Sk, dk, dv


def synchronize() -> None:
    """Wait for everything enqueued with ``sync=False`` and raise if a kernel reported a failure."""
    _lib.check(_lib.load().tx_sdpa_finish(None))


def _forward(query, key, value, mask, causal=False, kv_lens=None, flags=0, who="SDPA", out_dtype="float32",
             want_lse=False, sync=True):
    B, H, Hkv, Sq, Sk, dk, dv = _validate(query, key, value, mask, who)
    if query.device != "cuda":
        raise RuntimeError(
            f"{who}: tensorax_b200 implements the CUDA path only; move Q, K, V to 'cuda' "
            "(there is no CPU compute path and no CPU fallback)")
    if not (query.dtype == key.dtype == value.dtype):
        raise RuntimeError(f"{who}: Query, Key, Value must share one dtype")
    if mask is not None and mask.dtype != "float32":
        raise RuntimeError(f"{who}: Mask must be float32")
    f16 = query.dtype in ("float16", "half")
    # reference: output dtype string = query dtype for the generic entries; fp16 inputs give
    # float32 output exactly as scaled_dot_product_attention_mma_fp16 does
    if out_dtype not in ("float32", "float16"):
        raise RuntimeError(f"{who}: out_dtype must be 'float32' or 'float16'")
    out = TensorImpl([B, H, Sq, dv], out_dtype, "cuda")
    if out_dtype == "float16":
        flags = int(flags) | _lib.TX_SDPA_OUT_F16
    lse = TensorImpl([B, H, Sq], "float32", "cuda") if want_lse else None
    lens_buf = None
    if kv_lens is not None:
        lens = np.ascontiguousarray(kv_lens, dtype=np.int32)
        if lens.shape != (B,):
            raise RuntimeError(f"{who}: kv_lens must hold one length per batch element")
        lens_buf = _lib.to_device(lens)
    desc = _lib.SdpaDesc(
        q=query.data_ptr, k=key.data_ptr, v=value.data_ptr,
        mask=mask.data_ptr if mask is not None else None,
        kv_lens=lens_buf.ptr if lens_buf is not None else None, out=out.data_ptr,
        batch=B, q_heads=H, kv_heads=Hkv, seq_q=Sq, seq_k=Sk, d_k=dk, d_v=dv,
        dtype=_lib.TX_DTYPE_F16 if f16 else _lib.TX_DTYPE_F32, causal=int(bool(causal)),
        flags=int(flags), stream=None, lse=lse.data_ptr if lse is not None else None)
    lib = _lib.load()
    _lib.check(lib.tx_sdpa_forward(ctypes.byref(desc)))
    if sync:
        _lib.check(lib.tx_sdpa_finish(None))   # the reference launchers return a finished result
    # sync=False: the launch is stream-ordered; buffers freed meanwhile (the key lengths above) go back to
    # the pool in stream order, so nothing is reused before the kernel has read it
    return (out, lse) if want_lse else out


def sdpa_backward_supported(query, key, value, mask) -> bool:
    """Shapes the backward kernels take: float16 CUDA tensors, d_k == d_v in {64, 128, 256}, no dense mask."""
    return (mask is None and query.device == "cuda" and query.dtype in ("float16", "half")
            and key.dtype == query.dtype and value.dtype == query.dtype
            and query._shape[3] == value._shape[3] and query._shape[3] in (64, 128, 256))


def scaled_dot_product_attention_backward(query, key, value, out, lse, grad, causal=False, kv_lens=None):
    """Gradients (dq, dk, dv), float32, of ``out = SDPA(query, key, value)`` for the upstream
    gradient ``grad`` -- the reference's autograd rule, tensorax/tensor.py:806-827, which there
    runs through dense [Sq,Sk] temporaries (and cannot run at all: Tensor.transpose rejects the
    negative dims it is called with, tensorax/tensor.py:963-964).  ``lse`` is the row statistic
    the forward returned with ``want_lse``."""
    B, H, Hkv, Sq, Sk, dk, dv = _validate(query, key, value, None, "SDPA backward")
    if not sdpa_backward_supported(query, key, value, None):
        raise RuntimeError("SDPA backward: built for float16 CUDA tensors with d_k == d_v in {64, 128, 256} and "
                           "implicit (causal / kv_lens) masks")
    if list(grad._shape) != [B, H, Sq, dv] or grad.dtype != "float32" or grad.device != "cuda":
        raise RuntimeError("SDPA backward: grad must be a float32 CUDA tensor shaped like the output")
    if list(out._shape) != [B, H, Sq, dv] or list(lse._shape) != [B, H, Sq]:
        raise RuntimeError("SDPA backward: out / lse do not belong to these inputs")
    dq = TensorImpl([B, H, Sq, dk], "float32", "cuda")
    dkk = TensorImpl([B, Hkv, Sk, dk], "float32", "cuda")
    dvv = TensorImpl([B, Hkv, Sk, dv], "float32", "cuda")
    lens_buf = None
    if kv_lens is not None:
        lens = np.ascontiguousarray(kv_lens, dtype=np.int32)
        if lens.shape != (B,):
            raise RuntimeError("SDPA backward: kv_lens must hold one length per batch element")
        lens_buf = _lib.to_device(lens)
    desc = _lib.SdpaBwdDesc(
        q=query.data_ptr, k=key.data_ptr, v=value.data_ptr, out=out.data_ptr, dout=grad.data_ptr,
        lse=lse.data_ptr, kv_lens=lens_buf.ptr if lens_buf is not None else None,
        dq=dq.data_ptr, dk=dkk.data_ptr, dv=dvv.data_ptr, batch=B, q_heads=H, kv_heads=Hkv, seq_q=Sq, seq_k=Sk,
        d=dk, causal=int(bool(causal)), flags=_lib.TX_SDPA_OUT_F16 if out.dtype == "float16" else 0, stream=None)
    lib = _lib.load()
    _lib.check(lib.tx_sdpa_backward(ctypes.byref(desc)))
    _lib.check(lib.tx_sdpa_finish(None))
    return dq, dkk, dvv


def scaled_dot_product_attention(query, key, value, mask=None) -> TensorImpl:
    """csrc/tensor_ops.cpp:830-933."""
    return _forward(query, key, value, mask)


def scaled_dot_product_attention_tiled(query, key, value, mask=None) -> TensorImpl:
    """csrc/tensor_ops.cpp:935-982."""
    return _forward(query, key, value, mask)


def scaled_dot_product_attention_flash(query, key, value, mask=None) -> TensorImpl:
    """csrc/tensor_ops.cpp:1085-1132."""
    return _forward(query, key, value, mask)


def scaled_dot_product_attention_flash_optimized(query, key, value, mask=None) -> TensorImpl:
    """csrc/tensor_ops.cpp:1134-1181."""
    return _forward(query, key, value, mask)


def scaled_dot_product_attention_mma(query, key, value, mask=None) -> TensorImpl:
    """csrc/tensor_ops.cpp:984-1031."""
    return _forward(query, key, value, mask)


def scaled_dot_product_attention_mma_fp16(query, key, value) -> TensorImpl:
    """csrc/tensor_ops.cpp:1047-1083: fp16 CUDA inputs, float32 output, no mask."""
    if len(query._shape) != 4 or len(key._shape) != 4 or len(value._shape) != 4:
        raise RuntimeError("SDPA fp16: Q, K, V must be 4D tensors")
    if query.device != "cuda" or key.device != "cuda" or value.device != "cuda":
        raise RuntimeError("SDPA fp16: all tensors must be on CUDA")
    if query.dtype != "float16" or key.dtype != "float16" or value.dtype != "float16":
        raise RuntimeError("SDPA fp16: all inputs must have dtype float16")
    return _forward(query, key, value, None, who="SDPA fp16")


def profile_sections_sdpa(query, key, value, causal=False) -> List[int]:
    """Section profile of the fp16 tensor-core kernels, the counterpart for that path of the reference's
    ``profile_sections_sdpa_*`` bindings (csrc/tensor_ops.cpp:1434-1507, 1622-1636): runs the call once on the
    instrumented kernel of its shape (fp16, d in {64, 128, 256, 512}) and returns 64 cycle counters of one CTA;
    the meaning of each slot is listed beside ``tx_profile_sections_sdpa`` in the C header."""
    B, H, Hkv, Sq, Sk, dk, dv = _validate(query, key, value, None, "profile_sections")
    if query.device != "cuda" or query.dtype != "float16":
        raise RuntimeError("profile_sections: float16 CUDA tensors expected")
    out = TensorImpl([B, H, Sq, dv], "float32", "cuda")
    desc = _lib.SdpaDesc(q=query.data_ptr, k=key.data_ptr, v=value.data_ptr, mask=None, kv_lens=None,
                         out=out.data_ptr, batch=B, q_heads=H, kv_heads=Hkv, seq_q=Sq, seq_k=Sk, d_k=dk,
                         d_v=dv, dtype=_lib.TX_DTYPE_F16, causal=int(bool(causal)), flags=0, stream=None)
    ticks = (ctypes.c_longlong * 64)()
    _lib.check(_lib.load().tx_profile_sections_sdpa(ctypes.byref(desc), ticks))
    return list(ticks)


def _profile_sections_f32(name, query, key, value, mask=None) -> List[int]:
    """The reference's ``profile_sections_sdpa_{naive,tiled,flash,mma,flash_optimized}`` (csrc/tensor_ops.cpp:1434-1507):
    float32 CUDA tensors, 32 clock64 stamps of one instrumented launch of the exact-fp32 kernel."""
    B, H, Hkv, Sq, Sk, dk, dv = _validate(query, key, value, mask, "profile_sections")
    if query.device != "cuda":
        raise RuntimeError("profile_sections requires CUDA tensors")
    if query.dtype != "float32" or Hkv != H:
        raise RuntimeError("profile_sections: float32 tensors with equal head counts expected")
    out = TensorImpl([B, H, Sq, dv], "float32", "cuda")
    ticks = (ctypes.c_longlong * 32)()
    fn = getattr(_lib.load(), f"tx_sdpa_{name}_profile_sections_cuda")
    _lib.check(fn(query.data_ptr, key.data_ptr, value.data_ptr, mask.data_ptr if mask is not None else None,
                  out.data_ptr, B, H, Sq, Sk, dk, dv, ticks))
    return list(ticks)


def profile_sections_sdpa_naive(q, k, v, mask=None) -> List[int]:
    return _profile_sections_f32("naive", q, k, v, mask)


def profile_sections_sdpa_tiled(q, k, v, mask=None) -> List[int]:
    return _profile_sections_f32("tiled", q, k, v, mask)


def profile_sections_sdpa_flash(q, k, v, mask=None) -> List[int]:
    return _profile_sections_f32("flash", q, k, v, mask)


def profile_sections_sdpa_mma(q, k, v, mask=None) -> List[int]:
    return _profile_sections_f32("mma", q, k, v, mask)


def profile_sections_sdpa_flash_optimized(q, k, v, mask=None) -> List[int]:
    return _profile_sections_f32("optimized_flash", q, k, v, mask)


def scaled_dot_product_attention_ex(query, key, value, mask=None, causal=False, kv_lens=None,
                                    flags=0, out_dtype="float32", want_lse=False, sync=True, fp16_compute=False):
    """No reference counterpart: implicit masks for sizes where the dense
    [B,H,Sq,Sk] mask cannot exist.  ``causal``: key j visible to query i iff
    j <= i; ``kv_lens``: per-batch count of valid keys; ``out_dtype``: 'float32'
    (what every reference entry returns) or 'float16' (half the result bytes); ``sync=False``: return
    right after the launch (the reference's launchers end in cudaDeviceSynchronize, csrc/cuda/kernels/attn.cu:1519-1520);
    call ``synchronize()`` before reading the result on the host -- device-side consumers need nothing;
    ``fp16_compute=True``: float32 inputs are rounded to fp16 on the device and run on the tensor cores
    (what the reference's ``_mma`` variant does inside its kernel, csrc/cuda/kernels/attn.cu:441-603)."""
    if fp16_compute:
        flags = int(flags) | _lib.TX_SDPA_F32_VIA_F16
    return _forward(query, key, value, mask, causal=causal, kv_lens=kv_lens, flags=flags, out_dtype=out_dtype,
                    want_lse=want_lse, sync=sync)
