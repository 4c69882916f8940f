"""The SDPA section of the reference's functional API (tensorax/functional.py:243-407)
with the same names, argument names, checks and error types.

``ValueError`` is raised here for rank / device / dtype problems before the
backend is entered, ``RuntimeError`` comes from the backend, exactly as the
reference layers them (tests/test_attention.py:327-388 match on the messages).
"""
from __future__ import annotations

from typing import Optional, Sequence

from .tensor import Tensor

try:  # the backend is the in-tree CUDA library; nothing replaces it when it is missing
    from . import _C
    from ._lib import load as _load_backend
    _load_backend()
except Exception:  # pragma: no cover - exercised by the "backend missing" test through monkeypatching
    _C = None


def _result(c_tensor, requires_grad=False, grad_fn=None) -> Tensor:
    out = Tensor._wrap(c_tensor, requires_grad)
    out._grad_fn = grad_fn
    return out


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """Linear transformation x @ weight.T + bias (tensorax/functional.py:105-110), CUDA tensors."""
    if not _C:
        raise RuntimeError("C++ backend not available.")
    return _result(_C.linear(x._c_tensor, weight._c_tensor, bias._c_tensor if bias is not None else None))


def _check(query, key, value, mask, msg4d):
    if len(query.shape) != 4 or len(key.shape) != 4 or len(value.shape) != 4:
        raise ValueError(msg4d)
    if query.device != key.device or query.device != value.device:
        raise ValueError("All tensors must be on the same device")
    if mask is not None and mask.device != query.device:
        raise ValueError("Mask must be on the same device as Q, K, V")


_MSG4D = "Query, Key, and Value must be 4D tensors [batch, heads, seq_len, d]"


def scaled_dot_product_attention(query: Tensor, key: Tensor, value: Tensor,
                                 mask: Optional[Tensor] = None) -> Tensor:
    """Attention(Q, K, V) = softmax(Q K^T / sqrt(d_k) + mask) V  (tensorax/functional.py:243-321).

    query [B,H,Sq,d_k], key [B,Hkv,Sk,d_k], value [B,Hkv,Sk,d_v], optional additive
    mask [B,H,Sq,Sk] (-inf masks a position).  Returns [B,H,Sq,d_v].
    """
    _check(query, key, value, mask, _MSG4D)
    if not _C:
        raise RuntimeError("C++ backend not available. Please build the package first.")
    needs_grad = query.requires_grad or key.requires_grad or value.requires_grad
    mask_c = mask._c_tensor if mask is not None else None
    if needs_grad and _C.sdpa_backward_supported(query._c_tensor, key._c_tensor, value._c_tensor, mask_c):
        return _with_saved_stats(query, key, value, mask, False, None, "float32")
    c = _C.scaled_dot_product_attention(query._c_tensor, key._c_tensor, value._c_tensor, mask_c)
    if needs_grad:
        # same autograd tuple as the reference (tensorax/functional.py:314-316); backward() of this
        # result raises, because only the float16 tensor-core shapes have a backward kernel
        return _result(c, True, ("scaled_dot_product_attention", query, key, value, mask))
    return _result(c)


def _with_saved_stats(query, key, value, mask, causal, kv_lens, out_dtype) -> Tensor:
    """Forward that also keeps the per-row log-sum-exp, so that Tensor.backward can rebuild P."""
    c, lse = _C.scaled_dot_product_attention_ex(query._c_tensor, key._c_tensor, value._c_tensor, None,
                                                causal=causal, kv_lens=kv_lens, out_dtype=out_dtype, want_lse=True)
    out = _result(c, True, ("scaled_dot_product_attention", query, key, value, mask))
    out._saved = {"lse": lse, "causal": bool(causal), "kv_lens": None if kv_lens is None else list(kv_lens)}
    return out


def _sdpa_variant(query, key, value, mask, backend_name: str) -> Tensor:
    """tensorax/functional.py:324-351."""
    _check(query, key, value, mask, _MSG4D)
    if not _C:
        raise RuntimeError("C++ backend not available.")
    fn = getattr(_C, backend_name)
    return _result(fn(query._c_tensor, key._c_tensor, value._c_tensor,
                      mask._c_tensor if mask is not None else None))


def scaled_dot_product_attention_tiled(query, key, value, mask=None) -> Tensor:
    return _sdpa_variant(query, key, value, mask, "scaled_dot_product_attention_tiled")


def scaled_dot_product_attention_flash(query, key, value, mask=None) -> Tensor:
    return _sdpa_variant(query, key, value, mask, "scaled_dot_product_attention_flash")


def scaled_dot_product_attention_mma(query, key, value, mask=None) -> Tensor:
    return _sdpa_variant(query, key, value, mask, "scaled_dot_product_attention_mma")


def scaled_dot_product_attention_flash_optimized(query, key, value, mask=None) -> Tensor:
    return _sdpa_variant(query, key, value, mask, "scaled_dot_product_attention_flash_optimized")


def cast_to_fp16(tensor: Tensor) -> Tensor:
    """tensorax/functional.py:366-380."""
    if tensor.dtype == "float16":
        return tensor
    if tensor.device != "cuda":
        raise ValueError("cast_to_fp16: only CUDA tensors supported")
    if not _C:
        raise RuntimeError("C++ backend not available.")
    return _result(_C.cast_to_fp16(tensor._c_tensor))


def scaled_dot_product_attention_mma_fp16(query: Tensor, key: Tensor, value: Tensor) -> Tensor:
    """tensorax/functional.py:383-404: float16 CUDA inputs, float32 result, no mask."""
    if len(query.shape) != 4 or len(key.shape) != 4 or len(value.shape) != 4:
        raise ValueError("Q, K, V must be 4D tensors [batch, heads, seq_len, d]")
    if query.dtype != "float16" or key.dtype != "float16" or value.dtype != "float16":
        raise ValueError("scaled_dot_product_attention_mma_fp16: inputs must be float16 (use F.cast_to_fp16)")
    if not _C:
        raise RuntimeError("C++ backend not available.")
    return _result(_C.scaled_dot_product_attention_mma_fp16(query._c_tensor, key._c_tensor,
                                                           value._c_tensor))


def scaled_dot_product_attention_ex(query: Tensor, key: Tensor, value: Tensor,
                                    mask: Optional[Tensor] = None, causal: bool = False,
                                    kv_lens: Optional[Sequence[int]] = None,
                                    out_dtype: str = "float32", sync: bool = True,
                                    fp16_compute: bool = False) -> Tensor:
    """No reference counterpart.  Implicit masks for shapes where the reference's
    dense [B,H,Sq,Sk] masks cannot be built: ``causal`` (key j visible to query i
    iff j <= i, what create_causal_mask encodes) and ``kv_lens`` (per-batch valid
    key count, what create_padding_mask encodes).  K/V may have fewer heads than Q.
    ``out_dtype='float16'`` returns a float16 tensor (the reference's fp16 entry always
    returns float32, tensorax/functional.py:397).  ``sync=False`` returns right after the launch;
    ``tensorax_b200.synchronize()`` (or any download of the result) waits for it.
    ``fp16_compute=True``: float32 tensors are rounded to fp16 on the device and attended on the
    tensor cores (fp32 accumulation and result), as the reference's ``_mma`` variant does internally."""
    _check(query, key, value, mask, _MSG4D)
    if not _C:
        raise RuntimeError("C++ backend not available.")
    mask_c = mask._c_tensor if mask is not None else None
    needs_grad = query.requires_grad or key.requires_grad or value.requires_grad
    if needs_grad and _C.sdpa_backward_supported(query._c_tensor, key._c_tensor, value._c_tensor, mask_c):
        return _with_saved_stats(query, key, value, mask, causal, kv_lens, out_dtype)
    c = _C.scaled_dot_product_attention_ex(query._c_tensor, key._c_tensor, value._c_tensor, mask_c, causal=causal,
                                           kv_lens=kv_lens, out_dtype=out_dtype, sync=sync, fp16_compute=fp16_compute)
    if needs_grad:
        return _result(c, True, ("scaled_dot_product_attention", query, key, value, mask))
    return _result(c)
