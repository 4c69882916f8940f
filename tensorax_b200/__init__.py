"""tensorax_b200 -- the scaled-dot-product-attention forward path of tensorax,
rebuilt for NVIDIA B200 (sm_100a) behind the reference's own names.

    import tensorax_b200 as ts
    import tensorax_b200.functional as F
    q = ts.Tensor(q_np, device="cuda"); ...
    out = F.scaled_dot_product_attention_mma_fp16(F.cast_to_fp16(q), F.cast_to_fp16(k), F.cast_to_fp16(v))

The compute lives in ``csrc/libtensorax_b200.so`` (C ABI: ``include/tensorax_b200.h``).
There is no CPU path and no fallback: without the built library, or without a
CUDA device, compute calls raise.
"""
from . import functional, nn  # noqa: F401
from ._C import synchronize
from ._lib import cuda_is_available
from .tensor import Tensor

__version__ = "0.1.0"
cpu = "cpu"
cuda = "cuda"

__all__ = ["Tensor", "functional", "nn", "cuda_is_available", "synchronize", "cpu", "cuda"]
