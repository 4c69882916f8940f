"""Mask builders of the reference (tensorax/nn/attention/utils.py:4-21): dense
additive fp32 masks, 0 where a key is visible and -inf where it is not.

The dense forms are O(B*H*S^2) and only usable for short sequences; for long
ones pass ``causal=True`` / ``kv_lens=`` to
``functional.scaled_dot_product_attention_ex`` instead, which encodes the same
visibility rule without materialising the mask.
"""
from __future__ import annotations

import numpy as np

from ...tensor import Tensor


def create_causal_mask(seq_len: int, batch_size: int = 1, num_heads: int = 1,
                       device: str = "cpu") -> Tensor:
    """[batch, heads, seq, seq]; entry (i, j) is 0 if j <= i else -inf."""
    tri = np.where(np.tril(np.ones((seq_len, seq_len), dtype=bool)), 0.0, -np.inf).astype(np.float32)
    data = np.broadcast_to(tri, (batch_size, num_heads, seq_len, seq_len))
    return Tensor(np.ascontiguousarray(data), device=device)


def create_padding_mask(lengths: list, max_len: int, num_heads: int = 1, device: str = "cpu") -> Tensor:
    """[batch, heads, 1, max_len]; entry (b, ., 0, j) is 0 if j < lengths[b] else -inf.

    As in the reference, this shape is only accepted by SDPA when seq_len_q == 1
    (csrc/tensor_ops.cpp:891-898 requires [B,H,Sq,Sk] exactly)."""
    lens = np.asarray(lengths, dtype=np.int64).reshape(-1, 1, 1, 1)
    cols = np.arange(max_len).reshape(1, 1, 1, -1)
    data = np.where(cols < lens, 0.0, -np.inf).astype(np.float32)
    data = np.broadcast_to(data, (len(lengths), num_heads, 1, max_len))
    return Tensor(np.ascontiguousarray(data), device=device)
