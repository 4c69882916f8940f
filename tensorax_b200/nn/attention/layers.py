"""Attention layers with the reference's constructor arguments, ``forward``
signatures and ``repr`` strings (tensorax/nn/attention/layers.py:8-135)."""
from __future__ import annotations

import math

import numpy as np

from ... import functional as F
from ...tensor import Tensor


class ScaledDotProductAttention:
    """Pass-through to ``F.scaled_dot_product_attention`` (layers.py:8-17)."""

    def forward(self, query: Tensor, key: Tensor, value: Tensor, mask: Tensor = None) -> Tensor:
        return F.scaled_dot_product_attention(query, key, value, mask)

    def __call__(self, query: Tensor, key: Tensor, value: Tensor, mask: Tensor = None) -> Tensor:
        return self.forward(query, key, value, mask)

    def __repr__(self) -> str:
        return "ScaledDotProductAttention()"


class GroupedQueryAttention:
    """Grouped-query attention (layers.py:19-50).

    ``forward`` keeps the reference's behaviour to the letter: K and V are
    replicated ``num_heads // num_kv_heads`` times along dim 2 and the result is
    handed to SDPA unchanged, so dim 1 is what SDPA treats as the head axis.
    For the usual [batch, heads, seq, dim] layout with fewer K/V heads, use
    ``forward_bhsd``: no copy is made, query head h reads K/V head
    h // (num_heads // num_kv_heads) inside the kernel.
    """

    def __init__(self, num_heads: int, num_kv_heads: int):
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        assert num_heads % num_kv_heads == 0, "num_heads must be divisible by num_kv_heads"
        self.num_queries_per_kv = num_heads // num_kv_heads

    def forward(self, query: Tensor, key: Tensor, value: Tensor, mask: Tensor = None) -> Tensor:
        if self.num_queries_per_kv > 1:
            key = key.repeat_interleave(self.num_queries_per_kv, dim=2)
            value = value.repeat_interleave(self.num_queries_per_kv, dim=2)
        return F.scaled_dot_product_attention(query, key, value, mask)

    def forward_bhsd(self, query: Tensor, key: Tensor, value: Tensor, mask: Tensor = None,
                     causal: bool = False, kv_lens=None) -> Tensor:
        """query [B, num_heads, S, d]; key/value [B, num_kv_heads, S, d]."""
        if query.shape[1] != self.num_heads or key.shape[1] != self.num_kv_heads:
            raise ValueError("forward_bhsd: head counts do not match the layer")
        return F.scaled_dot_product_attention_ex(query, key, value, mask, causal=causal, kv_lens=kv_lens)

    def __call__(self, query: Tensor, key: Tensor, value: Tensor, mask: Tensor = None) -> Tensor:
        return self.forward(query, key, value, mask)

    def __repr__(self) -> str:
        return f"GroupedQueryAttention(num_heads={self.num_heads}, num_kv_heads={self.num_kv_heads})"


class MultiHeadAttention:
    """Multi-head attention (layers.py:53-135): same constructor, parameters,
    initialisation scale, ``forward`` signature and ``repr``.

    ``forward`` does what the reference's forward spells out -- three projections,
    split into heads, SDPA, merge, output projection (layers.py:112-128) -- on CUDA
    tensors.  The reference cannot run its own forward (it calls the unbound
    ``_C.transpose_dims``, tensorax/tensor.py:976); here the reshape + transpose
    steps are folded into the projections, which write and read the
    [batch, heads, seq, head_dim] layout directly.  ``dropout`` is stored and never
    applied, as in the reference.

    Additive (no reference counterpart): ``attention_dtype="float16"`` rounds the projected heads to
    fp16 and runs the attention step on the tensor-core kernel (fp32 accumulation, fp32 result; fp16
    tolerances instead of fp32 ones); ``forward(..., causal=, kv_lens=)`` take the implicit masks.
    """

    def __init__(self, embed_dim: int, num_heads: int, bias: bool = True, dropout: float = 0.0,
                 device: str = "cpu", attention_dtype: str = "float32"):
        if attention_dtype not in ("float32", "float16"):
            raise ValueError("attention_dtype must be 'float32' or 'float16'")
        self.attention_dtype = attention_dtype
        if embed_dim % num_heads != 0:
            raise ValueError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads})")
        self.embed_dim = embed_dim
        self.num_heads = num_heads
        self.head_dim = embed_dim // num_heads
        self.dropout = dropout
        self._parameters = {}
        std = math.sqrt(2.0 / (embed_dim + embed_dim))
        rng = np.random.default_rng()
        for name in ("q_weight", "k_weight", "v_weight", "out_weight"):
            w = (rng.standard_normal((embed_dim, embed_dim)) * std).astype(np.float32)
            self._parameters[name] = Tensor(w, device=device, requires_grad=True)
        for name in ("q_bias", "k_bias", "v_bias", "out_bias"):
            self._parameters[name] = (Tensor.zeros((embed_dim,), device=device, requires_grad=True)
                                      if bias else None)

    def parameters(self):
        return [p for p in self._parameters.values() if p is not None]

    def cuda(self) -> "MultiHeadAttention":
        for name, p in self._parameters.items():
            if p is not None:
                self._parameters[name] = p.cuda()
        return self

    def attend(self, q: Tensor, k: Tensor, v: Tensor, mask: Tensor = None, causal: bool = False,
               kv_lens=None) -> Tensor:
        """The SDPA step of forward (layers.py:122) on already projected and
        head-split tensors [batch, num_heads, seq, head_dim]."""
        if q.shape[1] != self.num_heads or q.shape[3] != self.head_dim:
            raise ValueError("attend: expected [batch, num_heads, seq, head_dim]")
        if causal or kv_lens is not None:
            return F.scaled_dot_product_attention_ex(q, k, v, mask, causal=causal, kv_lens=kv_lens)
        return F.scaled_dot_product_attention(q, k, v, mask)

    def forward(self, query: Tensor, key: Tensor, value: Tensor, mask: Tensor = None, causal: bool = False,
                kv_lens=None) -> Tensor:
        """query (batch, seq_q, embed_dim); key, value (batch, seq_k, embed_dim); mask optional
        (batch, num_heads, seq_q, seq_k).  Returns (batch, seq_q, embed_dim)."""
        from ... import _C
        P = self._parameters

        def project(x, w, b):
            return Tensor._wrap(_C.linear(x._c_tensor, P[w]._c_tensor,
                                          P[b]._c_tensor if P[b] is not None else None,
                                          heads_out=self.num_heads))

        q = project(query, "q_weight", "q_bias")          # (batch, heads, seq, head_dim), no transpose pass
        k = project(key, "k_weight", "k_bias")
        v = project(value, "v_weight", "v_bias")
        if self.attention_dtype == "float16":
            q, k, v = F.cast_to_fp16(q), F.cast_to_fp16(k), F.cast_to_fp16(v)
        attn = self.attend(q, k, v, mask, causal=causal, kv_lens=kv_lens)
        out = _C.linear(attn._c_tensor, P["out_weight"]._c_tensor,
                        P["out_bias"]._c_tensor if P["out_bias"] is not None else None,
                        heads_in=self.num_heads)         # heads merged while reading
        return Tensor._wrap(out)

    def __call__(self, query: Tensor, key: Tensor, value: Tensor, mask: Tensor = None, causal: bool = False,
                 kv_lens=None) -> Tensor:
        return self.forward(query, key, value, mask, causal=causal, kv_lens=kv_lens)

    def __repr__(self) -> str:
        return (f"MultiHeadAttention(embed_dim={self.embed_dim}, num_heads={self.num_heads}, "
                f"head_dim={self.head_dim}, dropout={self.dropout})")
